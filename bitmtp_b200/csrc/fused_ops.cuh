// Small fused operators of the decode step: activation absmax/INT8 quantisation,
// (residual add +) RMSNorm (+ quantisation), SiLU*up + quantisation, q/k head
// norm + RoPE + KV append, embedding gather, argmax / confidence reductions.
//
// Each kernel states the reference expression it replaces.  All of them round
// where the reference's eager tensor code rounds (bf16 in memory, fp32
// arithmetic) and reduce in the order fixed by oracle/bm_oracle.c, so results
// equal the oracle's bit for bit.
#pragma once

#include "bm_common.cuh"

namespace bm {

// Device-resident description of the replay in flight.  Written by
// bm_set_step_state (a one-thread kernel, so it can sit in front of a captured
// graph) and read by the attention kernels, so that a captured graph can be
// replayed for any cache length and pending count.
struct StepState {
    int cache_len;   // history rows [0, cache_len) are valid
    int n_pend;      // pending rows at the head of a draft replay
    int role;        // BM_ROLE_*
    int P;           // M - D
};

// ---- block-wide helpers -------------------------------------------------------
// Sum of per-warp values in ascending warp order, same result in every thread.
__device__ __forceinline__ float block_sum_ordered(float warp_val, float *sh, int lane, int warp,
                                                   int nwarps) {
    if (lane == 0) sh[warp] = warp_val;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < nwarps; ++w) t += sh[w];
    __syncthreads();
    return t;
}

__device__ __forceinline__ float block_max(float v, float *sh, int lane, int warp, int nwarps) {
    v = warp_max(v);
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float t = sh[0];
    for (int w = 1; w < nwarps; ++w) t = fmaxf(t, sh[w]);
    __syncthreads();
    return t;
}

__device__ __forceinline__ void unpack8(const uint4 &v, float (&f)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        w[i] = (uint32_t)bm_f32_to_bf16(f[2 * i]) | ((uint32_t)bm_f32_to_bf16(f[2 * i + 1]) << 16);
    return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ uint2 quant8(const float (&f)[8], float s) {
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        lo |= ((uint32_t)(bm_quant_i8(f[i], s) & 0xff)) << (8 * i);
        hi |= ((uint32_t)(bm_quant_i8(f[4 + i], s) & 0xff)) << (8 * i);
    }
    return make_uint2(lo, hi);
}

// Where the INT8 codes of a row go.  `nat` is the natural-order row the reference's
// operator API exposes; `prep` + `asum` are the GEMV-ready form: within every run of 16
// elements the bytes are transposed 4x4 (prep[4t+e] = nat[4e+t]), which is the order the
// GEMV kernels' fragments want, and asum[g] is the sum of the 128 codes of group g.  Any
// of the three may be null.
struct QuantSink {
    int8_t *nat;
    int8_t *prep;
    int32_t *asum;
};

// Stores the 8 codes of 8-element unit `unit` of a row.  Whole warps call this together
// (lanes whose unit lies past the row pass active = false): lane pairs (l, l^1) hold the
// two halves of a 16-element run and exchange them, 16 consecutive lanes hold one group.
__device__ __forceinline__ void emit_codes(const QuantSink &sink, size_t row_off, int K, int unit,
                                           uint2 codes, bool active, int lane) {
    if (sink.nat && active) reinterpret_cast<uint2 *>(sink.nat + row_off)[unit] = codes;
    if (sink.prep == nullptr) return;
    if (!active) codes = make_uint2(0u, 0u);
    const uint2 other = make_uint2(__shfl_xor_sync(0xffffffffu, codes.x, 1),
                                   __shfl_xor_sync(0xffffffffu, codes.y, 1));
    const bool odd = unit & 1;
    const uint2 lo = odd ? other : codes, hi = odd ? codes : other;
    const uint32_t sel = odd ? 0x7362u : 0x5140u;
    const uint32_t t = __byte_perm(lo.x, lo.y, sel), u = __byte_perm(hi.x, hi.y, sel);
    if (active)
        reinterpret_cast<uint2 *>(sink.prep + row_off)[unit] =
            make_uint2(__byte_perm(t, u, 0x5410), __byte_perm(t, u, 0x7632));
    int sum = __dp4a((int)codes.x, 0x01010101, 0);
    sum = __dp4a((int)codes.y, 0x01010101, sum);
#pragma unroll
    for (int off = 1; off < 16; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (active && (lane & 15) == 0) sink.asum[(row_off / K) * (K / BM_GROUP) + (unit >> 4)] = sum;
}

// =============================================================================
// quant_rows: per-row absmax INT8 quantisation of bf16 activations.
// Replaces T2LinearKernel.quant_input (src/bonsai_sft/gpu/model.py:632-636) and
// the inline copy in _lm_head (model.py:1247-1249).  One CTA per row.
// =============================================================================
constexpr int kRowThreads = 512;

__global__ void __launch_bounds__(kRowThreads) quant_rows_kernel(const uint16_t *__restrict__ x,
                                                                 int K, QuantSink sink,
                                                                 float *__restrict__ s_out,
                                                                 int pdl) {
    __shared__ float sh[kRowThreads / 32];
    pdl_launch_dependents();
    if (pdl) pdl_wait();
    const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint4 *xr = reinterpret_cast<const uint4 *>(x + (size_t)m * K);
    const int units = K / 8;
    float amax = 0.0f;
    for (int u = threadIdx.x; u < units; u += kRowThreads) {
        float f[8];
        unpack8(xr[u], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
    }
    amax = block_max(amax, sh, lane, warp, kRowThreads / 32);
    const float s = bm_act_scale(amax);
    for (int u0 = 0; u0 < units; u0 += kRowThreads) {
        const int u = u0 + threadIdx.x;
        const bool active = u < units;
        float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (active) unpack8(xr[u], f);
        emit_codes(sink, (size_t)m * K, K, u, quant8(f, s), active, lane);
    }
    if (threadIdx.x == 0) s_out[m] = s;
}

// =============================================================================
// quant_rows with the row absmax already known: the gate|up projection with the SiLU epilogue
// (t2_gemv.cuh) leaves bf16 `inner` rows and, by atomic max, the bits of each row's absmax; this kernel
// turns them into INT8 codes for the down projection.  Replaces the quant_input half of
// `inner = F.silu(g) * u; quant_input(inner)` (model.py:1059-1061).  Units of 8 elements are dealt to
// the threads of a flat grid, so the work spreads over many SMs instead of one CTA per row.
// `amax_zero` (optional): M words cleared for the next producer (a different array from amax_in).
// =============================================================================
constexpr int kQuantAmaxThreads = 256;

__global__ void __launch_bounds__(kQuantAmaxThreads) quant_rows_amax_kernel(
    const uint16_t *__restrict__ x, const unsigned int *__restrict__ amax_in, unsigned int *amax_zero, int M, int K,
    QuantSink sink, float *__restrict__ s_out, int pdl) {
    pdl_launch_dependents();
    if (pdl) pdl_wait();
    const int units = K / 8, lane = threadIdx.x & 31;
    const int u = blockIdx.x * kQuantAmaxThreads + threadIdx.x;   // whole warps stay inside one row (units % 32 == 0)
    const bool active = u < M * units;
    const int m = active ? u / units : 0, i = active ? u - m * units : 0;
    float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    float s = 0.0f;
    if (active) {
        unpack8(reinterpret_cast<const uint4 *>(x + (size_t)m * K)[i], v);
        s = bm_act_scale(__uint_as_float(amax_in[m]));
        if (i == 0) s_out[m] = s;
    }
    emit_codes(sink, (size_t)m * K, K, i, quant8(v, s), active, lane);
    if (amax_zero != nullptr && blockIdx.x == 0)
        for (int r = threadIdx.x; r < M; r += kQuantAmaxThreads) amax_zero[r] = 0u;
}

// =============================================================================
// (gather | residual add) + RMSNorm + (INT8 quantisation | bf16 store).
// Replaces _fused_norm_quant (model.py:307-319), _fused_add_norm_quant
// (model.py:322-336), RMSNorm.forward on the logit rows (model.py:290-295,
// 1401-1402) and the embedding gather in front of layer 0 (model.py:1386).
//   x        bf16 rows; with `gather` row m is x[gather[m]] (embedding table)
//   res      optional bf16 [M, dim]: h = bf16(x + res)
//   h_out    optional bf16 [M, dim]: the (gathered / summed) row before the norm
//   q, s     optional INT8 row + multiplier of the normed row
//   n_out    optional bf16 normed row
// One CTA per row, dim/8 threads (dim a multiple of 256): thread t owns
// elements 8t..8t+7, which is exactly the lane-partial of the oracle's
// sum-of-squares order; warps are its 256-element chunks.
// =============================================================================
// Row of a gathered table, kept inside the table whatever the id is (a corrupt id then reads a valid
// row instead of memory far outside the allocation).
__device__ __forceinline__ size_t gather_row(int64_t id, int rows) {
    return (size_t)(id < 0 ? 0 : (id >= rows ? rows - 1 : id));
}

struct NormParams {
    const uint16_t *x;
    const int64_t *gather;
    int gather_rows;   // rows of x when `gather` is given: indices are clamped to [0, gather_rows)
    const uint16_t *res;
    const uint16_t *w;
    uint16_t *h_out;
    QuantSink q;
    float *s;
    uint16_t *n_out;
    float eps;
    int dim;
    int row0;        // first row of x / res to read (logit rows start at logits_start)
    int pdl;
};

__global__ void __launch_bounds__(1024) rmsnorm_kernel(const NormParams p) {
    __shared__ float sh[32];
    pdl_launch_dependents();
    const int m = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int nwarps = blockDim.x >> 5;
    // the norm weights do not depend on the previous kernel: requested before the wait, used after the sum
    const uint4 wraw = reinterpret_cast<const uint4 *>(p.w)[t];
    if (p.pdl) pdl_wait();
    const size_t src_row = p.gather ? gather_row(p.gather[m], p.gather_rows) : (size_t)(p.row0 + m);
    float h[8];
    unpack8(reinterpret_cast<const uint4 *>(p.x + src_row * p.dim)[t], h);
    if (p.res) {
        float r[8];
        unpack8(reinterpret_cast<const uint4 *>(p.res + (size_t)(p.row0 + m) * p.dim)[t], r);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = bm_bf16_rn(h[i] + r[i]);
    }
    if (p.h_out) reinterpret_cast<uint4 *>(p.h_out + (size_t)m * p.dim)[t] = pack8(h);
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = fmaf(h[i], h[i], acc);
    const float total = block_sum_ordered(warp_sum_butterfly(acc), sh, lane, warp, nwarps);
    const float r = bm_rsqrtf(total / (float)p.dim + p.eps);
    float wv[8], n[8];
    unpack8(wraw, wv);
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        n[i] = bm_bf16_rn(wv[i] * bm_bf16_rn(h[i] * r));
        amax = fmaxf(amax, fabsf(n[i]));
    }
    if (p.n_out) reinterpret_cast<uint4 *>(p.n_out + (size_t)m * p.dim)[t] = pack8(n);
    if (p.s) {
        amax = block_max(amax, sh, lane, warp, nwarps);
        const float s = bm_act_scale(amax);
        emit_codes(p.q, (size_t)m * p.dim, p.dim, t, quant8(n, s), true, lane);
        if (t == 0) p.s[m] = s;
    }
}

// =============================================================================
// SiLU(gate) * up + INT8 quantisation of the down-projection input.
// Replaces `inner = F.silu(g) * u; quant_input(inner)` (model.py:1059-1061).
// gu bf16 [M, 2F] holds gate | up.  One CTA per row; the bf16 products wait in
// shared memory between the absmax pass and the quantisation pass.
// =============================================================================
__global__ void __launch_bounds__(kRowThreads) silu_mul_quant_kernel(
    const uint16_t *__restrict__ gu, int F, QuantSink sink, float *__restrict__ s_out,
    uint16_t *__restrict__ inner_out, int pdl) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ float sh[kRowThreads / 32];
    pdl_launch_dependents();
    if (pdl) pdl_wait();
    uint4 *inner = reinterpret_cast<uint4 *>(dyn);
    const int m = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint4 *g = reinterpret_cast<const uint4 *>(gu + (size_t)m * 2 * F);
    const uint4 *u = reinterpret_cast<const uint4 *>(gu + (size_t)m * 2 * F + F);
    const int units = F / 8;
    float amax = 0.0f;
    for (int i = threadIdx.x; i < units; i += kRowThreads) {
        float gf[8], uf[8], v[8];
        unpack8(g[i], gf);
        unpack8(u[i], uf);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            v[e] = bm_bf16_rn(bm_silu_bf16(gf[e]) * uf[e]);
            amax = fmaxf(amax, fabsf(v[e]));
        }
        const uint4 packed = pack8(v);
        inner[i] = packed;
        if (inner_out) reinterpret_cast<uint4 *>(inner_out + (size_t)m * F)[i] = packed;
    }
    amax = block_max(amax, sh, lane, warp, kRowThreads / 32);
    const float s = bm_act_scale(amax);
    for (int i0 = 0; i0 < units; i0 += kRowThreads) {
        const int i = i0 + threadIdx.x;
        const bool active = i < units;
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (active) unpack8(inner[i], v);
        emit_codes(sink, (size_t)m * F, F, i, quant8(v, s), active, lane);
    }
    if (threadIdx.x == 0) s_out[m] = s;
}

// =============================================================================
// Split qkv, per-head RMSNorm of q and k, RoPE, append K and V rows.
// Replaces _fused_qkv_qknorm_rope_kv_write (model.py:388-436).
//   xqkv bf16 [M, (H + 2*Hkv)*128]; cos/sin bf16 [max_pos, 128]; positions int64
//   k_base/v_base: one layer of the shared KV buffer, bf16 [Hkv, kv_rows, 128];
//   rows [sigma, sigma+M) are written.  q_out bf16 [M, H, 128].
// One warp per head vector: lane l owns elements 4l..4l+3 (the oracle's lane
// partial for a 128-wide row); the RoPE partner i +- 64 lives in lane l ^ 16.
// =============================================================================
struct RopeParams {
    const uint16_t *xqkv;
    const uint16_t *q_w, *k_w;
    const uint16_t *cos_t, *sin_t;
    const int64_t *positions;
    uint16_t *k_base, *v_base, *q_out;
    float eps;
    int M, H, Hkv, kv_rows, sigma, pdl;
};

__global__ void __launch_bounds__(128) qknorm_rope_kvappend_kernel(const RopeParams p) {
    pdl_launch_dependents();
    if (p.pdl) pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int heads = p.H + 2 * p.Hkv;
    const int m = blockIdx.y;
    const int hd = blockIdx.x * 4 + warp;
    if (hd >= heads) return;
    const uint16_t *src = p.xqkv + ((size_t)m * heads + hd) * 128 + 4 * lane;
    const uint2 raw = *reinterpret_cast<const uint2 *>(src);
    if (hd >= p.H + p.Hkv) {                          // V head: plain copy
        const int hk = hd - p.H - p.Hkv;
        *reinterpret_cast<uint2 *>(p.v_base + ((size_t)hk * p.kv_rows + p.sigma + m) * 128 + 4 * lane) = raw;
        return;
    }
    float x[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                  __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u)};
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc = fmaf(x[i], x[i], acc);
    const float total = warp_sum_butterfly(acc);      // one chunk: 0 + chunk sum
    const float r = bm_rsqrtf((0.0f + total) / 128.0f + p.eps);
    const uint16_t *wsrc = (hd < p.H ? p.q_w : p.k_w) + 4 * lane;
    const uint2 wraw = *reinterpret_cast<const uint2 *>(wsrc);
    const float w[4] = {__uint_as_float(wraw.x << 16), __uint_as_float(wraw.x & 0xffff0000u),
                        __uint_as_float(wraw.y << 16), __uint_as_float(wraw.y & 0xffff0000u)};
    const size_t pos = (size_t)p.positions[m];
    const uint2 craw = *reinterpret_cast<const uint2 *>(p.cos_t + pos * 128 + 4 * lane);
    const uint2 sraw = *reinterpret_cast<const uint2 *>(p.sin_t + pos * 128 + 4 * lane);
    const float c[4] = {__uint_as_float(craw.x << 16), __uint_as_float(craw.x & 0xffff0000u),
                        __uint_as_float(craw.y << 16), __uint_as_float(craw.y & 0xffff0000u)};
    const float sn[4] = {__uint_as_float(sraw.x << 16), __uint_as_float(sraw.x & 0xffff0000u),
                         __uint_as_float(sraw.y << 16), __uint_as_float(sraw.y & 0xffff0000u)};
    float n[4], o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) n[i] = bm_bf16_rn(w[i] * bm_bf16_rn(x[i] * r));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float partner = __shfl_xor_sync(0xffffffffu, n[i], 16);
        const float rot = lane < 16 ? -partner : partner;
        o[i] = bm_bf16_rn(n[i] * c[i]) + bm_bf16_rn(rot * sn[i]);
    }
    const uint2 packed = make_uint2(
        (uint32_t)bm_f32_to_bf16(o[0]) | ((uint32_t)bm_f32_to_bf16(o[1]) << 16),
        (uint32_t)bm_f32_to_bf16(o[2]) | ((uint32_t)bm_f32_to_bf16(o[3]) << 16));
    uint16_t *dst = hd < p.H
                        ? p.q_out + ((size_t)m * p.H + hd) * 128
                        : p.k_base + ((size_t)(hd - p.H) * p.kv_rows + p.sigma + m) * 128;
    *reinterpret_cast<uint2 *>(dst + 4 * lane) = packed;
}

// =============================================================================
// Step state and KV row promotion
// =============================================================================
__global__ void set_step_state_kernel(StepState *st, int cache_len, int n_pend, int role, int P) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        st->cache_len = cache_len;
        st->n_pend = n_pend;
        st->role = role;
        st->P = P;
    }
}

// Token ids, positions and the step record of one replay in ONE launch (the reference fills them with
// half a dozen tensor ops per step, fast_generate.py:1015-1037 draft, 1040-1055 verify, 247-256 AR).
//   kind 0  draft of width M = P + D:  tok = pending[0..n_pend) | 0.. | pending[n_pend-1] | MASK..,
//           pos = cache_len + i for the pending rows, 0 for the padding rows,
//           cache_len + n_pend - 1 + k for the D block rows
//   kind 1  verify of width M = D + 1: tok = pending[n_pend-1] | draft[0..D), pos = cache_len - 1 + i
//   kind 2  AR (M = 1): tok = src_a[0], pos = cache_len
//   kind 3  prompt slab of width M with n_pend real rows: tok = src_a[0..n_pend) | 0.., pos = cache_len + i | 0..
// `src_a` = pending tokens (prompt rows for kind 3), `src_b` = draft tokens (kind 1).  The record is what bm_set_step_state writes.
__global__ void stage_replay_inputs_kernel(int kind, const int64_t *__restrict__ src_a,
                                           const int64_t *__restrict__ src_b, int n_pend, int cache_len, int M, int D,
                                           int64_t mask_id, int role, int P, int state_n_pend,
                                           int64_t *__restrict__ tok, int64_t *__restrict__ pos, StepState *st) {
    const int i = threadIdx.x;
    if (i == 0) {
        st->cache_len = cache_len;
        st->n_pend = state_n_pend;
        st->role = role;
        st->P = P;
    }
    if (i >= M) return;
    if (kind == 0) {
        int64_t t, q;
        if (i > P) { t = mask_id; q = cache_len + n_pend - 1 + (i - P); }
        else if (i == P) { t = src_a[n_pend - 1]; q = cache_len + n_pend - 1; }
        else if (i < n_pend) { t = src_a[i]; q = cache_len + i; }
        else { t = 0; q = 0; }
        tok[i] = t;
        pos[i] = q;
    } else if (kind == 1) {
        tok[i] = i == 0 ? src_a[n_pend - 1] : src_b[i - 1];
        pos[i] = cache_len - 1 + i;
    } else if (kind == 2) {
        tok[i] = src_a[0];
        pos[i] = cache_len;
    } else {
        tok[i] = i < n_pend ? src_a[i] : 0;
        pos[i] = i < n_pend ? cache_len + i : 0;
    }
}

// The end of one decode step and the start of the next in one launch: the committed ids go to the output
// buffer and become the pending rows (all of them after a confidence commit, the last one = the verifier's
// token after a verified step: fast_generate.py:1121-1140), then the draft inputs are staged from them as
// stage_replay_inputs_kernel kind 0 does.  One warp; n_commit <= 32.  stage == 0: commit only.
__global__ void commit_stage_draft_kernel(const int64_t *__restrict__ src, int n_commit, int verified,
                                          int64_t *__restrict__ gen_dst, int64_t *__restrict__ pending, int stage,
                                          int cache_len, int M, int D, int64_t mask_id, int role, int P,
                                          int64_t *__restrict__ tok, int64_t *__restrict__ pos, StepState *st) {
    const int i = threadIdx.x;
    if (i < n_commit) {
        const int64_t t = src[i];
        gen_dst[i] = t;
        if (!verified) pending[i] = t;
        else if (i == n_commit - 1) pending[0] = t;
    }
    if (!stage) return;
    __syncwarp();
    const int n_pend = verified ? 1 : n_commit;
    if (i == 0) {
        st->cache_len = cache_len;
        st->n_pend = n_pend > P ? P : n_pend;
        st->role = role;
        st->P = P;
    }
    if (i >= M) return;
    int64_t t, q;
    if (i > P) { t = mask_id; q = cache_len + n_pend - 1 + (i - P); }
    else if (i == P) { t = pending[n_pend - 1]; q = cache_len + n_pend - 1; }
    else if (i < n_pend) { t = pending[i]; q = cache_len + i; }
    else { t = 0; q = 0; }
    tok[i] = t;
    pos[i] = q;
}

// Copies rows [src_row, src_row + n) to [dst_row, dst_row + n) in every
// (k|v, layer, kv head) plane of the shared buffer [planes, kv_rows, 128] bf16.
// Replaces GraphAtlas.commit_kv / commit_kv_from_verify
// (src/bonsai_sft/gpu/fast_runtime.py:467-508); the two ranges never overlap
// because the source rows sit at or beyond sigma and the destination below it.
__global__ void kv_copy_rows_kernel(uint16_t *kv, int planes, int kv_rows, int src_row, int dst_row,
                                    int n) {
    const int plane = blockIdx.x;
    if (plane >= planes) return;
    uint4 *base = reinterpret_cast<uint4 *>(kv + (size_t)plane * kv_rows * 128);
    for (int i = threadIdx.x; i < n * 16; i += blockDim.x)
        base[(size_t)dst_row * 16 + i] = base[(size_t)src_row * 16 + i];
}

// =============================================================================
// Freeze + pack: bf16 weights [N, K] -> the {-s, 0, +s} grid of each 128-group and its packed form.
// Replaces, on the device, freeze_quantize_to_ternary_g128 (src/bonsai_sft/ternary_modules.py:86-93)
// followed by _pack_t2_g128 (src/bonsai_sft/gpu/convert_bonsai_mtp_to_gpu.py:127-144), which the
// reference's converter runs tensor by tensor on the CPU:
//   s = max(absmax of the group, 1e-8) (fp32); q = clamp(round_half_even(w / s), -1, 1);
//   frozen = bf16(q * s); scale = bf16(absmax of frozen) (= bf16(s) unless the group is all zero);
//   code = q + 2, element j of a row in bits 2 (j % 4) of byte j / 4.
// Half a warp per (row, group): lane l owns elements 8l .. 8l+7, i.e. two packed bytes.
// =============================================================================
__global__ void __launch_bounds__(256) pack_t2_g128_kernel(const uint16_t *__restrict__ w, int N, int K,
                                                           uint8_t *__restrict__ packed, uint16_t *__restrict__ scale,
                                                           uint16_t *__restrict__ frozen) {
    // half a warp per (row, group): lane l of the half owns elements 8l .. 8l+7 (one 16-byte load, two packed bytes)
    const int lane = threadIdx.x & 31, sub = lane & 15, ng = K / BM_GROUP;
    const long long unit = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 2 + (lane >> 4);
    const bool live = unit < (long long)N * ng;            // K % 128 == 0: a row's groups never straddle rows
    const long long u = live ? unit : 0;
    const int n = (int)(u / ng), g = (int)(u - (long long)n * ng);
    const size_t base = (size_t)n * K + (size_t)g * BM_GROUP + 8 * sub;
    const uint4 raw = *reinterpret_cast<const uint4 *>(w + base);
    float x[8];
    unpack8(raw, x);
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(x[i]));
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const float s = fmaxf(amax, 1e-8f);
    float fr[8], famax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float r = rintf(x[i] / s);
        r = r < -1.0f ? -1.0f : (r > 1.0f ? 1.0f : r);
        fr[i] = bm_bf16_rn(r * s);
        famax = fmaxf(famax, fabsf(fr[i]));
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) famax = fmaxf(famax, __shfl_xor_sync(0xffffffffu, famax, off));
    const uint16_t sc = bm_f32_to_bf16(famax);
    // the packer rounds the frozen value against the bf16 scale once more (identity on the grid)
    const float sden = fmaxf(bm_bf16_to_f32(sc), 1e-30f);
    uint32_t two = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float r = rintf(fr[i] / sden);
        r = r < -1.0f ? -1.0f : (r > 1.0f ? 1.0f : r);
        two |= (uint32_t)((int)r + 2) << (2 * i);
    }
    if (!live) return;
    *reinterpret_cast<uint16_t *>(packed + (size_t)n * (K / 4) + (size_t)g * 32 + 2 * sub) = (uint16_t)two;
    if (sub == 0) scale[(size_t)n * ng + g] = sc;
    if (frozen != nullptr) *reinterpret_cast<uint4 *>(frozen + base) = pack8(fr);
}

// =============================================================================
// Logit reductions
// =============================================================================
// Row argmax with the lowest index winning ties.  logits fp32 [rows, ld].
// Replaces `.argmax(dim=-1)` on logits_out (fast_generate.py:786,809,1079) and
// the max of _fused_draft_chain (fast_generate.py:125).  One CTA per row.
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float *__restrict__ logits,
                                                           int vocab, int ld,
                                                           int64_t *__restrict__ idx,
                                                           float *__restrict__ max_out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float *x = logits + (size_t)r * ld;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int v = threadIdx.x; v < vocab; v += blockDim.x) {
        const float f = x[v];
        if (bm_argmax_better(f, v, best, bi)) { best = f; bi = v; }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (bm_argmax_better(ob, oi, best, bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (bm_argmax_better(sv[w], si[w], best, bi)) { best = sv[w]; bi = si[w]; }
        idx[r] = bi;
        if (max_out) max_out[r] = best;
    }
}

// Sum of exp(x - max) per row in the oracle's chunk order (256-element chunks:
// 32 lanes x 8 consecutive terms, butterfly, chunks added in ascending order),
// then conf = exp(max - (max + log(sum))).  One CTA of 8 warps per row: warp w
// takes chunks w, w+8, ... and keeps their sums in shared memory; thread 0 adds
// them in order.  Part of _fused_draft_chain (fast_generate.py:126-127).
constexpr int kConfMaxChunks = 1024;   // vocab <= 262144

__global__ void __launch_bounds__(256) row_confidence_kernel(const float *__restrict__ logits,
                                                             int vocab, int ld,
                                                             const float *__restrict__ row_max,
                                                             float *__restrict__ conf) {
    __shared__ float chunk_sum[kConfMaxChunks];
    const int r = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float *x = logits + (size_t)r * ld;
    const float mx = row_max[r];
    const int nchunks = (vocab + 255) / 256;
    for (int c = warp; c < nchunks; c += 8) {
        float acc = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const int v = c * 256 + lane * 8 + e;
            if (v < vocab) acc += bm_expf(x[v] - mx);
        }
        acc = warp_sum_butterfly(acc);
        if (lane == 0) chunk_sum[c] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int c = 0; c < nchunks; ++c) total += chunk_sum[c];
        const float lse = mx + bm_logf(total);
        conf[r] = bm_expf(mx - lse);
    }
}

// iter_accept = 1 + longest prefix of rows r >= 1 with conf[r] > tau
// (fast_generate.py:128-129); accept = longest prefix with draft == verify
// (fast_generate.py:146).  Single-thread kernels over <= 32 values.
__global__ void chain_length_kernel(const float *conf, int D, float tau, int *out) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int n = 1;
    for (int r = 1; r < D; ++r) {
        if (conf[r] > tau) ++n; else break;
    }
    *out = n;
}

// ---- the same reductions spread over many CTAs ------------------------------------------------
// One CTA per logit row leaves 140 of 148 SMs idle on rows of 151936 values (measured: 129 us for the
// confidence chain of 8 rows, 37 us for an argmax).  Here a row is cut into S ranges of whole 256-element
// chunks, one CTA each (S = logit_splits(rows): more ranges when there are few rows); the last CTA of a row to finish (a
// ticket counter in the caller's scratch) combines the row, and for the confidence chain the last row
// to finish computes the chain length.  Results are identical to the one-CTA kernels: the argmax
// comparison does not depend on order, the chunk sums are the same chunk sums and are added in ascending
// chunk order by one thread.  Scratch (LogitScratch, zero before first use; the kernels leave the
// counters zero again).
constexpr int kLogitMaxRows = 32;
constexpr int kLogitMaxParts = 512;      // rows * S

__host__ __device__ inline int logit_splits(int rows) {
    int s = kLogitMaxParts / rows;       // 16 at 32 rows
    return s > 128 ? 128 : (s > 32 && rows > 2 ? 32 : s);
}

struct LogitScratch {
    unsigned int arg_tickets[kLogitMaxRows];
    unsigned int conf_tickets[kLogitMaxRows];
    unsigned int rows_done;
    unsigned int pad[63];
    float part_max[kLogitMaxParts];
    int part_idx[kLogitMaxParts];
    float chunk_sum[kLogitMaxRows * kConfMaxChunks];
};

__device__ __forceinline__ void logit_split_range(int vocab, int split, int S, int &v_lo, int &v_hi) {
    const int nchunks = (vocab + 255) / 256;
    const int per = (nchunks + S - 1) / S;
    v_lo = min(vocab, split * per * 256);
    v_hi = min(vocab, (split + 1) * per * 256);
}

// grid (S, rows), 256 threads
__global__ void __launch_bounds__(256) argmax_split_kernel(const float *__restrict__ logits, int vocab, int ld,
                                                          int64_t *__restrict__ idx, float *__restrict__ max_out,
                                                          LogitScratch *sc) {
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ unsigned int ticket;
    const int split = blockIdx.x, S = gridDim.x, r = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float *x = logits + (size_t)r * ld;
    int v_lo, v_hi;
    logit_split_range(vocab, split, S, v_lo, v_hi);
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int v = v_lo + threadIdx.x; v < v_hi; v += 256) {
        const float f = x[v];
        if (bm_argmax_better(f, v, best, bi)) { best = f; bi = v; }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (bm_argmax_better(ob, oi, best, bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (bm_argmax_better(sv[w], si[w], best, bi)) { best = sv[w]; bi = si[w]; }
        sc->part_max[r * S + split] = best;
        sc->part_idx[r * S + split] = bi;
        __threadfence();
        ticket = atomicAdd(&sc->arg_tickets[r], 1u);
    }
    __syncthreads();
    if (ticket != (unsigned int)(S - 1) || threadIdx.x != 0) return;
    // last CTA of the row: every partial is visible
    __threadfence();
    best = -INFINITY;
    bi = 0x7fffffff;
    for (int s = 0; s < S; ++s) {
        const float f = __ldcg(&sc->part_max[r * S + s]);
        const int i = __ldcg(&sc->part_idx[r * S + s]);
        if (bm_argmax_better(f, i, best, bi)) { best = f; bi = i; }
    }
    idx[r] = bi;
    if (max_out) max_out[r] = best;
    sc->arg_tickets[r] = 0u;
}

// grid (S, D), 256 threads.  row_max[r] must be final (argmax_split_kernel of the same rows has
// completed: stream order).  The last row to finish writes the chain length.
__global__ void __launch_bounds__(256) confidence_split_kernel(const float *__restrict__ logits, int vocab, int ld,
                                                              const float *__restrict__ row_max,
                                                              float *__restrict__ conf, int D, float tau,
                                                              int *__restrict__ n_out, LogitScratch *sc) {
    __shared__ unsigned int ticket;
    const int split = blockIdx.x, S = gridDim.x, r = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float *x = logits + (size_t)r * ld;
    const float mx = row_max[r];
    const int nchunks = (vocab + 255) / 256;
    const int per = (nchunks + S - 1) / S;
    const int c_lo = min(nchunks, split * per), c_hi = min(nchunks, (split + 1) * per);
    float *sums = sc->chunk_sum + (size_t)r * kConfMaxChunks;
    const bool vec = (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
    for (int c = c_lo + warp; c < c_hi; c += 8) {
        const int v0 = c * 256 + lane * 8;
        float acc = 0.0f;
        if (vec && v0 + 8 <= vocab) {
            const float4 a = *reinterpret_cast<const float4 *>(x + v0), b = *reinterpret_cast<const float4 *>(x + v0 + 4);
            acc += bm_expf(a.x - mx); acc += bm_expf(a.y - mx); acc += bm_expf(a.z - mx); acc += bm_expf(a.w - mx);
            acc += bm_expf(b.x - mx); acc += bm_expf(b.y - mx); acc += bm_expf(b.z - mx); acc += bm_expf(b.w - mx);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e)
                if (v0 + e < vocab) acc += bm_expf(x[v0 + e] - mx);
        }
        acc = warp_sum_butterfly(acc);
        if (lane == 0) sums[c] = acc;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        ticket = atomicAdd(&sc->conf_tickets[r], 1u);
    }
    __syncthreads();
    if (ticket != (unsigned int)(S - 1)) return;
    // last CTA of the row: add the chunk sums in ascending order.  All threads fetch them into shared memory
    // first (one round trip instead of one per addend); thread 0 then adds them in the same order as before.
    __threadfence();
    __shared__ float staged[kConfMaxChunks];
    for (int c = threadIdx.x; c < nchunks; c += blockDim.x) staged[c] = __ldcg(&sums[c]);
    __syncthreads();
    if (threadIdx.x != 0) return;
    float total = 0.0f;
    for (int c = 0; c < nchunks; ++c) total += staged[c];
    const float lse = mx + bm_logf(total);
    conf[r] = bm_expf(mx - lse);
    sc->conf_tickets[r] = 0u;
    __threadfence();
    if (atomicAdd(&sc->rows_done, 1u) != (unsigned int)(D - 1)) return;
    // last row: the chain length over all confidences
    __threadfence();
    int n = 1;
    for (int q = 1; q < D; ++q) {
        if (__ldcg(&conf[q]) > tau) ++n; else break;
    }
    *n_out = n;
    sc->rows_done = 0u;
}

// ---- the confidence chain of a draft block in ONE launch -----------------------------------------
// argmax_split_kernel + confidence_split_kernel as one kernel: the kDraftClusterCtas CTAs of a logit row are a
// thread-block cluster (grid (kDraftClusterCtas, D), cluster (kDraftClusterCtas, 1, 1)).  Each CTA reads its
// range of whole 256-element chunks ONCE, into shared memory, and finds its maximum; the partial maxima go to
// every CTA of the cluster through distributed shared memory, so after one cluster barrier each CTA knows the
// row's maximum and argmax (same comparison, ranges in ascending order) and sums exp(x - max) over its chunks
// from shared memory in the oracle's order (lane = 8 consecutive terms, butterfly); the chunk sums go to the
// first CTA of the cluster, which after a second barrier adds them in ascending order and finishes the row as
// confidence_split_kernel does (the last row to finish writes the chain length).  Same results, one launch
// instead of two, the logits read once instead of twice, no fence / ticket / read-back inside a row.
constexpr int kDraftClusterCtas = 16;

__global__ void __launch_bounds__(256) draft_chain_cluster_kernel(const float *__restrict__ logits, int vocab, int ld,
                                                                 int64_t *__restrict__ idx, float *__restrict__ max_out,
                                                                 float *__restrict__ conf, int D, float tau,
                                                                 int *__restrict__ n_out, LogitScratch *sc) {
    extern __shared__ __align__(16) float slice[];            // this CTA's chunks of the row
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ float part_max[kDraftClusterCtas];
    __shared__ int part_idx[kDraftClusterCtas];
    __shared__ float sums[kConfMaxChunks];                    // chunk sums of the whole row (used in CTA 0)
    __shared__ float row_best;
    __shared__ int row_idx;
    const int rank = blockIdx.x, r = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    cluster_arrive();                      // waited for below, before the first store into another CTA: all have started
    const float *x = logits + (size_t)r * ld;
    const int nchunks = (vocab + 255) / 256;
    const int per = (nchunks + kDraftClusterCtas - 1) / kDraftClusterCtas;
    const int c_lo = min(nchunks, rank * per), c_hi = min(nchunks, (rank + 1) * per);
    const int v_lo = min(vocab, c_lo * 256), v_hi = min(vocab, c_hi * 256);
    // the whole range is requested at once (16-byte asynchronous copies where the row is aligned for them, so
    // that a thread has all its loads in flight together), then scanned from shared memory
    const int len = v_hi - v_lo;
    const bool vec = (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0;
    const int len4 = vec ? len / 4 : 0;
    for (int i = threadIdx.x; i < len4; i += 256) cp_async16(slice + 4 * i, x + v_lo + 4 * i);
    for (int i = 4 * len4 + threadIdx.x; i < len; i += 256) slice[i] = x[v_lo + i];
    cp_async_wait_all();
    __syncthreads();
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < len; i += 256) {
        const float f = slice[i];
        if (bm_argmax_better(f, v_lo + i, best, bi)) { best = f; bi = v_lo + i; }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, off);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
        if (bm_argmax_better(ob, oi, best, bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) { sv[warp] = best; si[warp] = bi; }
    __syncthreads();
    cluster_wait();
    if (warp == 0) {
        // lane t hands this CTA's partial to CTA t of the cluster
        best = sv[0]; bi = si[0];
        for (int w = 1; w < 8; ++w)
            if (bm_argmax_better(sv[w], si[w], best, bi)) { best = sv[w]; bi = si[w]; }
        if (lane < kDraftClusterCtas) {
            cluster_st_f32(cluster_map(&part_max[rank], (uint32_t)lane), best);
            cluster_st_s32(cluster_map(&part_idx[rank], (uint32_t)lane), bi);
        }
    }
    cluster_arrive();
    cluster_wait();
    if (threadIdx.x == 0) {
        best = -INFINITY;
        bi = 0x7fffffff;
        for (int s = 0; s < kDraftClusterCtas; ++s)
            if (bm_argmax_better(part_max[s], part_idx[s], best, bi)) { best = part_max[s]; bi = part_idx[s]; }
        row_best = best;
        row_idx = bi;
    }
    __syncthreads();
    const float mx = row_best;
    for (int c = c_lo + warp; c < c_hi; c += 8) {
        const int v0 = c * 256 + lane * 8;
        float acc = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e)
            if (v0 + e < vocab) acc += bm_expf(slice[v0 + e - v_lo] - mx);
        acc = warp_sum_butterfly(acc);
        if (lane == 0) cluster_st_f32(cluster_map(&sums[c], 0u), acc);
    }
    cluster_arrive();
    cluster_wait();
    if (rank != 0 || threadIdx.x != 0) return;
    float total = 0.0f;
    for (int c = 0; c < nchunks; ++c) total += sums[c];
    const float lse = mx + bm_logf(total);
    conf[r] = bm_expf(mx - lse);
    idx[r] = row_idx;
    max_out[r] = mx;
    __threadfence();
    if (atomicAdd(&sc->rows_done, 1u) != (unsigned int)(D - 1)) return;
    // last row: the chain length over all confidences
    __threadfence();
    int n = 1;
    for (int q = 1; q < D; ++q) {
        if (__ldcg(&conf[q]) > tau) ++n; else break;
    }
    *n_out = n;
    sc->rows_done = 0u;
}

__global__ void verify_accept_kernel(const int64_t *draft, const int64_t *verify, int D, int *out) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int n = 0;
    while (n < D && draft[n] == verify[n]) ++n;
    *out = n;
}

}  // namespace bm
