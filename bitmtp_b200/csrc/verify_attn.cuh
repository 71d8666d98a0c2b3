// Block-verify attention over the shared KV buffer, fused with the INT8
// quantisation of the o-projection input.
//
// Replaces, for one layer of one replay, the attention of
// Attention.forward_sdlm_graph_kernel (src/bonsai_sft/gpu/model.py:989-1005:
// flex_attention closure or matmul/softmax/matmul, the permute back to
// [M, q_dim] and o_proj.quant_input) together with the additive mask tensor the
// host rebuilds before every replay (src/bonsai_sft/gpu/fast_runtime.py:345-372,
// 391-465).  Differences in kind, not in result:
//   * visibility is evaluated from (role, cache_len, n_pend) held in device
//     memory (bm_visible in bm_math.h), so nothing is rebuilt on the host and a
//     captured graph serves every cache length;
//   * only history rows [0, cache_len) and the M rows of this replay are read,
//     not the whole padded buffer of sigma + M rows;
//   * the work is split over (kv head, 32-key chunk) CTAs and merged by a
//     second kernel (split-KV), whose last CTA per row quantises the row.
//
// Arithmetic and order: see bmo_attention in oracle/bm_oracle.c; the two agree
// bit for bit.  All accumulation is fp32 on the CUDA cores in a fixed order;
// tensor-core accumulation order is not specified by the hardware documents and
// could not be mirrored on the CPU.
//
// Scratch (caller-allocated, bm_verify_attention_scratch_bytes):
//   ctr  int32 [32]            per-row arrival counters, must be zero on entry; the
//                              kernel leaves them zero
//   amax uint32 [32]           per-row absmax bits, same rule
//   pm, pl fp32 [M, H, NC]     chunk max / chunk sum
//   po   fp32 [M, H, NC, 128]  chunk numerators
//   NC = ceil(sigma/32) + 1; chunk NC-1 holds the rows appended by this replay.
#pragma once

#include "bm_common.cuh"
#include "fused_ops.cuh"

namespace bm {

constexpr int kAttnThreads = 256;
constexpr int kKeyStride = 136;   // bf16 elements per staged key row (128 + 8 pad = 272 bytes)

struct AttnParams {
    const uint16_t *q;        // [M, H, 128]
    const uint16_t *k_base;   // [Hkv, kv_rows, 128]
    const uint16_t *v_base;
    const StepState *state;
    int M, H, Hkv, kv_rows, sigma, NC;
    int *ctr;
    unsigned int *amax;
    float *pm, *pl, *po;
    uint16_t *att;            // [M, H*128] bf16 attention output
    QuantSink q_out;          // [M, H*128] INT8 of att (natural and/or GEMV-ready)
    float *s_out;             // [M]
    int pdl;
};

__host__ __device__ inline size_t attn_scratch_bytes(int M, int H, int sigma) {
    const size_t NC = (size_t)(sigma + BM_ATTN_CHUNK - 1) / BM_ATTN_CHUNK + 1;
    return 256 + (size_t)M * H * NC * 4 * 2 + (size_t)M * H * NC * 128 * 4;
}

// ---- kernel 1: one (chunk, kv head) ------------------------------------------------
__global__ void __launch_bounds__(kAttnThreads, 1) attn_chunk_kernel(const AttnParams p) {
    extern __shared__ __align__(16) unsigned char dyn[];
    pdl_launch_dependents();
    if (p.pdl) pdl_wait();
    const int j = blockIdx.x, hk = blockIdx.y;
    const int cache_len = p.state->cache_len, n_pend = p.state->n_pend, role = p.state->role,
              P = p.state->P;
    const int n_hist = (cache_len + BM_ATTN_CHUNK - 1) / BM_ATTN_CHUNK;
    int c0, cn;
    if (j == p.NC - 1) { c0 = p.sigma; cn = p.M; }
    else if (j < n_hist) { c0 = j * BM_ATTN_CHUNK; cn = min(BM_ATTN_CHUNK, cache_len - c0); }
    else return;

    const int G = p.H / p.Hkv, QV = G * p.M;
    uint16_t *Ks = reinterpret_cast<uint16_t *>(dyn);                    // [32][136]
    uint16_t *Vs = Ks + 32 * kKeyStride;                                  // [32][128]
    float *Qs = reinterpret_cast<float *>(Vs + 32 * 128);                 // [QV][128]
    float *Ss = Qs + (size_t)QV * 128;                                    // [QV][32]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    const uint16_t *kg = p.k_base + ((size_t)hk * p.kv_rows + c0) * 128;
    const uint16_t *vg = p.v_base + ((size_t)hk * p.kv_rows + c0) * 128;
    for (int i = tid; i < cn * 16; i += kAttnThreads) {
        const int c = i >> 4, u = i & 15;
        *reinterpret_cast<uint4 *>(Ks + c * kKeyStride + 8 * u) =
            reinterpret_cast<const uint4 *>(kg)[i];
        reinterpret_cast<uint4 *>(Vs)[i] = reinterpret_cast<const uint4 *>(vg)[i];
    }
    for (int i = tid; i < QV * 16; i += kAttnThreads) {
        const int qv = i >> 4, u = i & 15;
        const int g = qv / p.M, m = qv - g * p.M;
        float f[8];
        unpack8(reinterpret_cast<const uint4 *>(p.q + ((size_t)m * p.H + hk * G + g) * 128)[u], f);
        float4 *dst = reinterpret_cast<float4 *>(Qs + (size_t)qv * 128 + 8 * u);
        dst[0] = make_float4(f[0], f[1], f[2], f[3]);
        dst[1] = make_float4(f[4], f[5], f[6], f[7]);
    }
    __syncthreads();

    // Scores: lane = key, the key row in registers, query vectors broadcast.
    {
        float kf[128];
        if (lane < cn) {
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                float f[8];
                unpack8(*reinterpret_cast<const uint4 *>(Ks + lane * kKeyStride + 8 * u), f);
#pragma unroll
                for (int e = 0; e < 8; ++e) kf[8 * u + e] = f[e];
            }
        } else {
#pragma unroll
            for (int d = 0; d < 128; ++d) kf[d] = 0.0f;
        }
        for (int qv = warp; qv < QV; qv += kAttnThreads / 32) {
            const float4 *qp = reinterpret_cast<const float4 *>(Qs + (size_t)qv * 128);
            float acc = 0.0f;
#pragma unroll
            for (int u = 0; u < 32; ++u) {
                const float4 qq = qp[u];
                acc = fmaf(qq.x, kf[4 * u], acc);
                acc = fmaf(qq.y, kf[4 * u + 1], acc);
                acc = fmaf(qq.z, kf[4 * u + 2], acc);
                acc = fmaf(qq.w, kf[4 * u + 3], acc);
            }
            const int m = qv % p.M;
            const bool vis = lane < cn && bm_visible(role, m, c0 + lane, p.sigma, cache_len, n_pend, P);
            const float sc = vis ? acc * 0.08838834764831845f : -INFINITY;
            const float mj = warp_max(sc);
            const float pr = vis ? bm_expf(sc - mj) : 0.0f;
            const float lj = warp_sum_butterfly(pr);
            Ss[qv * 32 + lane] = bm_bf16_rn(pr);
            if (lane == 0) {
                const int g = qv / p.M;
                const size_t o = ((size_t)m * p.H + hk * G + g) * p.NC + j;
                p.pm[o] = mj;
                p.pl[o] = lj;
            }
        }
    }
    __syncthreads();

    // Numerators: thread = (d, half of the query vectors), the V column in registers.
    {
        const int d = tid & 127, half = tid >> 7;
        float vf[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) vf[c] = c < cn ? bf16_bits_to_f32(Vs[c * 128 + d]) : 0.0f;
        for (int qv = half; qv < QV; qv += 2) {
            const float4 *pp = reinterpret_cast<const float4 *>(Ss + qv * 32);
            float acc = 0.0f;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float4 w = pp[u];
                // Positions >= cn hold weight 0 and value 0: fma(0, 0, acc) == acc.
                acc = fmaf(w.x, vf[4 * u], acc);
                acc = fmaf(w.y, vf[4 * u + 1], acc);
                acc = fmaf(w.z, vf[4 * u + 2], acc);
                acc = fmaf(w.w, vf[4 * u + 3], acc);
            }
            const int g = qv / p.M, m = qv - g * p.M;
            p.po[(((size_t)m * p.H + hk * G + g) * p.NC + j) * 128 + d] = acc;
        }
    }
}

// ---- kernel 2: merge chunks for (row m, head pair); last CTA of a row quantises it --
__global__ void __launch_bounds__(kAttnThreads) attn_merge_kernel(const AttnParams p) {
    __shared__ float w_s[2][160];        // merge weights per head of the pair (NC <= 160 => sigma <= 5088)
    __shared__ float pl_s[2][160];
    __shared__ float l_s[2];
    __shared__ float red[kAttnThreads / 32];
    __shared__ int is_last;
    pdl_launch_dependents();
    if (p.pdl) pdl_wait();
    const int m = blockIdx.y, h0 = blockIdx.x * 2;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cache_len = p.state->cache_len;
    const int n_hist = (cache_len + BM_ATTN_CHUNK - 1) / BM_ATTN_CHUNK;
    const int nv = n_hist + 1;                        // valid chunks: history, then NC-1

    if (warp < 2) {                                   // warp w: weights of head h0 + w
        const size_t base = ((size_t)m * p.H + h0 + warp) * p.NC;
        // chunk maxima and sums come into shared memory with independent loads; the ordered
        // sum below then runs on shared-memory operands
        float gmax = -INFINITY;
        for (int i = lane; i < nv; i += 32) {
            const int j = i < n_hist ? i : p.NC - 1;
            const float mj = p.pm[base + j];
            w_s[warp][i] = mj;
            pl_s[warp][i] = p.pl[base + j];
            gmax = fmaxf(gmax, mj);
        }
        gmax = warp_max(gmax);
        for (int i = lane; i < nv; i += 32) {
            const float mj = w_s[warp][i];
            w_s[warp][i] = mj > -INFINITY ? bm_expf(mj - gmax) : 0.0f;
        }
        __syncwarp();
        if (lane == 0) {
            float l = 0.0f;
            // a chunk without a visible key has weight 0 and sum 0: fma(0, 0, l) == l
            for (int i = 0; i < nv; ++i) l = fmaf(pl_s[warp][i], w_s[warp][i], l);
            l_s[warp] = l;
        }
    }
    __syncthreads();
    const int hh = tid >> 7, d = tid & 127, h = h0 + hh;
    const size_t obase = ((size_t)m * p.H + h) * p.NC;
    float o = 0.0f;
#pragma unroll 4
    for (int i = 0; i < nv; ++i) {
        const int j = i < n_hist ? i : p.NC - 1;
        const float w = w_s[hh][i];
        // A chunk without a visible key has weight 0 and a zero numerator; skipping it
        // and adding 0 * 0 are the same value, so no branch is needed.
        o = fmaf(p.po[(obase + j) * 128 + d], w, o);
    }
    const float val = bm_bf16_rn(o / l_s[hh]);
    const size_t row = (size_t)m * p.H * 128;
    p.att[row + h * 128 + d] = bm_f32_to_bf16(val);
    __threadfence();                                  // publish before this CTA is counted
    const float a = block_max(fabsf(val), red, lane, warp, kAttnThreads / 32);
    if (tid == 0) {
        atomicMax(&p.amax[m], __float_as_uint(a));
        __threadfence();
        const int arrived = atomicAdd(&p.ctr[m], 1);
        is_last = (arrived == (int)gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    const float amax = __uint_as_float(atomicOr(&p.amax[m], 0u));
    const float s = bm_act_scale(amax);
    const int units = p.H * 128 / 8;
    for (int u0 = 0; u0 < units; u0 += kAttnThreads) {
        const int u = u0 + tid;
        const bool active = u < units;
        float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (active) unpack8(__ldcg(reinterpret_cast<const uint4 *>(p.att + row) + u), f);
        emit_codes(p.q_out, row, p.H * 128, u, quant8(f, s), active, lane);
    }
    if (tid == 0) {
        p.s_out[m] = s;
        p.amax[m] = 0u;
        p.ctr[m] = 0;
    }
}

}  // namespace bm
