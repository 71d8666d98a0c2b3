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
//     second kernel (split-KV) with one CTA per query row, which also quantises
//     the row.
//
// Arithmetic and order: see bmo_attention in oracle/bm_oracle.c; the two agree
// bit for bit.  All accumulation is fp32 on the CUDA cores in a fixed order;
// tensor-core accumulation order is not specified by the hardware documents and
// could not be mirrored on the CPU.
//
// Scratch (caller-allocated, bm_verify_attention_scratch_bytes):
//   256 reserved bytes        (unused; kept zero)
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

// History length of this replay.  The record is written by other launches (or by the caller through
// the C ABI), so it is clamped to [0, sigma] before anything is indexed with it: the scratch, the
// shared-memory arrays and the K/V planes are all sized from sigma.  Identity for every valid record.
__device__ __forceinline__ int attn_cache_len(const AttnParams &p) {
    return min(max(p.state->cache_len, 0), p.sigma);
}

// ---- kernel 1: one (chunk, kv head); a warp serves NQ query vectors at a time --------
// lane = key in the score phase (NQ independent fma chains, one per query vector, each in
// ascending d), lane = 4 output dims in the numerator phase (4*NQ independent chains, each
// in ascending key order).  Shared memory: the chunk's K rows (padded), V rows, the query
// vectors of this kv head as fp32, and the bf16-rounded softmax weights.
constexpr int kAttnMinThreads = 128;           // staging uses at least 4 warps

__host__ __device__ inline int attn_nq(int QV) {
    return QV <= 16 ? 2 : (QV <= 32 ? 4 : 8);  // keeps ceil(QV/NQ) <= 8 warps up to QV = 64
}

template <int NQ>
__device__ __forceinline__ void attn_chunk_pass(const AttnParams &p, const uint16_t *Ks, const uint16_t *Vs,
                                                const float *Qs, float *Ps, int q0, int QV, int G,
                                                int hk, int j, int c0, int cn, int lane, int role,
                                                int cache_len, int n_pend, int P) {
    // rows past QV repeat the last query vector; their results are dropped
    const float *qrow[NQ];
#pragma unroll
    for (int t = 0; t < NQ; ++t) qrow[t] = Qs + (size_t)min(q0 + t, QV - 1) * 128;
    float acc[NQ];
#pragma unroll
    for (int t = 0; t < NQ; ++t) acc[t] = 0.0f;
    const uint16_t *krow = Ks + (lane < cn ? lane : 0) * kKeyStride;
#pragma unroll 4
    for (int u = 0; u < 16; ++u) {
        float kf[8];
        unpack8(*reinterpret_cast<const uint4 *>(krow + 8 * u), kf);
#pragma unroll
        for (int t = 0; t < NQ; ++t) {
            const float4 qa = *reinterpret_cast<const float4 *>(qrow[t] + 8 * u);
            const float4 qb = *reinterpret_cast<const float4 *>(qrow[t] + 8 * u + 4);
            acc[t] = fmaf(qa.x, kf[0], acc[t]);
            acc[t] = fmaf(qa.y, kf[1], acc[t]);
            acc[t] = fmaf(qa.z, kf[2], acc[t]);
            acc[t] = fmaf(qa.w, kf[3], acc[t]);
            acc[t] = fmaf(qb.x, kf[4], acc[t]);
            acc[t] = fmaf(qb.y, kf[5], acc[t]);
            acc[t] = fmaf(qb.z, kf[6], acc[t]);
            acc[t] = fmaf(qb.w, kf[7], acc[t]);
        }
    }
#pragma unroll
    for (int t = 0; t < NQ; ++t) {
        const int qv = q0 + t;
        if (qv >= QV) break;                           // warp-uniform
        const int g = qv / p.M, m = qv - g * p.M;
        const bool vis = lane < cn && bm_visible(role, m, c0 + lane, p.sigma, cache_len, n_pend, P);
        const float sc = vis ? acc[t] * 0.08838834764831845f : -INFINITY;
        const float mj = warp_max(sc);
        const float pr = vis ? bm_expf(sc - mj) : 0.0f;
        const float lj = warp_sum_butterfly(pr);
        Ps[qv * 32 + lane] = bm_bf16_rn(pr);
        if (lane == 0) {
            const size_t o = ((size_t)m * p.H + hk * G + g) * p.NC + j;
            p.pm[o] = mj;
            p.pl[o] = lj;
        }
    }
    __syncwarp();
    // numerators: lane owns dims 4*lane .. 4*lane+3 of the NQ query vectors
    const float *prow[NQ];
#pragma unroll
    for (int t = 0; t < NQ; ++t) prow[t] = Ps + min(q0 + t, QV - 1) * 32;
    float o[NQ][4];
#pragma unroll
    for (int t = 0; t < NQ; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[t][e] = 0.0f;
    for (int cb = 0; cb < cn; cb += 4) {
        float v[4][4];
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            // keys past cn have weight 0 and are given value 0
            const uint2 raw = (cb + cc < cn)
                                  ? *reinterpret_cast<const uint2 *>(Vs + (cb + cc) * 128 + 4 * lane)
                                  : make_uint2(0u, 0u);
            v[cc][0] = __uint_as_float(raw.x << 16);
            v[cc][1] = __uint_as_float(raw.x & 0xffff0000u);
            v[cc][2] = __uint_as_float(raw.y << 16);
            v[cc][3] = __uint_as_float(raw.y & 0xffff0000u);
        }
#pragma unroll
        for (int t = 0; t < NQ; ++t) {
            const float4 w = *reinterpret_cast<const float4 *>(prow[t] + cb);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                o[t][e] = fmaf(w.x, v[0][e], o[t][e]);
                o[t][e] = fmaf(w.y, v[1][e], o[t][e]);
                o[t][e] = fmaf(w.z, v[2][e], o[t][e]);
                o[t][e] = fmaf(w.w, v[3][e], o[t][e]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < NQ; ++t) {
        const int qv = q0 + t;
        if (qv >= QV) break;
        const int g = qv / p.M, m = qv - g * p.M;
        *reinterpret_cast<float4 *>(p.po + (((size_t)m * p.H + hk * G + g) * p.NC + j) * 128 + 4 * lane) =
            make_float4(o[t][0], o[t][1], o[t][2], o[t][3]);
    }
    __syncwarp();
}

// q/k head norm + RoPE of one 128-wide head vector by one warp, as qknorm_rope_kvappend_kernel does it:
// lane l owns elements 4l..4l+3 (`raw`: its four bf16 inputs, `wraw`: its norm weights, `craw` / `sraw`:
// its cos / sin table entries), the RoPE partner lives in lane l ^ 16.  o[] receives the sums before
// the final bf16 rounding.
__device__ __forceinline__ void rope_head_vector(uint2 raw, uint2 wraw, uint2 craw, uint2 sraw, float eps, int lane,
                                                 float (&o)[4]) {
    const float x[4] = {__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                        __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u)};
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) acc = fmaf(x[i], x[i], acc);
    const float total = warp_sum_butterfly(acc);
    const float r = bm_rsqrtf((0.0f + total) / 128.0f + eps);
    const float wv[4] = {__uint_as_float(wraw.x << 16), __uint_as_float(wraw.x & 0xffff0000u),
                         __uint_as_float(wraw.y << 16), __uint_as_float(wraw.y & 0xffff0000u)};
    const float c[4] = {__uint_as_float(craw.x << 16), __uint_as_float(craw.x & 0xffff0000u),
                        __uint_as_float(craw.y << 16), __uint_as_float(craw.y & 0xffff0000u)};
    const float sn[4] = {__uint_as_float(sraw.x << 16), __uint_as_float(sraw.x & 0xffff0000u),
                         __uint_as_float(sraw.y << 16), __uint_as_float(sraw.y & 0xffff0000u)};
    float n[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) n[i] = bm_bf16_rn(wv[i] * bm_bf16_rn(x[i] * r));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float partner = __shfl_xor_sync(0xffffffffu, n[i], 16);
        const float rot = lane < 16 ? -partner : partner;
        o[i] = bm_bf16_rn(n[i] * c[i]) + bm_bf16_rn(rot * sn[i]);
    }
}

// ---- kernel 1b: kernel 1 with the q/k norm, RoPE and KV append of the replay's rows folded in ----
// Reads the qkv projection output instead of rotated queries: every CTA rotates the query vectors it
// serves, the CTAs of the chunk that holds the replay's own rows compute their K rows (norm + RoPE),
// copy their V rows, and the z == 0 one appends both to the layer's planes.  Replaces
// qknorm_rope_kvappend_kernel + attn_chunk_kernel (one launch less per layer); same arithmetic.
struct AttnRopeParams {
    AttnParams a;
    const uint16_t *xqkv;            // [M, (H + 2 Hkv) * 128] bf16
    const uint16_t *q_w, *k_w;       // head-norm weights, bf16 [128]
    const uint16_t *cos_t, *sin_t;   // bf16 [max_pos, 128]
    const int64_t *positions;        // [M]
    uint16_t *k_out, *v_out;         // the layer's planes (same memory as a.k_base / a.v_base)
    float eps;
};

constexpr int kRopeBatch = 4;        // head vectors a warp rotates per batch (loads issued together)

// MINB: CTAs per SM the register budget is cut for.  3 (<= 85 registers) makes a chunk's pass ~20 % slower
// but lets half as many CTAs again run at once: worth it when the history is long enough for several waves of
// CTAs (measured at width 16: 1245 -> 1286 us per replay at cache_len 300, where 176 CTAs are one wave either
// way; 1406 -> 1336 us at cache_len 700, where 368 CTAs need two waves at two per SM).  The host picks it
// from the segment size.
template <int NQ, int MINB>
__global__ void __launch_bounds__(kAttnThreads, MINB) attn_chunk_rope_kernel(const AttnRopeParams P) {
    extern __shared__ __align__(16) unsigned char dyn[];
    const AttnParams &p = P.a;
    pdl_launch_dependents();
    const bool early = (p.pdl & BM_PDL_STABLE_STATE) != 0;
    if (p.pdl && !early) pdl_wait();
    const int j = blockIdx.x, hk = blockIdx.y;
    const int cache_len = attn_cache_len(p), n_pend = p.state->n_pend, role = p.state->role, P_ = p.state->P;
    const int n_hist = (cache_len + BM_ATTN_CHUNK - 1) / BM_ATTN_CHUNK;
    int c0, cn;
    if (j == p.NC - 1) { c0 = p.sigma; cn = p.M; }
    else if (j < n_hist) { c0 = j * BM_ATTN_CHUNK; cn = min(BM_ATTN_CHUNK, cache_len - c0); }
    else return;
    const bool fresh = j == p.NC - 1;

    const int G = p.H / p.Hkv, QV = G * p.M, heads = p.H + 2 * p.Hkv;
    uint16_t *Ks = reinterpret_cast<uint16_t *>(dyn);                    // [32][136]
    uint16_t *Vs = Ks + 32 * kKeyStride;                                  // [32][128]
    float *Qs = reinterpret_cast<float *>(Vs + 32 * 128);                 // [QV][128]
    float *Ps = Qs + (size_t)QV * 128;                                    // [QV][32]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthr = blockDim.x, nwarps = nthr >> 5;
    const int per = (QV + (int)gridDim.z - 1) / (int)gridDim.z;
    const int q_lo = (int)blockIdx.z * per, q_hi = min(QV, q_lo + per);

    // Nothing below depends on the previous kernel until the wait: history rows, positions, tables.
    // The chunk's history rows go straight to shared memory (asynchronous 16-byte copies, no registers
    // held across the rotation below).
    if (!fresh) {
        const uint4 *kg = reinterpret_cast<const uint4 *>(p.k_base + ((size_t)hk * p.kv_rows + c0) * 128);
        const uint4 *vg = reinterpret_cast<const uint4 *>(p.v_base + ((size_t)hk * p.kv_rows + c0) * 128);
        for (int i = tid; i < cn * 16; i += nthr) {
            cp_async16(Ks + (i >> 4) * kKeyStride + 8 * (i & 15), kg + i);
            cp_async16(Vs + 8 * i, vg + i);
        }
    }
    const uint2 qw = *reinterpret_cast<const uint2 *>(P.q_w + 4 * lane);
    const uint2 kw = *reinterpret_cast<const uint2 *>(P.k_w + 4 * lane);
    if (early) pdl_wait();                                                // xqkv comes from the predecessor

    if (fresh) {
        for (int m0 = warp; m0 < p.M; m0 += nwarps * kRopeBatch) {
            uint2 kraw[kRopeBatch], vraw[kRopeBatch], cr[kRopeBatch], sr[kRopeBatch];
#pragma unroll
            for (int k = 0; k < kRopeBatch; ++k) {
                const int m = m0 + k * nwarps;
                if (m < p.M) {
                    const size_t pos = (size_t)P.positions[m];
                    kraw[k] = *reinterpret_cast<const uint2 *>(P.xqkv + ((size_t)m * heads + p.H + hk) * 128 + 4 * lane);
                    vraw[k] = *reinterpret_cast<const uint2 *>(P.xqkv + ((size_t)m * heads + p.H + p.Hkv + hk) * 128 + 4 * lane);
                    cr[k] = *reinterpret_cast<const uint2 *>(P.cos_t + pos * 128 + 4 * lane);
                    sr[k] = *reinterpret_cast<const uint2 *>(P.sin_t + pos * 128 + 4 * lane);
                }
            }
#pragma unroll
            for (int k = 0; k < kRopeBatch; ++k) {
                const int m = m0 + k * nwarps;
                if (m >= p.M) break;                                       // warp-uniform
                float o[4];
                rope_head_vector(kraw[k], kw, cr[k], sr[k], P.eps, lane, o);
                const uint2 kbits = make_uint2(
                    (uint32_t)bm_f32_to_bf16(o[0]) | ((uint32_t)bm_f32_to_bf16(o[1]) << 16),
                    (uint32_t)bm_f32_to_bf16(o[2]) | ((uint32_t)bm_f32_to_bf16(o[3]) << 16));
                *reinterpret_cast<uint2 *>(Ks + m * kKeyStride + 4 * lane) = kbits;
                *reinterpret_cast<uint2 *>(Vs + m * 128 + 4 * lane) = vraw[k];
                if (blockIdx.z == 0) {
                    const size_t row = ((size_t)hk * p.kv_rows + p.sigma + m) * 128 + 4 * lane;
                    *reinterpret_cast<uint2 *>(P.k_out + row) = kbits;
                    *reinterpret_cast<uint2 *>(P.v_out + row) = vraw[k];
                }
            }
        }
    }
    for (int v0 = q_lo + warp; v0 < q_hi; v0 += nwarps * kRopeBatch) {
        uint2 qraw[kRopeBatch], cr[kRopeBatch], sr[kRopeBatch];
#pragma unroll
        for (int k = 0; k < kRopeBatch; ++k) {
            const int qv = v0 + k * nwarps;
            if (qv < q_hi) {
                const int g = qv / p.M, m = qv - g * p.M;
                const size_t pos = (size_t)P.positions[m];
                qraw[k] = *reinterpret_cast<const uint2 *>(P.xqkv + ((size_t)m * heads + hk * G + g) * 128 + 4 * lane);
                cr[k] = *reinterpret_cast<const uint2 *>(P.cos_t + pos * 128 + 4 * lane);
                sr[k] = *reinterpret_cast<const uint2 *>(P.sin_t + pos * 128 + 4 * lane);
            }
        }
#pragma unroll
        for (int k = 0; k < kRopeBatch; ++k) {
            const int qv = v0 + k * nwarps;
            if (qv >= q_hi) break;                                         // warp-uniform
            float o[4];
            rope_head_vector(qraw[k], qw, cr[k], sr[k], P.eps, lane, o);
            *reinterpret_cast<float4 *>(Qs + (size_t)qv * 128 + 4 * lane) =
                make_float4(bm_bf16_rn(o[0]), bm_bf16_rn(o[1]), bm_bf16_rn(o[2]), bm_bf16_rn(o[3]));
        }
    }
    cp_async_wait_all();
    __syncthreads();
    for (int q0 = q_lo + warp * NQ; q0 < q_hi; q0 += nwarps * NQ)
        attn_chunk_pass<NQ>(p, Ks, Vs, Qs, Ps, q0, q_hi, G, hk, j, c0, cn, lane, role, cache_len, n_pend, P_);
}

template <int NQ>
__global__ void __launch_bounds__(kAttnThreads) attn_chunk_kernel(const AttnParams p) {
    extern __shared__ __align__(16) unsigned char dyn[];
    pdl_launch_dependents();
    // BM_PDL_STABLE_STATE: the step record and the history rows were written by launches
    // that had completed before this call's chain of overlapped launches began, so they
    // may be read while the predecessor is still running.
    const bool early = (p.pdl & BM_PDL_STABLE_STATE) != 0;
    if (p.pdl && !early) pdl_wait();
    const int j = blockIdx.x, hk = blockIdx.y;
    const int cache_len = attn_cache_len(p), n_pend = p.state->n_pend, role = p.state->role,
              P = p.state->P;
    const int n_hist = (cache_len + BM_ATTN_CHUNK - 1) / BM_ATTN_CHUNK;
    int c0, cn;
    if (j == p.NC - 1) { c0 = p.sigma; cn = p.M; }
    else if (j < n_hist) { c0 = j * BM_ATTN_CHUNK; cn = min(BM_ATTN_CHUNK, cache_len - c0); }
    else return;
    const bool fresh_rows = j == p.NC - 1;            // rows the predecessor appended
    if (early && fresh_rows) pdl_wait();

    const int G = p.H / p.Hkv, QV = G * p.M;
    uint16_t *Ks = reinterpret_cast<uint16_t *>(dyn);                    // [32][136]
    uint16_t *Vs = Ks + 32 * kKeyStride;                                  // [32][128]
    float *Qs = reinterpret_cast<float *>(Vs + 32 * 128);                 // [QV][128]
    float *Ps = Qs + (size_t)QV * 128;                                    // [QV][32]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthr = blockDim.x;

    const uint16_t *kg = p.k_base + ((size_t)hk * p.kv_rows + c0) * 128;
    const uint16_t *vg = p.v_base + ((size_t)hk * p.kv_rows + c0) * 128;
    for (int i = tid; i < cn * 16; i += nthr) {
        const int c = i >> 4, u = i & 15;
        *reinterpret_cast<uint4 *>(Ks + c * kKeyStride + 8 * u) = reinterpret_cast<const uint4 *>(kg)[i];
        reinterpret_cast<uint4 *>(Vs)[i] = reinterpret_cast<const uint4 *>(vg)[i];
    }
    if (early && !fresh_rows) pdl_wait();             // the query rows come from the predecessor
    const int qs_per = (QV + (int)gridDim.z - 1) / (int)gridDim.z;
    const int qs_lo = (int)blockIdx.z * qs_per, qs_hi = min(QV, qs_lo + qs_per);
    for (int i = qs_lo * 16 + tid; i < qs_hi * 16; i += nthr) {
        const int qv = i >> 4, u = i & 15;
        const int g = qv / p.M, m = qv - g * p.M;
        float f[8];
        unpack8(reinterpret_cast<const uint4 *>(p.q + ((size_t)m * p.H + hk * G + g) * 128)[u], f);
        float4 *dst = reinterpret_cast<float4 *>(Qs + (size_t)qv * 128 + 8 * u);
        dst[0] = make_float4(f[0], f[1], f[2], f[3]);
        dst[1] = make_float4(f[4], f[5], f[6], f[7]);
    }
    __syncthreads();

    // The query vectors of the kv head are dealt to gridDim.z CTAs (more resident warps per
    // chunk when there are many of them): this CTA serves [q_lo, q_hi).
    const int per = (QV + (int)gridDim.z - 1) / (int)gridDim.z;
    const int q_lo = (int)blockIdx.z * per, q_hi = min(QV, q_lo + per);
    const int nwarps = nthr >> 5;
    for (int q0 = q_lo + warp * NQ; q0 < q_hi; q0 += nwarps * NQ)
        attn_chunk_pass<NQ>(p, Ks, Vs, Qs, Ps, q0, q_hi, G, hk, j, c0, cn, lane, role, cache_len, n_pend, P);
}

// ---- kernel 2: one CTA per query row merges the chunks of every head and quantises ----
// Thread = 2 consecutive dims of one head.  The chunk numerators of a batch of up to 16
// chunks are requested first, so that their latencies overlap each other and the weight
// computation: per head (one warp each) the merge weights exp(m_j - max) and the ordered sum
// of l_j * w_j.  Then the numerators are merged in ascending chunk order, divided by l and
// rounded to bf16; the row's absmax is a block reduction and the INT8 codes follow from a
// shared-memory copy of the row.  No cross-CTA hand-off.
constexpr int kMergeMaxHeads = 32;
constexpr int kMergeThreads = 1024;
constexpr int kMergeBatch = 16;

// Row m of the merge: all threads of the CTA (any multiple of 32 up to kMergeThreads); `dyn` holds
// H*128 bf16 + H*nv floats, `l_s` kMergeMaxHeads floats, `red` one float per warp.  The chunk
// partials are read through L2 (ld.global.cg): in the persistent decode kernel another SM wrote them.
__device__ __forceinline__ void attn_merge_row(const AttnParams &p, int m, int cache_len, unsigned char *dyn,
                                               float *l_s, float *red) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthr = blockDim.x;
    const int n_hist = (cache_len + BM_ATTN_CHUNK - 1) / BM_ATTN_CHUNK;
    const int nv = n_hist + 1;                        // valid chunks: history, then NC-1
    uint16_t *row_s = reinterpret_cast<uint16_t *>(dyn);                  // [H*128] bf16 row
    float *w_s = reinterpret_cast<float *>(row_s + (size_t)p.H * 128);    // [H][nv] weights
    const int pairs = p.H * 64;                       // 2-dim units of the row
    const int nwarps = nthr >> 5;

    float amax = 0.0f;
    for (int base = 0; base < pairs; base += nthr) {
        const int u = base + tid;
        const bool live = u < pairs;
        const int h = live ? (u >> 6) : 0, d0 = (u & 63) * 2;
        const float *src = p.po + ((size_t)m * p.H + h) * p.NC * 128 + d0;
        float o0 = 0.0f, o1 = 0.0f;
        for (int b0 = 0; b0 < nv; b0 += kMergeBatch) {
            const int nb = min(kMergeBatch, nv - b0);
            float2 part[kMergeBatch];
#pragma unroll
            for (int i = 0; i < kMergeBatch; ++i) {
                const int c = b0 + i;
                const int j = c < n_hist ? c : p.NC - 1;
                part[i] = (live && i < nb) ? __ldcg(reinterpret_cast<const float2 *>(src + (size_t)j * 128))
                                           : make_float2(0.0f, 0.0f);
            }
            if (base == 0 && b0 == 0) {
                // weights of every head, while the numerators are in flight
                for (int hh = warp; hh < p.H; hh += nwarps) {
                    const size_t pb = ((size_t)m * p.H + hh) * p.NC;
                    float gmax = -INFINITY;
                    float pl0 = 0.0f;                  // chunk sum of this lane's first chunk
                    for (int i = lane; i < nv; i += 32) {
                        const int jj = i < n_hist ? i : p.NC - 1;
                        const float mj = __ldcg(p.pm + pb + jj);
                        if (i < 32) pl0 = __ldcg(p.pl + pb + jj);
                        w_s[hh * nv + i] = mj;
                        gmax = fmaxf(gmax, mj);
                    }
                    gmax = warp_max(gmax);
                    float l = 0.0f;
                    for (int i0 = 0; i0 < nv; i0 += 32) {
                        const int i = i0 + lane;
                        float w = 0.0f, pl = 0.0f;
                        if (i < nv) {
                            const float mj = w_s[hh * nv + i];
                            w = mj > -INFINITY ? bm_expf(mj - gmax) : 0.0f;
                            pl = i0 == 0 ? pl0 : __ldcg(p.pl + pb + (i < n_hist ? i : p.NC - 1));
                            w_s[hh * nv + i] = w;
                        }
                        // ordered sum; a chunk without a visible key has weight 0 and sum 0
                        const int cnt = min(32, nv - i0);
                        for (int k = 0; k < cnt; ++k)
                            l = fmaf(__shfl_sync(0xffffffffu, pl, k), __shfl_sync(0xffffffffu, w, k), l);
                    }
                    if (lane == 0) l_s[hh] = l;
                }
                __syncthreads();
            }
#pragma unroll
            for (int i = 0; i < kMergeBatch; ++i) {
                if (i < nb) {
                    // a chunk without a visible key has weight 0 and a zero numerator
                    const float w = w_s[h * nv + b0 + i];
                    o0 = fmaf(part[i].x, w, o0);
                    o1 = fmaf(part[i].y, w, o1);
                }
            }
        }
        if (live) {
            const float l = l_s[h];
            const float v0 = bm_bf16_rn(o0 / l), v1 = bm_bf16_rn(o1 / l);
            amax = fmaxf(amax, fmaxf(fabsf(v0), fabsf(v1)));
            reinterpret_cast<uint32_t *>(row_s)[u] =
                (uint32_t)bm_f32_to_bf16(v0) | ((uint32_t)bm_f32_to_bf16(v1) << 16);
        }
    }
    amax = block_max(amax, red, lane, warp, nwarps);   // also orders the row_s writes
    const float s = bm_act_scale(amax);
    const int units = p.H * 16;                       // 8-dim units of the row
    const size_t row = (size_t)m * p.H * 128;
    for (int base = 0; base < units; base += nthr) {
        if (base + warp * 32 >= units) break;          // warp-uniform
        const int u = base + tid;
        const bool active = u < units;
        float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (active) {
            const uint4 raw = reinterpret_cast<const uint4 *>(row_s)[u];
            unpack8(raw, f);
            if (p.att) reinterpret_cast<uint4 *>(p.att + row)[u] = raw;
        }
        emit_codes(p.q_out, row, p.H * 128, u, quant8(f, s), active, lane);
    }
    if (tid == 0) p.s_out[m] = s;
}


// ---- kernel 2b: the merge spread over (row, head group) CTAs, without the quantisation ----
// Same merge as attn_merge_row for `hpc` heads of one row per CTA (thread = 2 dims of one head, up to
// 32 chunk numerators per thread in flight): writes the bf16 attention row and folds its absmax into
// amax_out[m] by atomic max (float bits; zero on entry).  The INT8 codes then come from
// quant_rows_amax_kernel.  With M rows alone only M SMs would merge; this uses M * H / hpc of them.
constexpr int kMergePartBatch = 32;

__global__ void __launch_bounds__(256) attn_merge_part_kernel(const AttnParams p, unsigned int *amax_out, int hpc) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ float l_s[8];
    __shared__ float red[8];
    pdl_launch_dependents();
    const bool early = (p.pdl & BM_PDL_STABLE_STATE) != 0;
    if (p.pdl && !early) pdl_wait();
    const int cache_len = attn_cache_len(p);
    if (early) pdl_wait();
    const int m = blockIdx.x, h0 = blockIdx.y * hpc;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthr = blockDim.x, nwarps = nthr >> 5;
    const int n_hist = (cache_len + BM_ATTN_CHUNK - 1) / BM_ATTN_CHUNK;
    const int nv = n_hist + 1;
    float *w_s = reinterpret_cast<float *>(dyn);      // [hpc][nv] merge weights
    const int hl = tid >> 6, d0 = (tid & 63) * 2;     // local head, first of the two dims
    const int h = h0 + hl;
    const float *src = p.po + ((size_t)m * p.H + h) * p.NC * 128 + d0;
    float o0 = 0.0f, o1 = 0.0f;
    for (int b0 = 0; b0 < nv; b0 += kMergePartBatch) {
        const int nb = min(kMergePartBatch, nv - b0);
        float2 part[kMergePartBatch];
#pragma unroll
        for (int i = 0; i < kMergePartBatch; ++i) {
            const int c = b0 + i;
            const int j = c < n_hist ? c : p.NC - 1;
            part[i] = i < nb ? __ldcg(reinterpret_cast<const float2 *>(src + (size_t)j * 128)) : make_float2(0.0f, 0.0f);
        }
        if (b0 == 0) {
            // weights of this CTA's heads (one warp each), while the numerators are in flight
            for (int hh = warp; hh < hpc; hh += nwarps) {
                const size_t pb = ((size_t)m * p.H + h0 + hh) * p.NC;
                float gmax = -INFINITY;
                float pl0 = 0.0f;
                for (int i = lane; i < nv; i += 32) {
                    const int jj = i < n_hist ? i : p.NC - 1;
                    const float mj = __ldcg(p.pm + pb + jj);
                    if (i < 32) pl0 = __ldcg(p.pl + pb + jj);
                    w_s[hh * nv + i] = mj;
                    gmax = fmaxf(gmax, mj);
                }
                gmax = warp_max(gmax);
                float l = 0.0f;
                for (int i0 = 0; i0 < nv; i0 += 32) {
                    const int i = i0 + lane;
                    float w = 0.0f, pl = 0.0f;
                    if (i < nv) {
                        const float mj = w_s[hh * nv + i];
                        w = mj > -INFINITY ? bm_expf(mj - gmax) : 0.0f;
                        pl = i0 == 0 ? pl0 : __ldcg(p.pl + pb + (i < n_hist ? i : p.NC - 1));
                        w_s[hh * nv + i] = w;
                    }
                    const int cnt = min(32, nv - i0);
                    for (int k = 0; k < cnt; ++k)
                        l = fmaf(__shfl_sync(0xffffffffu, pl, k), __shfl_sync(0xffffffffu, w, k), l);
                }
                if (lane == 0) l_s[hh] = l;
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < kMergePartBatch; ++i) {
            if (i < nb) {
                const float w = w_s[hl * nv + b0 + i];
                o0 = fmaf(part[i].x, w, o0);
                o1 = fmaf(part[i].y, w, o1);
            }
        }
    }
    const float l = l_s[hl];
    const float v0 = bm_bf16_rn(o0 / l), v1 = bm_bf16_rn(o1 / l);
    reinterpret_cast<uint32_t *>(p.att + (size_t)m * p.H * 128 + h * 128)[tid & 63] =
        (uint32_t)bm_f32_to_bf16(v0) | ((uint32_t)bm_f32_to_bf16(v1) << 16);
    const float amax = block_max(fmaxf(fabsf(v0), fabsf(v1)), red, lane, warp, nwarps);
    if (tid == 0 && amax != 0.0f) atomicMax(&amax_out[m], __float_as_uint(amax));
}

__global__ void __launch_bounds__(kMergeThreads) attn_merge_kernel(const AttnParams p) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ float l_s[kMergeMaxHeads];
    __shared__ float red[kMergeThreads / 32];
    pdl_launch_dependents();
    const bool early = (p.pdl & BM_PDL_STABLE_STATE) != 0;
    if (p.pdl && !early) pdl_wait();
    const int cache_len = attn_cache_len(p);
    if (early) pdl_wait();
    attn_merge_row(p, blockIdx.x, cache_len, dyn, l_s, red);
}

}  // namespace bm
