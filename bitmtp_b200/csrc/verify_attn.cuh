// Block-verify attention over the shared KV buffer: scores, softmax, numerators and the merge of
// the split-KV partials in ONE launch per layer.
//
// Replaces, for one layer of one replay, the attention of Attention.forward_sdlm_graph_kernel
// (src/bonsai_sft/gpu/model.py:989-1004: flex_attention closure or matmul/softmax/matmul and the
// permute back to [M, q_dim]) together with the additive mask tensor the host rebuilds before every
// replay (src/bonsai_sft/gpu/fast_runtime.py:345-372, 391-465) and, in the ROPE build, the q/k head
// norm, RoPE and KV append of _fused_qkv_qknorm_rope_kv_write (model.py:388-436).  Differences in
// kind, not in result:
//   * visibility is evaluated from (role, cache_len, n_pend) held in device memory (bm_visible in
//     bm_math.h), so nothing is rebuilt on the host and a captured graph serves every cache length;
//   * only history rows [0, cache_len) and the M rows of this replay are read, not the whole padded
//     buffer of sigma + M rows;
//   * the keys are cut into super-chunks of 128 (four sub-chunks of 32); one CTA serves one
//     (super-chunk, kv head, group of up to 8 query vectors), its 8 warps = 4 sub-chunks x 2 query
//     sub-groups; the CTA merges its four sub-chunk partials in shared memory and writes one partial
//     per query vector; the last CTA of a (kv head, query group) to finish (a ticket counter in the
//     scratch) merges the super-chunk partials, divides and writes the bf16 rows.
//
// Arithmetic and order: see bmo_attention in oracle/bm_oracle.c; the two agree bit for bit.  All
// accumulation is fp32 on the CUDA cores in a fixed order; tensor-core accumulation order is not
// specified by the hardware documents and could not be mirrored on the CPU.
//
// Scratch (caller-allocated, bm_verify_attention_scratch_bytes; zero before the first call, the
// kernel leaves its counters zero):
//   1024 bytes                 224 ticket counters, then 32 row-absmax words
//   pm, pl fp32 [M, H, NJ]      super-chunk max / sum
//   po   fp32 [M, H, NJ, 128]   super-chunk numerators
//   rows bf16 [M, H*128]        attention rows when the caller passes no att_out
//   NJ = ceil(sigma/128) + 1; super-chunk NJ-1 holds the rows appended by this replay.
#pragma once

#include "bm_common.cuh"
#include "fused_ops.cuh"

namespace bm {

constexpr int kAttnThreads = 256;
constexpr int kAttnSub = BM_ATTN_SUPER / BM_ATTN_CHUNK;   // sub-chunks per super-chunk (4)
constexpr int kKeyStride = 136;        // bf16 elements per staged key row (128 + 8 pad = 272 bytes)
constexpr int kAttnHeaderBytes = 1024;
constexpr int kAttnTickets = 224;      // counters in the header; the row absmax words follow
constexpr int kAttnMaxQ = 8;           // query vectors per CTA (2 sub-groups of up to 4)
constexpr int kAttnMaxNJ = 64;         // super-chunk partials one merging warp handles (2 per lane)
constexpr int kAttnMaxCluster = 16;    // super-chunks (CTAs) of one cluster in the cluster build

struct AttnParams {
    const uint16_t *q;        // [M, H, 128] rotated queries (plain build)
    const uint16_t *k_base;   // [Hkv, kv_rows, 128]
    const uint16_t *v_base;
    const StepState *state;
    int M, H, Hkv, kv_rows, sigma, NJ;
    unsigned int *tickets;    // [Hkv * gridDim.z], zero between launches
    unsigned int *amax;       // [M] row absmax bits, gathered by atomic max (zero on entry)
    float *pm, *pl, *po;
    uint16_t *att;            // [M, H*128] bf16 attention output
    int pdl;
    // ROPE build: the qkv projection output and what the rotation needs
    const uint16_t *xqkv;            // [M, (H + 2 Hkv) * 128] bf16
    const uint16_t *q_w, *k_w;       // head-norm weights, bf16 [128]
    const uint16_t *cos_t, *sin_t;   // bf16 [max_pos, 128]
    const int64_t *positions;        // [M]
    uint16_t *k_out, *v_out;         // the layer's planes (same memory as k_base / v_base)
    float eps;
    // Prompt mode (plain build only; slab_rows > 0): M prompt rows whose K / V already sit at rows
    // [slab_hist0, slab_hist0 + M) of the planes are served as AR-causal slabs of slab_rows rows: slab s
    // sees history [0, slab_hist0 + s * slab_rows) and its own rows.  blockIdx.x runs over the
    // (slab, super-chunk) pairs in slab order; `state` is not read; q, att, amax and the partials are
    // indexed by prompt row; tickets [slabs][Hkv][gridDim.z].
    int slab_rows, slab_hist0;
    int slots;       // CTAs the device holds at once (0: keep the coarse query split)
};

__host__ __device__ inline size_t attn_scratch_bytes(int M, int H, int sigma) {
    const size_t NJ = (size_t)(sigma + BM_ATTN_SUPER - 1) / BM_ATTN_SUPER + 1;
    return kAttnHeaderBytes + (size_t)M * H * NJ * 4 * 2 + (size_t)M * H * NJ * 128 * 4 + (size_t)M * H * 128 * 2;
}

// Query vectors per CTA sub-group (1..4) and CTAs per (super-chunk, kv head) for QV query vectors.
__host__ __device__ inline void attn_query_split(int QV, int *nq, int *z) {
    const int zz = (QV + kAttnMaxQ - 1) / kAttnMaxQ;
    *z = zz;
    *nq = (QV + 2 * zz - 1) / (2 * zz);
}

// The split above is the coarsest one (fewest CTAs).  A replay's launch carries more z-slices than that
// and every CTA picks, from the history length it reads on the device, the FINEST split whose working
// CTAs still fit the machine in one wave: query vectors per CTA between kAttnMinQ and 2 * nq.  With few
// history chunks that spreads the queries over more SMs (4 instead of 8 vectors per CTA is a quarter
// faster at width 16); with many it falls back to the coarse split, because a second wave costs more
// than the finer split saves.  Which CTA computes a query vector changes nothing in the arithmetic.
constexpr int kAttnMinQ = 4;
__host__ __device__ inline int attn_zmax(int QV, int nq) {
    const int qc_min = 2 * nq < kAttnMinQ ? 2 * nq : kAttnMinQ;
    return (QV + qc_min - 1) / qc_min;
}
__host__ __device__ inline int attn_pick_qc(int QV, int nq, int alive_chunks_x_heads, int slots) {
    const int QC = 2 * nq;
    for (int qc = (QC < kAttnMinQ ? QC : kAttnMinQ); qc < QC; ++qc)
        if (alive_chunks_x_heads * ((QV + qc - 1) / qc) <= slots) return qc;
    return QC;
}

__host__ __device__ inline size_t attn_smem_bytes(int nq) {
    const size_t QC = 2 * (size_t)nq;
    return (size_t)BM_ATTN_SUPER * kKeyStride * 2 + (size_t)BM_ATTN_SUPER * 128 * 2   // K (padded), V
           + QC * 128 * 4 + QC * BM_ATTN_SUPER * 4                                     // queries, weights
           + (size_t)kAttnSub * QC * 2 * 4 + (size_t)kAttnSub * QC * 128 * 4;          // sub-chunk partials
}

// History length of this replay.  The record is written by other launches (or by the caller through
// the C ABI), so it is clamped to [0, sigma] before anything is indexed with it: the scratch, the
// shared-memory arrays and the K/V planes are all sized from sigma.  Identity for every valid record.
__device__ __forceinline__ int attn_cache_len(const AttnParams &p) {
    return min(max(p.state->cache_len, 0), p.sigma);
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

// One warp, one sub-chunk of up to 32 keys, NQ query vectors.  lane = key in the score phase (NQ
// independent fma chains, one per query vector, each in ascending d), lane = 4 output dims in the
// numerator phase (4*NQ independent chains, each in ascending key order).
//   Ks / Vs   the sub-chunk's rows in shared memory (Ks padded to kKeyStride)
//   Qs        [NQ][128] fp32 query vectors of this warp;  Ps [NQ][BM_ATTN_SUPER] weights, the warp
//             uses columns [pcol, pcol + 32)
//   rows[t]   query row (0..M-1) of vector t, for the visibility predicate
//   out: mc[t], lc[t] (max, sum) and oc[t][128] (numerators) in shared memory
template <int NQ>
__device__ __forceinline__ void attn_sub_pass(const uint16_t *Ks, const uint16_t *Vs, const float *Qs, float *Ps,
                                              int pcol, const int (&rows)[NQ], int key0, int cn, int lane, int sigma,
                                              int role, int cache_len, int n_pend, int P, float *mc, float *lc,
                                              float *oc) {
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
            const float4 qa = *reinterpret_cast<const float4 *>(Qs + t * 128 + 8 * u);
            const float4 qb = *reinterpret_cast<const float4 *>(Qs + t * 128 + 8 * u + 4);
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
        const bool vis = lane < cn && bm_visible(role, rows[t], key0 + lane, sigma, cache_len, n_pend, P);
        const float sc = vis ? acc[t] * 0.08838834764831845f : -INFINITY;
        const float mj = warp_max(sc);
        const float pr = vis ? bm_expf(sc - mj) : 0.0f;
        const float lj = warp_sum_butterfly(pr);
        Ps[t * BM_ATTN_SUPER + pcol + lane] = bm_bf16_rn(pr);
        if (lane == 0) {
            mc[t] = mj;
            lc[t] = lj;
        }
    }
    __syncwarp();
    // numerators: lane owns dims 4*lane .. 4*lane+3 of the NQ query vectors
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
            const uint2 raw = (cb + cc < cn) ? *reinterpret_cast<const uint2 *>(Vs + (cb + cc) * 128 + 4 * lane)
                                             : make_uint2(0u, 0u);
            v[cc][0] = __uint_as_float(raw.x << 16);
            v[cc][1] = __uint_as_float(raw.x & 0xffff0000u);
            v[cc][2] = __uint_as_float(raw.y << 16);
            v[cc][3] = __uint_as_float(raw.y & 0xffff0000u);
        }
#pragma unroll
        for (int t = 0; t < NQ; ++t) {
            const float4 w = *reinterpret_cast<const float4 *>(Ps + t * BM_ATTN_SUPER + pcol + cb);
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
    for (int t = 0; t < NQ; ++t)
        *reinterpret_cast<float4 *>(oc + t * 128 + 4 * lane) = make_float4(o[t][0], o[t][1], o[t][2], o[t][3]);
}

// grid (NJ, Hkv, Z), 256 threads.  NQ: query vectors per warp (the CTA serves 2*NQ); ROPE: queries and
// the replay's own K/V rows are made here from the qkv projection output.
// CLUSTER: the NJ CTAs of a (kv head, query group) are one thread-block cluster (launch attribute
// (NJ, 1, 1), NJ <= kAttnMaxCluster).  The super-chunk partials then stay in the shared memory of the CTA
// that made them; the CTA of the replay's own rows (cluster rank NJ - 1, always working) reads them
// through distributed shared memory after one cluster barrier and merges them in the same order as the
// ticket build, so the fence, the ticket and the read-back from global memory drop out of the chain.  A
// second barrier keeps the other CTAs' shared memory alive until it has been read.  CTAs of super-chunks
// without rows take part in both barriers and do nothing else.
template <int NQ, bool ROPE, bool CLUSTER = false>
__global__ void __launch_bounds__(kAttnThreads, 2) attn_fused_kernel(const AttnParams p) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ unsigned int sh_ticket;
    constexpr int QC = 2 * NQ;
    pdl_launch_dependents();
    // BM_PDL_STABLE_STATE: the step record, the positions and the history rows were written by launches
    // that had completed before this call's chain of overlapped launches began, so they may be read
    // while the predecessor is still running.
    const bool early = (p.pdl & BM_PDL_STABLE_STATE) != 0;
    if (p.pdl && !early) pdl_wait();
    const int hk = blockIdx.y, z = blockIdx.z;
    int J = blockIdx.x, M_ = p.M, sigma_ = p.sigma, r0 = 0, cache_len, n_pend, role, P_;
    unsigned int *ticket = p.tickets + hk * gridDim.z + z;
    if (!ROPE && p.slab_rows > 0) {
        // prompt mode: find this CTA's slab; a slab with history h has ceil(h / 128) + 1 super-chunks
        int s = 0, rem = J, h = p.slab_hist0;
        for (;;) {
            const int units = (h + BM_ATTN_SUPER - 1) / BM_ATTN_SUPER + 1;
            if (rem < units) break;
            rem -= units;
            ++s;
            h += p.slab_rows;
        }
        r0 = s * p.slab_rows;
        M_ = min(p.slab_rows, p.M - r0);
        cache_len = sigma_ = h;
        n_pend = 0; role = BM_ROLE_AR; P_ = 0;
        J = rem < (h + BM_ATTN_SUPER - 1) / BM_ATTN_SUPER ? rem : p.NJ - 1;
        ticket += (size_t)s * p.Hkv * gridDim.z;
        if (M_ <= 0) return;
    } else {
        cache_len = attn_cache_len(p); n_pend = p.state->n_pend; role = p.state->role; P_ = p.state->P;
    }
    const int n_hs = (cache_len + BM_ATTN_SUPER - 1) / BM_ATTN_SUPER;     // history super-chunks with rows
    const bool fresh = J == p.NJ - 1;
    const int G = p.H / p.Hkv, QV = G * M_, heads = p.H + 2 * p.Hkv;
    // query vectors per CTA for this history length (see attn_pick_qc); sub-group 0 takes the larger half
    const int qc = (p.slots > 0 && p.slab_rows == 0) ? attn_pick_qc(QV, NQ, (n_hs + 1) * p.Hkv, p.slots) : QC;
    const int nq0 = (qc + 1) >> 1;
    const int q_lo = z * qc;
    if (q_lo >= QV) return;                // a surplus query group: all its CTAs (a whole cluster) leave here
    if (!fresh && J >= n_hs) {
        if (CLUSTER) {                     // a super-chunk without rows: both barrier phases, nothing else
            cluster_arrive(); cluster_wait();
            cluster_arrive(); cluster_wait();
        }
        return;
    }
    const int key0 = fresh ? sigma_ : J * BM_ATTN_SUPER;
    const int nkeys = fresh ? M_ : min(BM_ATTN_SUPER, cache_len - key0);

    uint16_t *Ks = reinterpret_cast<uint16_t *>(dyn);                              // [128][136]
    uint16_t *Vs = Ks + BM_ATTN_SUPER * kKeyStride;                                 // [128][128]
    float *Qs = reinterpret_cast<float *>(Vs + BM_ATTN_SUPER * 128);                // [QC][128]
    float *Ps = Qs + QC * 128;                                                      // [QC][128 keys]
    float *mc = Ps + QC * BM_ATTN_SUPER;                                            // [4][QC]
    float *lc = mc + kAttnSub * QC;                                                 // [4][QC]
    float *oc = lc + kAttnSub * QC;                                                 // [4][QC][128]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // Nothing below depends on the previous kernel until the wait: history rows, positions, tables.
    // The history rows go straight to shared memory (asynchronous 16-byte copies, no registers held).
    if (!fresh) {
        const uint4 *kg = reinterpret_cast<const uint4 *>(p.k_base + ((size_t)hk * p.kv_rows + key0) * 128);
        const uint4 *vg = reinterpret_cast<const uint4 *>(p.v_base + ((size_t)hk * p.kv_rows + key0) * 128);
        for (int i = tid; i < nkeys * 16; i += kAttnThreads) {
            cp_async16(Ks + (i >> 4) * kKeyStride + 8 * (i & 15), kg + i);
            cp_async16(Vs + 8 * i, vg + i);
        }
    }
    // this warp's query vector (one per warp: QC <= 8) and, in the CTA of the replay's own rows, its
    // share of those rows (m = warp, warp + 8, ...: at most kFreshPerWarp)
    const int qi = warp, qv = q_lo + qi;
    const bool q_live = qi < qc && qv < QV;
    const int qg_ = q_live ? qv / M_ : 0, qm = q_live ? qv - qg_ * M_ : 0;
    constexpr int kFreshPerWarp = BM_MAX_W / (kAttnThreads / 32);
    uint2 qw = make_uint2(0u, 0u), kw = qw, qcos = qw, qsin = qw;
    uint2 kcos[kFreshPerWarp], ksin[kFreshPerWarp];
    if (ROPE) {
        qw = *reinterpret_cast<const uint2 *>(p.q_w + 4 * lane);
        kw = *reinterpret_cast<const uint2 *>(p.k_w + 4 * lane);
        if (early) {
            // the positions were staged before the replay: their table rows can be fetched before the wait
            if (q_live) {
                const size_t pos = (size_t)p.positions[qm];
                qcos = *reinterpret_cast<const uint2 *>(p.cos_t + pos * 128 + 4 * lane);
                qsin = *reinterpret_cast<const uint2 *>(p.sin_t + pos * 128 + 4 * lane);
            }
            if (fresh) {
#pragma unroll
                for (int k = 0; k < kFreshPerWarp; ++k) {
                    const int m = warp + k * (kAttnThreads / 32);
                    if (m < M_) {
                        const size_t pos = (size_t)p.positions[m];
                        kcos[k] = *reinterpret_cast<const uint2 *>(p.cos_t + pos * 128 + 4 * lane);
                        ksin[k] = *reinterpret_cast<const uint2 *>(p.sin_t + pos * 128 + 4 * lane);
                    }
                }
            }
        }
    }
    if (early) pdl_wait();            // xqkv / q (and, in the plain build, the replay's own rows) come from the predecessor

    if (ROPE) {
        // every load that depends on the predecessor is issued before the first of them is used: one
        // memory round trip for the query vector and the replay's own K / V rows together
        uint2 qraw = make_uint2(0u, 0u), kraw[kFreshPerWarp], vraw[kFreshPerWarp];
        if (q_live) qraw = *reinterpret_cast<const uint2 *>(p.xqkv + ((size_t)qm * heads + hk * G + qg_) * 128 + 4 * lane);
        if (fresh) {
#pragma unroll
            for (int k = 0; k < kFreshPerWarp; ++k) {
                const int m = warp + k * (kAttnThreads / 32);
                if (m < M_) {
                    kraw[k] = *reinterpret_cast<const uint2 *>(p.xqkv + ((size_t)m * heads + p.H + hk) * 128 + 4 * lane);
                    vraw[k] = *reinterpret_cast<const uint2 *>(p.xqkv + ((size_t)m * heads + p.H + p.Hkv + hk) * 128 + 4 * lane);
                }
            }
        }
        if (!early) {
            if (q_live) {
                const size_t pos = (size_t)p.positions[qm];
                qcos = *reinterpret_cast<const uint2 *>(p.cos_t + pos * 128 + 4 * lane);
                qsin = *reinterpret_cast<const uint2 *>(p.sin_t + pos * 128 + 4 * lane);
            }
            if (fresh) {
#pragma unroll
                for (int k = 0; k < kFreshPerWarp; ++k) {
                    const int m = warp + k * (kAttnThreads / 32);
                    if (m < M_) {
                        const size_t pos = (size_t)p.positions[m];
                        kcos[k] = *reinterpret_cast<const uint2 *>(p.cos_t + pos * 128 + 4 * lane);
                        ksin[k] = *reinterpret_cast<const uint2 *>(p.sin_t + pos * 128 + 4 * lane);
                    }
                }
            }
        }
        if (qi < QC) {
            float4 qf = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (q_live) {
                float o[4];
                rope_head_vector(qraw, qw, qcos, qsin, p.eps, lane, o);
                qf = make_float4(bm_bf16_rn(o[0]), bm_bf16_rn(o[1]), bm_bf16_rn(o[2]), bm_bf16_rn(o[3]));
            }
            *reinterpret_cast<float4 *>(Qs + qi * 128 + 4 * lane) = qf;
        }
        if (fresh) {
            // the replay's own rows: K through norm + RoPE, V as it is; the z == 0 CTA appends them to the planes
#pragma unroll
            for (int k = 0; k < kFreshPerWarp; ++k) {
                const int m = warp + k * (kAttnThreads / 32);
                if (m >= M_) break;                                       // warp-uniform
                float o[4];
                rope_head_vector(kraw[k], kw, kcos[k], ksin[k], p.eps, lane, o);
                const uint2 kbits = make_uint2((uint32_t)bm_f32_to_bf16(o[0]) | ((uint32_t)bm_f32_to_bf16(o[1]) << 16),
                                               (uint32_t)bm_f32_to_bf16(o[2]) | ((uint32_t)bm_f32_to_bf16(o[3]) << 16));
                *reinterpret_cast<uint2 *>(Ks + m * kKeyStride + 4 * lane) = kbits;
                *reinterpret_cast<uint2 *>(Vs + m * 128 + 4 * lane) = vraw[k];
                if (z == 0) {
                    const size_t row = ((size_t)hk * p.kv_rows + sigma_ + m) * 128 + 4 * lane;
                    *reinterpret_cast<uint2 *>(p.k_out + row) = kbits;
                    *reinterpret_cast<uint2 *>(p.v_out + row) = vraw[k];
                }
            }
        }
    } else {
        if (fresh) {
            const uint4 *kg = reinterpret_cast<const uint4 *>(p.k_base + ((size_t)hk * p.kv_rows + key0) * 128);
            const uint4 *vg = reinterpret_cast<const uint4 *>(p.v_base + ((size_t)hk * p.kv_rows + key0) * 128);
            for (int i = tid; i < nkeys * 16; i += kAttnThreads) {
                cp_async16(Ks + (i >> 4) * kKeyStride + 8 * (i & 15), kg + i);
                cp_async16(Vs + 8 * i, vg + i);
            }
        }
        if (qi < QC) {
            float4 qf = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (q_live) {
                const uint2 raw = *reinterpret_cast<const uint2 *>(p.q + ((size_t)(r0 + qm) * p.H + hk * G + qg_) * 128 + 4 * lane);
                qf = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xffff0000u),
                                 __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xffff0000u));
            }
            *reinterpret_cast<float4 *>(Qs + qi * 128 + 4 * lane) = qf;
        }
    }
    cp_async_wait_all();
    __syncthreads();

    // level 0: warp = (sub-chunk c, query sub-group sg)
    {
        const int c = warp & (kAttnSub - 1), sg = warp >> 2;
        const int cn = min(BM_ATTN_CHUNK, nkeys - c * BM_ATTN_CHUNK);
        const int qoff = sg ? nq0 : 0, nqs = sg ? qc - nq0 : nq0;     // this warp's vectors: [qoff, qoff + nqs)
        float *mcw = mc + c * QC + qoff, *lcw = lc + c * QC + qoff;
        float *ocw = oc + ((size_t)c * QC + qoff) * 128;
        if (cn > 0) {
            const uint16_t *Kc = Ks + c * BM_ATTN_CHUNK * kKeyStride, *Vc = Vs + c * BM_ATTN_CHUNK * 128;
            const float *Qw = Qs + qoff * 128;
            float *Pw = Ps + qoff * BM_ATTN_SUPER;
            const int k0 = key0 + c * BM_ATTN_CHUNK, pc = c * BM_ATTN_CHUNK, qb = q_lo + qoff;
            // vectors past QV repeat the last one; their results are dropped by q_live below
#define BM_ATTN_PASS(N_)                                                                                          \
    {                                                                                                             \
        int rows[N_];                                                                                             \
        _Pragma("unroll") for (int t = 0; t < N_; ++t) {                                                          \
            const int v = min(qb + t, QV - 1);                                                                    \
            rows[t] = v - (v / M_) * M_;                                                                          \
        }                                                                                                         \
        attn_sub_pass<N_>(Kc, Vc, Qw, Pw, pc, rows, k0, cn, lane, sigma_, role, cache_len, n_pend, P_, mcw, lcw,  \
                          ocw);                                                                                   \
    }
            if (NQ >= 4 && nqs == 4) BM_ATTN_PASS(4)
            else if (NQ >= 3 && nqs == 3) BM_ATTN_PASS(3)
            else if (NQ >= 2 && nqs == 2) BM_ATTN_PASS(2)
            else if (nqs == 1) BM_ATTN_PASS(1)
#undef BM_ATTN_PASS
        } else {
            for (int t = 0; t < nqs; ++t) {
                if (lane == 0) { mcw[t] = -INFINITY; lcw[t] = 0.0f; }
                *reinterpret_cast<float4 *>(ocw + t * 128 + 4 * lane) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        }
    }
    __syncthreads();

    // level 1: the four sub-chunk partials of query vector qi, merged in ascending sub-chunk order
    if (q_live) {
        float mm[kAttnSub], MJ = -INFINITY;
#pragma unroll
        for (int c = 0; c < kAttnSub; ++c) { mm[c] = mc[c * QC + qi]; MJ = fmaxf(MJ, mm[c]); }
        float L = 0.0f, O[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int c = 0; c < kAttnSub; ++c) {
            const float w = mm[c] > -INFINITY ? bm_expf(mm[c] - MJ) : 0.0f;
            L = fmaf(lc[c * QC + qi], w, L);
            const float4 o = *reinterpret_cast<const float4 *>(oc + ((size_t)c * QC + qi) * 128 + 4 * lane);
            O[0] = fmaf(o.x, w, O[0]);
            O[1] = fmaf(o.y, w, O[1]);
            O[2] = fmaf(o.z, w, O[2]);
            O[3] = fmaf(o.w, w, O[3]);
        }
        if (CLUSTER) {
            // the partial stays in this CTA: numerators over the softmax weights and max / sum over the query
            // vector, both spent since the CTA barrier after level 0
            *reinterpret_cast<float4 *>(Ps + qi * BM_ATTN_SUPER + 4 * lane) = make_float4(O[0], O[1], O[2], O[3]);
            if (lane == 0) *reinterpret_cast<float2 *>(Qs + qi * 128) = make_float2(MJ, L);
        } else {
            const size_t pb = ((size_t)(r0 + qm) * p.H + hk * G + qg_) * p.NJ + J;
            *reinterpret_cast<float4 *>(p.po + pb * 128 + 4 * lane) = make_float4(O[0], O[1], O[2], O[3]);
            if (lane == 0) { p.pm[pb] = MJ; p.pl[pb] = L; }
        }
    }
    if (CLUSTER) {
        cluster_arrive();
        cluster_wait();
        if (fresh && q_live) {
            // level 2 in the cluster: history super-chunks (cluster ranks 0 .. n_hs-1) in ascending order, then
            // this CTA's own partial; at most kAttnMaxCluster of them, requested in batches of eight
            const int nv = n_hs + 1;
            const float *own_ml = Qs + qi * 128, *own_o = Ps + qi * BM_ATTN_SUPER + 4 * lane;
            float2 ml = make_float2(-INFINITY, 0.0f);
            if (lane < n_hs) ml = cluster_ld2(cluster_map(own_ml, (uint32_t)lane));
            else if (lane == n_hs) ml = *reinterpret_cast<const float2 *>(own_ml);
            constexpr int kBatch = 8;
            float4 part[kBatch];
#pragma unroll
            for (int i = 0; i < kBatch; ++i)
                part[i] = i < n_hs    ? cluster_ld4(cluster_map(own_o, (uint32_t)i))
                          : i == n_hs ? *reinterpret_cast<const float4 *>(own_o)
                                      : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            const float gmax = warp_max(ml.x);
            const float w0 = ml.x > -INFINITY ? bm_expf(ml.x - gmax) : 0.0f;
            float l = 0.0f, o[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int b0 = 0; b0 < nv; b0 += kBatch) {
                if (b0 > 0) {
#pragma unroll
                    for (int i = 0; i < kBatch; ++i) {
                        const int c = b0 + i;
                        part[i] = c < n_hs    ? cluster_ld4(cluster_map(own_o, (uint32_t)c))
                                  : c == n_hs ? *reinterpret_cast<const float4 *>(own_o)
                                              : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                    }
                }
#pragma unroll
                for (int i = 0; i < kBatch; ++i) {
                    const int c = b0 + i;
                    if (c < nv) {                                      // warp-uniform
                        const float w = __shfl_sync(0xffffffffu, w0, c);
                        const float lj = __shfl_sync(0xffffffffu, ml.y, c);
                        l = fmaf(lj, w, l);
                        o[0] = fmaf(part[i].x, w, o[0]);
                        o[1] = fmaf(part[i].y, w, o[1]);
                        o[2] = fmaf(part[i].z, w, o[2]);
                        o[3] = fmaf(part[i].w, w, o[3]);
                    }
                }
            }
            float v[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) v[e] = bm_bf16_rn(o[e] / l);
            const uint2 bits = make_uint2((uint32_t)bm_f32_to_bf16(v[0]) | ((uint32_t)bm_f32_to_bf16(v[1]) << 16),
                                          (uint32_t)bm_f32_to_bf16(v[2]) | ((uint32_t)bm_f32_to_bf16(v[3]) << 16));
            *reinterpret_cast<uint2 *>(p.att + (size_t)(r0 + qm) * p.H * 128 + (hk * G + qg_) * 128 + 4 * lane) = bits;
            const float amax = warp_max(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
            if (lane == 0 && amax != 0.0f) atomicMax(&p.amax[r0 + qm], __float_as_uint(amax));
        }
        // every remote value has been consumed above: the other CTAs of the cluster may leave
        cluster_arrive();
        cluster_wait();
        return;
    }
    // ticket: the last CTA of this (kv head, query group) to get here merges the super-chunks
    __threadfence();
    __syncthreads();
    if (tid == 0) sh_ticket = atomicAdd(ticket, 1u);
    __syncthreads();
    if (sh_ticket != (unsigned int)n_hs) return;                  // n_hs + 1 CTAs take part
    __threadfence();
    if (tid == 0) *ticket = 0u;                                   // ready for the next launch
    if (!q_live) return;

    // level 2: super-chunk partials of query vector qi in ascending order (history, then the replay's rows)
    const int nv = n_hs + 1;
    const size_t pb = ((size_t)(r0 + qm) * p.H + hk * G + qg_) * p.NJ;
    constexpr int kBatch = 8;
    float4 part[kBatch];
    // the first batch of numerators is requested together with the maxima and sums: one round trip
#pragma unroll
    for (int i = 0; i < kBatch; ++i) {
        const int j = i < n_hs ? i : p.NJ - 1;
        part[i] = i < nv ? __ldcg(reinterpret_cast<const float4 *>(p.po + (pb + j) * 128 + 4 * lane))
                         : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;
    if (lane < nv) {
        const int j = lane < n_hs ? lane : p.NJ - 1;
        m0 = __ldcg(p.pm + pb + j);
        l0 = __ldcg(p.pl + pb + j);
    }
    if (lane + 32 < nv) {
        const int j = lane + 32 < n_hs ? lane + 32 : p.NJ - 1;
        m1 = __ldcg(p.pm + pb + j);
        l1 = __ldcg(p.pl + pb + j);
    }
    const float gmax = warp_max(fmaxf(m0, m1));
    const float w0 = m0 > -INFINITY ? bm_expf(m0 - gmax) : 0.0f;
    const float w1 = m1 > -INFINITY ? bm_expf(m1 - gmax) : 0.0f;
    float l = 0.0f, o[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int b0 = 0; b0 < nv; b0 += kBatch) {
        if (b0 > 0) {
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
                const int c = b0 + i;
                const int j = c < n_hs ? c : p.NJ - 1;
                part[i] = c < nv ? __ldcg(reinterpret_cast<const float4 *>(p.po + (pb + j) * 128 + 4 * lane))
                                 : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            }
        }
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
            const int c = b0 + i;
            if (c < nv) {                                          // warp-uniform
                const float w = __shfl_sync(0xffffffffu, c < 32 ? w0 : w1, c & 31);
                const float lj = __shfl_sync(0xffffffffu, c < 32 ? l0 : l1, c & 31);
                l = fmaf(lj, w, l);
                o[0] = fmaf(part[i].x, w, o[0]);
                o[1] = fmaf(part[i].y, w, o[1]);
                o[2] = fmaf(part[i].z, w, o[2]);
                o[3] = fmaf(part[i].w, w, o[3]);
            }
        }
    }
    float v[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = bm_bf16_rn(o[e] / l);
    const uint2 bits = make_uint2((uint32_t)bm_f32_to_bf16(v[0]) | ((uint32_t)bm_f32_to_bf16(v[1]) << 16),
                                  (uint32_t)bm_f32_to_bf16(v[2]) | ((uint32_t)bm_f32_to_bf16(v[3]) << 16));
    *reinterpret_cast<uint2 *>(p.att + (size_t)(r0 + qm) * p.H * 128 + (hk * G + qg_) * 128 + 4 * lane) = bits;
    const float amax = warp_max(fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3]))));
    if (lane == 0 && amax != 0.0f) atomicMax(&p.amax[r0 + qm], __float_as_uint(amax));
}

}  // namespace bm
