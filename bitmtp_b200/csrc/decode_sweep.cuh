// One persistent kernel for all transformer layers of a decode replay.
//
// Replaces, for the layer stack of forward_sdlm_decode_graph_kernel
// (src/bonsai_sft/gpu/model.py:1363-1404 with 1119-1137, 958-1009, 1053-1064), the ten
// launches per layer of the operator-by-operator path: (residual add +) RMSNorm + quant,
// qkv GEMV, q/k norm + RoPE + KV append + attention chunks, chunk merge + quant, o GEMV,
// residual add + RMSNorm + quant, gate|up GEMV + SiLU*up, quant, down GEMV.  The final norm and
// the head stay separate launches.
//
// Why: at batch 1 every operator is a few microseconds of launch, drain and two or three
// dependent memory round trips around well under a microsecond of HBM time; a replay of ~310
// launches sits at ~7 % of its HBM roofline.  Here one CTA per SM stays resident, the stages
// are separated by a software grid barrier (one release-add and an acquire-poll on a global
// counter, bounded), and each CTA asks L2 for the weights of its next stage before it waits.
//
// Arithmetic: every stage calls the same device functions as the stand-alone kernels
// (mma_group_step, emit_codes, attn_chunk_pass, attn_merge_row, the bm_math.h scalars) in the
// same order, so the outputs are bit-identical to the operator-by-operator path, which is
// what the tests check.  Data that another CTA produced in an earlier stage is always read
// with ld.global.cg (L2): L1 is not coherent between SMs and the buffers are reused by
// every layer.
//
// Geometry served: dim == 2048 (one thread per 8 elements of a row), head_dim 128,
// K in {2048, 6144} for the GEMVs (K % 2048 == 0), M <= 16.  Other geometries use the
// operator-by-operator path.
#pragma once

#include "bm_common.cuh"
#include "t2_gemv.cuh"
#include "fused_ops.cuh"
#include "verify_attn.cuh"

namespace bm {

constexpr int kSweepThreads = 256;
constexpr unsigned int kSweepSpinLimit = 1u << 22;
enum : int { kErrSweepBarrierTimeout = 3 };

struct SweepLayer {
    const uint8_t *wqkv, *wo, *wgu, *wdown;            // packed codes
    const uint16_t *wqkv_s, *wo_s, *wgu_s, *wdown_s;    // bf16 scales
    const uint16_t *ln1, *ln2, *qn, *kn;                // norm weights
    uint16_t *k_base, *v_base;                          // this layer's [Hkv, kv_rows, 128] planes
};

struct SweepParams {
    const SweepLayer *layers;
    int n_layers, M, dim, H, Hkv, ffn, kv_rows, sigma, NC;
    float eps;
    const int64_t *tokens, *positions;
    const uint16_t *embed, *cos_t, *sin_t;
    const StepState *state;
    uint16_t *h;                 // [M, dim] residual stream
    int8_t *xq;                  // [M, dim] GEMV-ready codes of the normed row
    int32_t *xsum;               // [M, dim/128]
    float *xs;                   // [M]
    uint16_t *xqkv;              // [M, (H + 2 Hkv) * 128]
    float *pm, *pl, *po;         // attention chunk partials
    int8_t *attq;                // [M, H*128]
    int32_t *attsum;
    float *atts;
    uint16_t *attn_out;          // [M, dim]
    uint16_t *inner;             // [M, ffn] SiLU(gate) * up, bf16
    unsigned int *inner_amax;    // [M] bits of the row absmax (non-negative floats order as integers)
    int8_t *iq;                  // [M, ffn]
    int32_t *isum;
    float *is_;
    uint16_t *ffn_out;           // [M, dim]
    unsigned int *bar;           // [0] arrivals (zero at launch), [1] abort flag (zero at launch)
    unsigned long long *timing;  // optional [19]: global timer of CTA 0 at the stage boundaries of layer 1
};

// ---- loads of data written by other CTAs in an earlier stage ---------------------------
__device__ __forceinline__ uint4 ldcg4(const void *p) { return __ldcg(reinterpret_cast<const uint4 *>(p)); }
__device__ __forceinline__ uint2 ldcg2(const void *p) { return __ldcg(reinterpret_cast<const uint2 *>(p)); }

__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add(unsigned int *p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void *p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// ---- grid barrier -------------------------------------------------------------------------
// Every CTA of the (co-resident) grid arrives once; `target` counts arrivals so far.  The wait
// is bounded: a CTA that gives up raises the abort flag, after which no CTA waits or works any
// more and the kernel drains through its remaining barriers at once.
struct SweepSync {
    unsigned int target;
    bool alive;
};

__device__ __forceinline__ bool sweep_grid_sync(const SweepParams &p, SweepSync &st, int *sh_flag) {
    // bar.sync orders the CTA's writes before thread 0's release-add, which is cumulative
    __syncthreads();
    st.target += gridDim.x;
    if (threadIdx.x == 0) {
        bool alive = st.alive;
        if (alive) {
            red_release_add(&p.bar[0], 1u);
            unsigned int spins = 0;
            while (ld_acquire_u32(&p.bar[0]) < st.target) {
                if ((++spins & 63u) == 0u && (ld_acquire_u32(&p.bar[1]) != 0u || spins > kSweepSpinLimit)) {
                    atomicExch(&p.bar[1], 1u);
                    report_error(kErrSweepBarrierTimeout);
                    alive = false;
                    break;
                }
            }
        }
        *sh_flag = alive ? 1 : 0;
    }
    __syncthreads();
    st.alive = *sh_flag != 0;
    return st.alive;
}

// ---- stage: (gather | residual add) + RMSNorm + quantisation of one row --------------------
// Same arithmetic as rmsnorm_kernel; the CTA is dim/8 threads wide.
__device__ __noinline__ void sweep_norm_row(const SweepParams &p, int m, const uint16_t *x_row, bool x_shared,
                                               bool add_res, const uint16_t *w, float *sh) {
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, nwarps = kSweepThreads / 32;
    float h[8];
    const uint4 xv = x_shared ? ldcg4(x_row + 8 * t) : reinterpret_cast<const uint4 *>(x_row)[t];
    const uint4 wraw = reinterpret_cast<const uint4 *>(w)[t];    // requested with the row, used after the sum
    unpack8(xv, h);
    if (add_res) {
        float r[8];
        unpack8(ldcg4(p.h + (size_t)m * p.dim + 8 * t), r);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = bm_bf16_rn(h[i] + r[i]);
    }
    reinterpret_cast<uint4 *>(p.h + (size_t)m * p.dim)[t] = pack8(h);
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
    amax = block_max(amax, sh, lane, warp, nwarps);
    const float s = bm_act_scale(amax);
    const QuantSink sink{nullptr, p.xq, p.xsum};
    emit_codes(sink, (size_t)m * p.dim, p.dim, t, quant8(n, s), true, lane);
    if (t == 0) p.xs[m] = s;
}

// ---- stage: GEMV tiles ------------------------------------------------------------------------
// Fragments of group g for tokens r and r+8 from GEMV-ready rows written by another CTA.
template <bool HALF>
__device__ __forceinline__ void load_afrag_cg(AFrag<HALF> &f, const int8_t *rows, int K, const int32_t *asum,
                                              int W, int ng, int g, int r, int q) {
    f.lo0 = f.hi0 = f.lo8 = f.hi8 = make_uint4(0u, 0u, 0u, 0u);
    f.nb0 = f.nb8 = 0;
    if (r < W) {
        const int8_t *ap = rows + (size_t)r * K + BM_GROUP * g + 32 * q;
        f.lo0 = ldcg4(ap);
        f.hi0 = ldcg4(ap + 16);
        f.nb0 = -2 * __ldcg(asum + r * ng + g);
    }
    if (!HALF && r + 8 < W) {
        const int8_t *ap8 = rows + (size_t)(r + 8) * K + BM_GROUP * g + 32 * q;
        f.lo8 = ldcg4(ap8);
        f.hi8 = ldcg4(ap8 + 16);
        f.nb8 = -2 * __ldcg(asum + (r + 8) * ng + g);
    }
}

// Asks L2 for `bytes` bytes at `ptr` (whole 128-byte lines), all threads of the CTA.
__device__ __forceinline__ void sweep_prefetch(const void *ptr, size_t bytes) {
    const char *p = static_cast<const char *>(ptr);
    for (size_t off = (size_t)threadIdx.x * 128; off < bytes; off += (size_t)kSweepThreads * 128) prefetch_l2(p + off);
}

// Weight words and scales of one tile of RB blocks of 8 output rows, as lane (r, q) of warp w needs
// them: block rb is rows rowbase[rb] .. rowbase[rb]+7 of the packed matrix [N, K/4] with scales
// [N, K/128]; chunk c is the groups 16c + 2w and 16c + 2w + 1.  Straight from global memory: each
// lane's 8-byte pieces are whole 32-byte sectors across the four q lanes.
template <int RB, int NCH>
struct SweepTile {
    uint2 wA[NCH][RB], wB[NCH][RB];
    uint32_t x0[NCH][RB], x1[NCH][RB];
};

template <int RB, int NCH>
__device__ __forceinline__ void sweep_tile_load(SweepTile<RB, NCH> &t, const uint8_t *__restrict__ B,
                                                const uint16_t *__restrict__ ws, int K, const int (&rowbase)[RB],
                                                bool valid) {
    const int ng = K / BM_GROUP;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = lane >> 2, q = lane & 3;
    const size_t row_bytes = (size_t)(K / 4);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        const int g0 = c * BM_SLOTS + 2 * warp;
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) {
            t.wA[c][rb] = t.wB[c][rb] = make_uint2(0u, 0u);
            t.x0[c][rb] = t.x1[c][rb] = 0u;
            if (valid) {
                const uint8_t *wp = B + (size_t)(rowbase[rb] + r) * row_bytes + 32 * g0 + 8 * q;
                t.wA[c][rb] = __ldg(reinterpret_cast<const uint2 *>(wp));
                t.wB[c][rb] = __ldg(reinterpret_cast<const uint2 *>(wp + 32));
                const uint16_t *sp = ws + (size_t)(rowbase[rb] + 2 * q) * ng + g0;
                t.x0[c][rb] = __ldg(reinterpret_cast<const uint32_t *>(sp));
                t.x1[c][rb] = __ldg(reinterpret_cast<const uint32_t *>(sp + ng));
            }
        }
    }
}

// Activation fragments of this lane for every chunk (the same for all tiles of a stage).
template <bool HALF, int NCH>
struct SweepActs {
    AFrag<HALF> fA[NCH], fB[NCH];
};

template <bool HALF, int NCH>
__device__ __forceinline__ void sweep_acts_load(SweepActs<HALF, NCH> &a, const int8_t *A, const int32_t *asum, int K,
                                                int W) {
    const int ng = K / BM_GROUP;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = lane >> 2, q = lane & 3;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        load_afrag_cg<HALF>(a.fA[c], A, K, asum, W, ng, c * BM_SLOTS + 2 * warp, r, q);
        load_afrag_cg<HALF>(a.fB[c], A, K, asum, W, ng, c * BM_SLOTS + 2 * warp + 1, r, q);
    }
}

// MMAs of one tile, same work split as t2_gemv_mma_kernel: warp w owns scale slots 2w and 2w+1, lane
// (r, q) feeds tokens r / r+8 and receives rows 2q / 2q+1.  Leaves the per-warp partial sums in `part`
// ([warp][token][R+8]); the caller combines them after the barrier inside.
template <int RB, bool HALF, int NCH>
__device__ __forceinline__ void sweep_tile_compute(const SweepTile<RB, NCH> &t, const SweepActs<HALF, NCH> &a,
                                                   float *part) {
    constexpr int R = 8 * RB, RP = R + 8, WROWS = HALF ? 8 : 16;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = lane >> 2, q = lane & 3;
    float acc[RB][2][4];
#pragma unroll
    for (int rb = 0; rb < RB; ++rb)
#pragma unroll
        for (int sl = 0; sl < 2; ++sl)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[rb][sl][e] = 0.0f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) {
            const uint32_t x0 = t.x0[c][rb], x1 = t.x1[c][rb];
            mma_group_step<HALF, false>(a.fA[c], t.wA[c][rb], __uint_as_float(x0 << 16), __uint_as_float(x1 << 16),
                                        acc[rb][0], nullptr, nullptr, 0);
            mma_group_step<HALF, false>(a.fB[c], t.wB[c][rb], __uint_as_float(x0 & 0xffff0000u),
                                        __uint_as_float(x1 & 0xffff0000u), acc[rb][1], nullptr, nullptr, 0);
        }
    }
    float *pw = part + warp * WROWS * RP;
#pragma unroll
    for (int rb = 0; rb < RB; ++rb) {
        const int row0 = rb * 8 + 2 * q;
        *reinterpret_cast<float2 *>(&pw[r * RP + row0]) =
            make_float2(acc[rb][0][0] + acc[rb][1][0], acc[rb][0][1] + acc[rb][1][1]);
        if (!HALF)
            *reinterpret_cast<float2 *>(&pw[(r + 8) * RP + row0]) =
                make_float2(acc[rb][0][2] + acc[rb][1][2], acc[rb][0][3] + acc[rb][1][3]);
    }
    __syncthreads();
}

// Remaining tree levels and the reciprocal multiply for token m, tile rows 4*rq .. 4*rq+3.
template <int RB, bool HALF>
__device__ __forceinline__ void sweep_gemv_combine(const float *part, const float *invs, int m, int rq, float (&y)[4]) {
    constexpr int R = 8 * RB, RP = R + 8, WROWS = HALF ? 8 : 16;
    float4 v[kGemvWarps];
#pragma unroll
    for (int w = 0; w < kGemvWarps; ++w) v[w] = *reinterpret_cast<const float4 *>(&part[(w * WROWS + m) * RP + 4 * rq]);
    const float is = invs[m];
#define BM_TREE(F) (((v[0].F + v[1].F) + (v[2].F + v[3].F)) + ((v[4].F + v[5].F) + (v[6].F + v[7].F))) * is
    y[0] = BM_TREE(x); y[1] = BM_TREE(y); y[2] = BM_TREE(z); y[3] = BM_TREE(w);
#undef BM_TREE
}

__device__ __forceinline__ void store_bf16x4(uint16_t *dst, const float (&y)[4]) {
    const uint32_t lo = (uint32_t)bm_f32_to_bf16(y[0]) | ((uint32_t)bm_f32_to_bf16(y[1]) << 16);
    const uint32_t hi = (uint32_t)bm_f32_to_bf16(y[2]) | ((uint32_t)bm_f32_to_bf16(y[3]) << 16);
    *reinterpret_cast<uint2 *>(dst) = make_uint2(lo, hi);
}

// Plain projection: C[m, n] bf16 for a matrix of N rows cut into tiles of 8*RB consecutive rows, at
// most MAXT tiles per CTA (the host checks N / (8*RB) <= MAXT * gridDim.x).  Every global read of the
// stage is issued before the first result is used.
template <int RB, bool HALF, int NCH, int MAXT>
__device__ __noinline__ void sweep_gemv_plain(const uint8_t *B, const uint16_t *ws, int N, int K, const int8_t *A,
                                                 const int32_t *asum, const float *s, int W, uint16_t *C, int ldc,
                                                 float *part, float *invs) {
    constexpr int R = 8 * RB;
    const int ntiles = N / R;
    SweepTile<RB, NCH> tile[MAXT];
#pragma unroll
    for (int i = 0; i < MAXT; ++i) {
        const int t = blockIdx.x + i * gridDim.x;
        int rowbase[RB];
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) rowbase[rb] = t * R + 8 * rb;
        sweep_tile_load<RB, NCH>(tile[i], B, ws, K, rowbase, t < ntiles);
    }
    if ((int)blockIdx.x >= ntiles) return;                // CTA-uniform: no tile, no barrier below
    SweepActs<HALF, NCH> acts;
    sweep_acts_load<HALF, NCH>(acts, A, asum, K, W);
    if (threadIdx.x < 16) invs[threadIdx.x] = threadIdx.x < W ? 1.0f / __ldcg(s + threadIdx.x) : 0.0f;
#pragma unroll
    for (int i = 0; i < MAXT; ++i) {
        const int t = blockIdx.x + i * gridDim.x;
        if (t >= ntiles) break;                           // CTA-uniform
        sweep_tile_compute<RB, HALF, NCH>(tile[i], acts, part);
        for (int o = threadIdx.x; o < W * (R / 4); o += kSweepThreads) {
            const int m = o / (R / 4), rq = o - m * (R / 4);
            float y[4];
            sweep_gemv_combine<RB, HALF>(part, invs, m, rq, y);
            store_bf16x4(C + (size_t)m * ldc + t * R + 4 * rq, y);
        }
        __syncthreads();
    }
}

// gate|up projection with SiLU(gate) * up in the epilogue.  Tile t pairs gate rows
// [16t, 16t+16) with up rows [F + 16t, F + 16t + 16) of the merged [2F, K] matrix, so the CTA holds
// both factors of 16 columns of `inner`.  Also folds |inner| into the per-row absmax.
template <bool HALF, int MAXT>
__device__ __noinline__ void sweep_gemv_gate_up(const SweepParams &p, const SweepLayer &L, float *part, float *invs,
                                                   unsigned int *amax_s) {
    const int F = p.ffn, W = p.M, ntiles = F / 16;
    SweepTile<4, 1> tile[MAXT];
#pragma unroll
    for (int i = 0; i < MAXT; ++i) {
        const int t = blockIdx.x + i * gridDim.x;
        const int rowbase[4] = {16 * t, 16 * t + 8, F + 16 * t, F + 16 * t + 8};
        sweep_tile_load<4, 1>(tile[i], L.wgu, L.wgu_s, p.dim, rowbase, t < ntiles);
    }
    if ((int)blockIdx.x >= ntiles) return;
    SweepActs<HALF, 1> acts;
    sweep_acts_load<HALF, 1>(acts, p.xq, p.xsum, p.dim, W);
    if (threadIdx.x < 16) {
        invs[threadIdx.x] = threadIdx.x < W ? 1.0f / __ldcg(p.xs + threadIdx.x) : 0.0f;
        amax_s[threadIdx.x] = 0u;
    }
#pragma unroll
    for (int i = 0; i < MAXT; ++i) {
        const int t = blockIdx.x + i * gridDim.x;
        if (t >= ntiles) break;
        sweep_tile_compute<4, HALF, 1>(tile[i], acts, part);
        for (int o = threadIdx.x; o < W * 4; o += kSweepThreads) {
            const int m = o >> 2, rq = o & 3;
            float g[4], u[4], v[4];
            sweep_gemv_combine<4, HALF>(part, invs, m, rq, g);
            sweep_gemv_combine<4, HALF>(part, invs, m, rq + 4, u);
            float amax = 0.0f;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                v[e] = bm_bf16_rn(bm_silu_bf16(bm_bf16_rn(g[e])) * bm_bf16_rn(u[e]));
                amax = fmaxf(amax, fabsf(v[e]));
            }
            store_bf16x4(p.inner + (size_t)m * F + 16 * t + 4 * rq, v);
            atomicMax(&amax_s[m], __float_as_uint(amax));
        }
        __syncthreads();
    }
    if (threadIdx.x < W && amax_s[threadIdx.x] != 0u) atomicMax(&p.inner_amax[threadIdx.x], amax_s[threadIdx.x]);
}

// ---- stage: quantisation of `inner` with the row absmax gathered by the previous stage -------
__device__ __noinline__ void sweep_quant_inner(const SweepParams &p) {
    const int F = p.ffn, units = F / 8, lane = threadIdx.x & 31;
    const QuantSink sink{nullptr, p.iq, p.isum};
    for (int base = blockIdx.x * kSweepThreads; base < p.M * units; base += gridDim.x * kSweepThreads) {
        const int u = base + threadIdx.x;                 // whole warps stay inside one row: units % 32 == 0
        const bool active = u < p.M * units;
        const int m = active ? u / units : 0, i = active ? u - m * units : 0;
        float v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        float s = 0.0f;
        if (active) {
            unpack8(ldcg4(p.inner + (size_t)m * F + 8 * i), v);
            s = bm_act_scale(__uint_as_float(__ldcg(p.inner_amax + m)));
            if (i == 0) p.is_[m] = s;
        }
        emit_codes(sink, (size_t)m * F, F, i, quant8(v, s), active, lane);
    }
}

// The merge of one row, out of line so that its registers are allotted on their own.
__device__ __noinline__ void sweep_merge_row(const AttnParams &ap, int m, int cache_len, unsigned char *dyn, float *l_s,
                                             float *red) {
    attn_merge_row(ap, m, cache_len, dyn, l_s, red);
}

__device__ __forceinline__ void sweep_stamp(const SweepParams &p, int layer, int slot) {
    if (p.timing != nullptr && layer == 1 && blockIdx.x == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        p.timing[slot] = t;
    }
}

// ---- stage: q/k norm + RoPE + KV append + attention chunks --------------------------------------
// rope_head_vector (verify_attn.cuh) with the table rows read from shared memory.
__device__ __forceinline__ void sweep_rope_vec(uint2 raw, uint2 wraw, const uint16_t *cos_row, const uint16_t *sin_row,
                                               float eps, int lane, float (&o)[4]) {
    rope_head_vector(raw, wraw, *reinterpret_cast<const uint2 *>(cos_row + 4 * lane),
                     *reinterpret_cast<const uint2 *>(sin_row + 4 * lane), eps, lane, o);
}

// Work items are (live chunk, kv head) pairs dealt round-robin to the CTAs.  The item that holds
// the rows of this replay computes their K (norm + RoPE) and V itself and appends them to the
// layer's planes; every item rotates the query vectors of its kv head itself (a few hundred
// elements), so no CTA waits for another inside the stage.  All global reads of an item (history
// rows, qkv rows) are issued before the first is used; the RoPE tables of the M positions sit in
// shared memory (`rope_s`: cos rows then sin rows, [M][128] bf16 each).
constexpr int kSweepVecBatch = 4;                 // head vectors a warp rotates per batch

template <int NQ>
__device__ __noinline__ void sweep_attention(const SweepParams &p, const SweepLayer &L, const AttnParams &ap,
                                                unsigned char *dyn, const uint16_t *rope_s, int cache_len, int n_pend,
                                                int role, int P) {
    const int G = p.H / p.Hkv, QV = G * p.M, heads = p.H + 2 * p.Hkv;
    const int n_hist = (cache_len + BM_ATTN_CHUNK - 1) / BM_ATTN_CHUNK;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = kSweepThreads / 32;
    uint16_t *Ks = reinterpret_cast<uint16_t *>(dyn);                    // [32][136]
    uint16_t *Vs = Ks + 32 * kKeyStride;                                  // [32][128]
    float *Qs = reinterpret_cast<float *>(Vs + 32 * 128);                 // [QV][128]
    float *Ps = Qs + (size_t)QV * 128;                                    // [QV][32]
    const uint16_t *cos_s = rope_s, *sin_s = rope_s + p.M * 128;
    const uint2 qw = *reinterpret_cast<const uint2 *>(L.qn + 4 * lane);
    const uint2 kw = *reinterpret_cast<const uint2 *>(L.kn + 4 * lane);
    for (int item = blockIdx.x; item < (n_hist + 1) * p.Hkv; item += gridDim.x) {
        const int jl = item / p.Hkv, hk = item - jl * p.Hkv;
        const bool fresh = jl == n_hist;
        const int j = fresh ? p.NC - 1 : jl;
        const int c0 = fresh ? p.sigma : j * BM_ATTN_CHUNK;
        const int cn = fresh ? p.M : min(BM_ATTN_CHUNK, cache_len - c0);
        // history rows: 512 16-byte pieces of K and of V over 256 threads
        uint4 kreg[2], vreg[2];
        if (!fresh) {
            const uint4 *kg = reinterpret_cast<const uint4 *>(L.k_base + ((size_t)hk * p.kv_rows + c0) * 128);
            const uint4 *vg = reinterpret_cast<const uint4 *>(L.v_base + ((size_t)hk * p.kv_rows + c0) * 128);
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int i = threadIdx.x + k * kSweepThreads;
                if (i < cn * 16) { kreg[k] = kg[i]; vreg[k] = vg[i]; }
            }
        }
        // rows of this replay: K through norm + RoPE, V as it is; to shared memory and to the planes
        if (fresh) {
            for (int m0 = warp; m0 < p.M; m0 += nwarps * kSweepVecBatch) {
                uint2 kraw[kSweepVecBatch], vraw[kSweepVecBatch];
#pragma unroll
                for (int k = 0; k < kSweepVecBatch; ++k) {
                    const int m = m0 + k * nwarps;
                    if (m < p.M) {
                        kraw[k] = ldcg2(p.xqkv + ((size_t)m * heads + p.H + hk) * 128 + 4 * lane);
                        vraw[k] = ldcg2(p.xqkv + ((size_t)m * heads + p.H + p.Hkv + hk) * 128 + 4 * lane);
                    }
                }
#pragma unroll
                for (int k = 0; k < kSweepVecBatch; ++k) {
                    const int m = m0 + k * nwarps;
                    if (m >= p.M) break;                       // warp-uniform
                    float o[4];
                    sweep_rope_vec(kraw[k], kw, cos_s + m * 128, sin_s + m * 128, p.eps, lane, o);
                    const uint2 kbits = make_uint2(
                        (uint32_t)bm_f32_to_bf16(o[0]) | ((uint32_t)bm_f32_to_bf16(o[1]) << 16),
                        (uint32_t)bm_f32_to_bf16(o[2]) | ((uint32_t)bm_f32_to_bf16(o[3]) << 16));
                    *reinterpret_cast<uint2 *>(Ks + m * kKeyStride + 4 * lane) = kbits;
                    *reinterpret_cast<uint2 *>(Vs + m * 128 + 4 * lane) = vraw[k];
                    const size_t row = ((size_t)hk * p.kv_rows + p.sigma + m) * 128 + 4 * lane;
                    *reinterpret_cast<uint2 *>(L.k_base + row) = kbits;
                    *reinterpret_cast<uint2 *>(L.v_base + row) = vraw[k];
                }
            }
        }
        // query vectors of this kv head
        for (int v0 = warp; v0 < QV; v0 += nwarps * kSweepVecBatch) {
            uint2 qraw[kSweepVecBatch];
#pragma unroll
            for (int k = 0; k < kSweepVecBatch; ++k) {
                const int qv = v0 + k * nwarps;
                if (qv < QV) {
                    const int g = qv / p.M, m = qv - g * p.M;
                    qraw[k] = ldcg2(p.xqkv + ((size_t)m * heads + hk * G + g) * 128 + 4 * lane);
                }
            }
#pragma unroll
            for (int k = 0; k < kSweepVecBatch; ++k) {
                const int qv = v0 + k * nwarps;
                if (qv >= QV) break;                           // warp-uniform
                const int g = qv / p.M, m = qv - g * p.M;
                float o[4];
                sweep_rope_vec(qraw[k], qw, cos_s + m * 128, sin_s + m * 128, p.eps, lane, o);
                *reinterpret_cast<float4 *>(Qs + (size_t)qv * 128 + 4 * lane) =
                    make_float4(bm_bf16_rn(o[0]), bm_bf16_rn(o[1]), bm_bf16_rn(o[2]), bm_bf16_rn(o[3]));
            }
        }
        if (!fresh) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int i = threadIdx.x + k * kSweepThreads;
                if (i < cn * 16) {
                    *reinterpret_cast<uint4 *>(Ks + (i >> 4) * kKeyStride + 8 * (i & 15)) = kreg[k];
                    reinterpret_cast<uint4 *>(Vs)[i] = vreg[k];
                }
            }
        }
        __syncthreads();
        for (int q0 = warp * NQ; q0 < QV; q0 += nwarps * NQ)
            attn_chunk_pass<NQ>(ap, Ks, Vs, Qs, Ps, q0, QV, G, hk, j, c0, cn, lane, role, cache_len, n_pend, P);
        __syncthreads();
    }
}

// ---- the kernel -----------------------------------------------------------------------------------
__global__ void __launch_bounds__(kSweepThreads, 1) decode_sweep_kernel(const SweepParams p) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ float sh[32];
    __shared__ float invs[16];
    __shared__ unsigned int amax_s[16];
    __shared__ float l_s[kMergeMaxHeads];
    __shared__ float red[kSweepThreads / 32];
    __shared__ int sh_flag;
    __shared__ __align__(16) uint16_t rope_s[2 * 16 * 128];   // cos rows, then sin rows, of the M positions
    SweepSync st{0u, true};
    for (int i = threadIdx.x; i < 2 * p.M * 16; i += kSweepThreads) {
        const int tab = i / (p.M * 16), rem = i - tab * (p.M * 16), m = rem >> 4, u = rem & 15;
        const uint16_t *src = (tab == 0 ? p.cos_t : p.sin_t) + (size_t)p.positions[m] * 128;
        reinterpret_cast<uint4 *>(rope_s + (size_t)tab * p.M * 128 + m * 128)[u] = reinterpret_cast<const uint4 *>(src)[u];
    }
    __syncthreads();
    const int cache_len = p.state->cache_len, n_pend = p.state->n_pend, role = p.state->role, P = p.state->P;
    const bool half = p.M <= 8;
    const int qkv_dim = (p.H + 2 * p.Hkv) * 128, q_dim = p.H * 128;
    const int G = p.H / p.Hkv, QV = G * p.M, nq = attn_nq(QV);
    float *part = reinterpret_cast<float *>(dyn);

    AttnParams ap;
    ap.q = nullptr;
    ap.k_base = ap.v_base = nullptr;
    ap.state = p.state;
    ap.M = p.M; ap.H = p.H; ap.Hkv = p.Hkv; ap.kv_rows = p.kv_rows; ap.sigma = p.sigma; ap.NC = p.NC;
    ap.ctr = nullptr; ap.amax = nullptr;
    ap.pm = p.pm; ap.pl = p.pl; ap.po = p.po;
    ap.att = nullptr;
    ap.q_out = QuantSink{nullptr, p.attq, p.attsum};
    ap.s_out = p.atts;
    ap.pdl = 0;

    for (int l = 0; l < p.n_layers; ++l) {
        const SweepLayer L = p.layers[l];
        sweep_stamp(p, l, 0);
        // 1. (embedding | residual add) + RMSNorm + quant
        if (st.alive) {
            if ((int)blockIdx.x < p.M) {
                const int m = blockIdx.x;
                if (l == 0)
                    sweep_norm_row(p, m, p.embed + (size_t)p.tokens[m] * p.dim, false, false, L.ln1, sh);
                else
                    sweep_norm_row(p, m, p.ffn_out + (size_t)m * p.dim, true, true, L.ln1, sh);
            }
            if (blockIdx.x == 0 && threadIdx.x < p.M) p.inner_amax[threadIdx.x] = 0u;
            if ((int)blockIdx.x < qkv_dim / 32) sweep_prefetch(L.wqkv + (size_t)blockIdx.x * 32 * (p.dim / 4), (size_t)32 * (p.dim / 4));
        }
        sweep_stamp(p, l, 1);
        sweep_grid_sync(p, st, &sh_flag);
        sweep_stamp(p, l, 2);
        // 2. qkv projection
        if (st.alive) {
            if (half) sweep_gemv_plain<4, true, 1, 1>(L.wqkv, L.wqkv_s, qkv_dim, p.dim, p.xq, p.xsum, p.xs, p.M, p.xqkv, qkv_dim, part, invs);
            else sweep_gemv_plain<4, false, 1, 1>(L.wqkv, L.wqkv_s, qkv_dim, p.dim, p.xq, p.xsum, p.xs, p.M, p.xqkv, qkv_dim, part, invs);
            if ((int)blockIdx.x < p.dim / 16) sweep_prefetch(L.wo + (size_t)blockIdx.x * 16 * (q_dim / 4), (size_t)16 * (q_dim / 4));
        }
        sweep_stamp(p, l, 3);
        sweep_grid_sync(p, st, &sh_flag);
        sweep_stamp(p, l, 4);
        // 3. q/k norm + RoPE + KV append + attention chunks
        if (st.alive) {
            if (nq == 2) sweep_attention<2>(p, L, ap, dyn, rope_s, cache_len, n_pend, role, P);
            else if (nq == 4) sweep_attention<4>(p, L, ap, dyn, rope_s, cache_len, n_pend, role, P);
            else sweep_attention<8>(p, L, ap, dyn, rope_s, cache_len, n_pend, role, P);
        }
        sweep_stamp(p, l, 5);
        sweep_grid_sync(p, st, &sh_flag);
        sweep_stamp(p, l, 6);
        // 4. chunk merge + quant of the attention rows
        if (st.alive) {
            if ((int)blockIdx.x < p.M) sweep_merge_row(ap, blockIdx.x, cache_len, dyn, l_s, red);
            for (int t = blockIdx.x; t < p.ffn / 16; t += gridDim.x) {   // gate|up tiles of this CTA
                sweep_prefetch(L.wgu + (size_t)t * 16 * (p.dim / 4), (size_t)16 * (p.dim / 4));
                sweep_prefetch(L.wgu + (size_t)(p.ffn + t * 16) * (p.dim / 4), (size_t)16 * (p.dim / 4));
            }
        }
        sweep_stamp(p, l, 7);
        sweep_grid_sync(p, st, &sh_flag);
        sweep_stamp(p, l, 8);
        // 5. o projection
        if (st.alive) {
            if (half) sweep_gemv_plain<2, true, 1, 1>(L.wo, L.wo_s, p.dim, q_dim, p.attq, p.attsum, p.atts, p.M, p.attn_out, p.dim, part, invs);
            else sweep_gemv_plain<2, false, 1, 1>(L.wo, L.wo_s, p.dim, q_dim, p.attq, p.attsum, p.atts, p.M, p.attn_out, p.dim, part, invs);
        }
        sweep_stamp(p, l, 9);
        sweep_grid_sync(p, st, &sh_flag);
        sweep_stamp(p, l, 10);
        // 6. residual add + RMSNorm + quant
        if (st.alive) {
            if ((int)blockIdx.x < p.M) sweep_norm_row(p, blockIdx.x, p.attn_out + (size_t)blockIdx.x * p.dim, true, true, L.ln2, sh);
            if ((int)blockIdx.x < p.dim / 16) sweep_prefetch(L.wdown + (size_t)blockIdx.x * 16 * (p.ffn / 4), (size_t)16 * (p.ffn / 4));
        }
        sweep_stamp(p, l, 11);
        sweep_grid_sync(p, st, &sh_flag);
        sweep_stamp(p, l, 12);
        // 7. gate|up projection + SiLU(gate) * up
        if (st.alive) {
            if (half) sweep_gemv_gate_up<true, 3>(p, L, part, invs, amax_s);
            else sweep_gemv_gate_up<false, 3>(p, L, part, invs, amax_s);
        }
        sweep_stamp(p, l, 13);
        sweep_grid_sync(p, st, &sh_flag);
        sweep_stamp(p, l, 14);
        // 8. quantisation of the down-projection input
        if (st.alive) sweep_quant_inner(p);
        sweep_stamp(p, l, 15);
        sweep_grid_sync(p, st, &sh_flag);
        sweep_stamp(p, l, 16);
        // 9. down projection
        if (st.alive) {
            if (half) sweep_gemv_plain<2, true, 3, 1>(L.wdown, L.wdown_s, p.dim, p.ffn, p.iq, p.isum, p.is_, p.M, p.ffn_out, p.dim, part, invs);
            else sweep_gemv_plain<2, false, 3, 1>(L.wdown, L.wdown_s, p.dim, p.ffn, p.iq, p.isum, p.is_, p.M, p.ffn_out, p.dim, part, invs);
        }
        sweep_stamp(p, l, 17);
        sweep_grid_sync(p, st, &sh_flag);
        sweep_stamp(p, l, 18);
    }
}

}  // namespace bm
