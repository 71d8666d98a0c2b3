// Packed T2-g128 product for MANY rows at once (a prompt): C[T, N] = ((A x ternary(B)) per-group
// scaled) / s, every row bit-identical to what the decode GEMV (t2_gemv.cuh) gives that row alone.
//
// Replaces, for the prompt forward, the dense fallback of T2LinearKernel.forward
// (src/bonsai_sft/gpu/model.py:650-656: unpack the layer to bf16, fake-quantise, cuBLAS) behind
// forward_sdlm_prefill (model.py:1306-1340).  Here the prompt goes through the packed integer path:
// every weight byte is read once per 32 prompt rows instead of once per row block of a GEMV launch,
// and nothing dense is ever materialised.
//
// This IS a contraction (a weight is reused by every prompt row), so it runs on the tensor cores:
// mma.sync.m16n8k32 with 16 weight rows as the M dimension (u8 codes as A), 8 prompt rows as the N
// dimension (s8 activations as B); four MMAs cover a 128-group with -2 * sum(a) as the first C
// operand, so the int32 fragment is the exact group sum.  The 2-bit -> 8-bit expansion happens in
// registers, once per group and warp, and is reused by the 32 prompt rows of the tile.
//
// fp32 order (the GEMV's, see the header of t2_gemv.cuh): group g -> slot g % 16, slot = fma(G,
// scale, slot) in ascending g, the 16 slots summed as a butterfly tree, times 1/s.  A wide tile cannot
// hold 16 slot accumulators per output, so the groups are visited SLOT BY SLOT (s, s+16, s+32, ...:
// one accumulator), and a finished slot is folded into a binary-counter tree (4 registers per output)
// whose additions are exactly the butterfly's.
//
// CTA = 8 warps = 128 weight rows x 32 prompt rows; the slots are staged through shared memory in
// batches (activations [32 rows][groups][128 B], codes [128 rows][groups][32 B], scales, group sums),
// 16-byte asynchronous copies, two CTAs per SM so that one computes while the other loads.
#pragma once

#include "bm_common.cuh"
#include "t2_gemv_rowwarp.cuh"

namespace bm {

constexpr int kWideThreads = 256;
constexpr int kWideRows = 128;          // weight rows per CTA (16 per warp)
constexpr int kWideTokens = 32;         // prompt rows per CTA (4 MMA column blocks)
constexpr int kWideMaxStageGroups = 12; // groups staged at once (about 100 KB)

struct WideParams {
    const int8_t *A;        // [T, K] GEMV-ready INT8 rows
    const int32_t *asum;    // [T, K/128]
    const float *s;         // [T]
    const uint8_t *B;       // [N, K/4]
    const uint16_t *ws;     // [N, K/128] bf16
    uint16_t *C;            // [T, ldc] bf16
    int T, N, K, ldc, pdl;
};

struct WideSmem {
    int act_stride, w_stride, act_off, w_off, sc_off, asum_off, total;
};

// Layout for a stage of `ngs` groups.  Strides are padded so that the fragment reads are free of bank
// conflicts: activation rows (16-byte reads of 8 rows x 4 quarters) want an odd number of 16-byte units,
// code rows (8-byte reads of 4 rows x 4 quarters) want 32 mod 128 bytes.
__host__ __device__ inline WideSmem wide_smem_layout(int ngs) {
    WideSmem L;
    L.act_stride = ngs * 128 + 16;
    int ws = ngs * 32;
    ws += (32 - (ws % 128) + 128) % 128;
    L.w_stride = ws;
    L.act_off = 0;
    L.w_off = L.act_off + kWideTokens * L.act_stride;
    L.sc_off = L.w_off + kWideRows * L.w_stride;
    L.asum_off = L.sc_off + kWideRows * ngs * 2;
    L.asum_off = (L.asum_off + 15) & ~15;
    L.total = L.asum_off + kWideTokens * ngs * 4;
    return L;
}

// Slots per stage: the largest power of two whose groups (terms per slot = ceil(ng / 16)) fit.
__host__ __device__ inline int wide_slots_per_stage(int ng) {
    const int terms = (ng + BM_SLOTS - 1) / BM_SLOTS;
    int sb = BM_SLOTS;
    while (sb > 1 && sb * terms > kWideMaxStageGroups) sb >>= 1;
    return sb;
}

// Folds slot `s` (compile-time) into the binary-counter tree: level l holds the sum of a finished block
// of 2^l slots whose partner has not arrived yet; `left + right` with the earlier block on the left,
// which is the butterfly order ((s0+s1)+(s2+s3))+... of the GEMV.
template <int S>
__device__ __forceinline__ void wide_tree_push(float (&tree)[4], float v) {
    if (S & 1) { v = tree[0] + v; } else { tree[0] = v; return; }
    if (S & 2) { v = tree[1] + v; } else { tree[1] = v; return; }
    if (S & 4) { v = tree[2] + v; } else { tree[2] = v; return; }
    if (S & 8) { v = tree[3] + v; } else { tree[3] = v; return; }
    tree[3] = v;            // S == 15: the total
}

template <int S>
struct WideSlot {
    // One slot of the canonical order for this warp's 16 rows x 32 prompt rows: its groups are in the staged
    // batch at local indices li0, li0 + 1, ... (n_terms of them).
    static __device__ __forceinline__ void run(const unsigned char *act, const unsigned char *wts, const uint16_t *sc,
                                               const int *asum_s, int ngs, const WideSmem &L, int li0, int n_terms,
                                               int g, int q, float (&tree)[4][4][4]) {
        constexpr uint32_t M3 = 0x03030303u;
        float acc[4][4];
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[b][e] = 0.0f;
        for (int c = 0; c < n_terms; ++c) {
            const int li = li0 + c;
            const uint2 x = *reinterpret_cast<const uint2 *>(wts + (size_t)g * L.w_stride + li * 32 + 8 * q);
            const uint2 y = *reinterpret_cast<const uint2 *>(wts + (size_t)(g + 8) * L.w_stride + li * 32 + 8 * q);
            const float s0 = bf16_bits_to_f32(sc[g * ngs + li]), s8 = bf16_bits_to_f32(sc[(g + 8) * ngs + li]);
            uint32_t a[4][4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                a[t][0] = (x.x >> (2 * t)) & M3;
                a[t][1] = (y.x >> (2 * t)) & M3;
                a[t][2] = (x.y >> (2 * t)) & M3;
                a[t][3] = (y.y >> (2 * t)) & M3;
            }
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const unsigned char *ap = act + (size_t)(8 * b + g) * L.act_stride + li * 128 + 32 * q;
                const uint4 lo = *reinterpret_cast<const uint4 *>(ap), hi = *reinterpret_cast<const uint4 *>(ap + 16);
                const int c0 = kGroupSumBias - 2 * asum_s[(8 * b + 2 * q) * ngs + li], c1 = kGroupSumBias - 2 * asum_s[(8 * b + 2 * q + 1) * ngs + li];
                int d[4];
                mma_u8s8(d, a[0][0], a[0][1], a[0][2], a[0][3], lo.x, hi.x, c0, c1, c0, c1);
                mma_u8s8(d, a[1][0], a[1][1], a[1][2], a[1][3], lo.y, hi.y, d[0], d[1], d[2], d[3]);
                mma_u8s8(d, a[2][0], a[2][1], a[2][2], a[2][3], lo.z, hi.z, d[0], d[1], d[2], d[3]);
                mma_u8s8(d, a[3][0], a[3][1], a[3][2], a[3][3], lo.w, hi.w, d[0], d[1], d[2], d[3]);
                acc[b][0] = fmaf(group_sum_to_float(d[0]), s0, acc[b][0]);
                acc[b][1] = fmaf(group_sum_to_float(d[1]), s0, acc[b][1]);
                acc[b][2] = fmaf(group_sum_to_float(d[2]), s8, acc[b][2]);
                acc[b][3] = fmaf(group_sum_to_float(d[3]), s8, acc[b][3]);
            }
        }
#pragma unroll
        for (int b = 0; b < 4; ++b)
#pragma unroll
            for (int e = 0; e < 4; ++e) wide_tree_push<S>(tree[b][e], acc[b][e]);
    }
};

// grid (N / 128, ceil(T / 32)), 256 threads.  K % 128 == 0, N % 128 == 0.
__global__ void __launch_bounds__(kWideThreads, 2) t2_gemm_wide_kernel(const WideParams p) {
    extern __shared__ __align__(16) unsigned char wsm[];
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, q = lane & 3;
    const int ng = p.K / BM_GROUP;
    const int n0 = blockIdx.x * kWideRows, t0 = blockIdx.y * kWideTokens;
    const int SB = wide_slots_per_stage(ng);
    float tree[4][4][4];                     // [token block][fragment element][level]
#pragma unroll
    for (int b = 0; b < 4; ++b)
#pragma unroll
        for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int l = 0; l < 4; ++l) tree[b][e][l] = 0.0f;

    bool waited = !p.pdl;
    for (int s0 = 0; s0 < BM_SLOTS; s0 += SB) {
        // groups of this stage, slot-major: local index li <-> (slot s0 + i, term c) with group s0 + i + 16 c
        int ngs = 0;
        for (int i = 0; i < SB; ++i) ngs += (ng - (s0 + i) + BM_SLOTS - 1) / BM_SLOTS > 0 ? (ng - (s0 + i) + BM_SLOTS - 1) / BM_SLOTS : 0;
        const WideSmem L = wide_smem_layout(ngs > 0 ? ngs : 1);
        if (s0 > 0) __syncthreads();                          // everyone is done with the previous stage
        // local index -> group, slot-major (every thread keeps the short table in registers)
        int grp_of[kWideMaxStageGroups];
        {
            int li = 0;
            for (int i = 0; i < SB; ++i)
                for (int grp = s0 + i; grp < ng && li < kWideMaxStageGroups; grp += BM_SLOTS) grp_of[li++] = grp;
        }
        // weights first: they do not depend on the previous kernel in the stream.  Codes by 16-byte
        // asynchronous copies; the scales (2 bytes per row and group) are fetched into registers together
        // and stored afterwards, so that the stage costs one memory round trip, not one per group.
        for (int e = tid; e < ngs * kWideRows * 2; e += kWideThreads) {
            const int li = e / (kWideRows * 2), j2 = e - li * (kWideRows * 2), r = j2 >> 1, h = j2 & 1;
            cp_async16(wsm + L.w_off + (size_t)r * L.w_stride + li * 32 + 16 * h,
                       p.B + (size_t)(n0 + r) * (p.K / 4) + grp_of[li] * 32 + 16 * h);
        }
        constexpr int kScPer = (kWideMaxStageGroups * kWideRows + kWideThreads - 1) / kWideThreads;   // 6
        uint16_t scv[kScPer];
#pragma unroll
        for (int k = 0; k < kScPer; ++k) {
            const int e = tid + k * kWideThreads;
            if (e < ngs * kWideRows) {
                const int li = e / kWideRows, r = e - li * kWideRows;
                scv[k] = p.ws[(size_t)(n0 + r) * ng + grp_of[li]];
            }
        }
        if (!waited) { pdl_wait(); waited = true; }
        for (int e = tid; e < ngs * kWideTokens * 8; e += kWideThreads) {
            const int li = e / (kWideTokens * 8), j2 = e - li * (kWideTokens * 8), r = j2 >> 3, h = j2 & 7;
            unsigned char *dst = wsm + L.act_off + (size_t)r * L.act_stride + li * 128 + 16 * h;
            if (t0 + r < p.T) cp_async16(dst, p.A + (size_t)(t0 + r) * p.K + grp_of[li] * 128 + 16 * h);
            else *reinterpret_cast<uint4 *>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
        constexpr int kAsPer = (kWideMaxStageGroups * kWideTokens + kWideThreads - 1) / kWideThreads;  // 2
        int asv[kAsPer];
#pragma unroll
        for (int k = 0; k < kAsPer; ++k) {
            const int e = tid + k * kWideThreads;
            asv[k] = 0;
            if (e < ngs * kWideTokens) {
                const int li = e / kWideTokens, r = e - li * kWideTokens;
                if (t0 + r < p.T) asv[k] = p.asum[(size_t)(t0 + r) * ng + grp_of[li]];
            }
        }
#pragma unroll
        for (int k = 0; k < kScPer; ++k) {
            const int e = tid + k * kWideThreads;
            if (e < ngs * kWideRows) {
                const int li = e / kWideRows, r = e - li * kWideRows;
                reinterpret_cast<uint16_t *>(wsm + L.sc_off)[r * ngs + li] = scv[k];
            }
        }
#pragma unroll
        for (int k = 0; k < kAsPer; ++k) {
            const int e = tid + k * kWideThreads;
            if (e < ngs * kWideTokens) {
                const int li = e / kWideTokens, r = e - li * kWideTokens;
                reinterpret_cast<int *>(wsm + L.asum_off)[r * ngs + li] = asv[k];
            }
        }
        cp_async_wait_all();
        __syncthreads();
        const unsigned char *act = wsm + L.act_off;
        const unsigned char *wts = wsm + L.w_off + (size_t)(16 * warp) * L.w_stride;
        const uint16_t *sc = reinterpret_cast<const uint16_t *>(wsm + L.sc_off) + (size_t)(16 * warp) * ngs;
        const int *asum_s = reinterpret_cast<const int *>(wsm + L.asum_off);
        int li = 0;
        // the slots of this stage in ascending order; the slot number must be a compile-time constant for the tree
#define BM_WIDE_SLOT(S_)                                                                                       \
        if (S_ >= s0 && S_ < s0 + SB) {                                                                        \
            const int nt = (ng - S_ + BM_SLOTS - 1) / BM_SLOTS > 0 ? (ng - S_ + BM_SLOTS - 1) / BM_SLOTS : 0;   \
            WideSlot<S_>::run(act, wts, sc, asum_s, ngs, L, li, nt, g, q, tree);                               \
            li += nt;                                                                                          \
        }
        BM_WIDE_SLOT(0) BM_WIDE_SLOT(1) BM_WIDE_SLOT(2) BM_WIDE_SLOT(3) BM_WIDE_SLOT(4) BM_WIDE_SLOT(5) BM_WIDE_SLOT(6)
        BM_WIDE_SLOT(7) BM_WIDE_SLOT(8) BM_WIDE_SLOT(9) BM_WIDE_SLOT(10) BM_WIDE_SLOT(11) BM_WIDE_SLOT(12)
        BM_WIDE_SLOT(13) BM_WIDE_SLOT(14) BM_WIDE_SLOT(15)
#undef BM_WIDE_SLOT
    }
    // tree[..][3] holds the sum of the 16 slots; times 1/s of the prompt row, to bf16
    const int row = n0 + 16 * warp + g;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const int ta = t0 + 8 * b + 2 * q, tb = ta + 1;
        if (ta < p.T) {
            const float is = 1.0f / p.s[ta];
            p.C[(size_t)ta * p.ldc + row] = bm_f32_to_bf16(tree[b][0][3] * is);
            p.C[(size_t)ta * p.ldc + row + 8] = bm_f32_to_bf16(tree[b][2][3] * is);
        }
        if (tb < p.T) {
            const float is = 1.0f / p.s[tb];
            p.C[(size_t)tb * p.ldc + row] = bm_f32_to_bf16(tree[b][1][3] * is);
            p.C[(size_t)tb * p.ldc + row + 8] = bm_f32_to_bf16(tree[b][3][3] * is);
        }
    }
}

}  // namespace bm
