// Packed T2-g128 GEMV for W <= 8 tokens and many output rows: every warp streams its own
// rows, nothing in the main loop synchronises the CTA.
//
// Same arithmetic and fp32 order as t2_gemv.cuh (see the header comment there); only the
// work split differs.  The profile of the tile-cooperative kernel on the 151936-row head
// showed warps waiting at the per-tile CTA barrier five times longer than they issued
// (issue slots 27 % busy, DRAM 20 %), so here:
//   * a warp owns blocks of 16 consecutive output rows and walks each block in panels of
//     512 k (128 packed bytes per row, four scale groups);
//   * the panel [16 rows x 128 B] arrives in the warp's private shared-memory ring by one
//     tiled TMA copy (cp.async.bulk.tensor.2d) with the 128-byte swizzle, which makes the
//     per-lane 8-byte reads of 8 rows at one column conflict-free without padding rows;
//     lane 0 of the warp issues the copies, up to `stages` panels ahead, and the warp waits
//     on its own mbarrier only;
//   * the MMA roles are swapped with respect to the cooperative kernel: the 16 weight rows
//     are the M dimension of mma.sync.m16n8k32 (u8 codes as A), up to 8 tokens the N
//     dimension (s8 activations as B), so one instruction covers 512 weights and the
//     int32 fragment is the exact group sum of 16 rows x 8 tokens;
//   * the 16 scale slots of the canonical order live in registers (64 accumulators per
//     lane), the tree over them is evaluated in registers, and the scales come straight
//     from global memory one panel ahead.
// K split (KS = 2 or 4, for matrices with too few rows to give every warp a block, e.g. the shard of a
// layer split over GPUs): a team of KS warps shares a block of 16 rows.  The canonical order survives
// the split because the panels are dealt by SLOT, not by range: panel p feeds slots 4(p % 4) .. +3, so
// warp ks of a pair takes the panels with (p % 4) / 2 == ks (slots 0-7 or 8-15), warp ks of a quad those
// with p % 4 == ks (four slots); every slot's chain stays with one warp, each warp sums its slots with
// its part of the butterfly tree, and warp 0 of the team adds the KS partial sums in tree order.
// Requires W <= 8, K % 512 == 0 (K % 2048 == 0 when split), N % 16 == 0.  One CTA of 16 warps per SM.
#pragma once

#include <cuda.h>

#include "bm_common.cuh"
#include "t2_gemv.cuh"

namespace bm {

constexpr int kRwMaxWarps = 16;
constexpr int kRwRows = 16;                 // output rows per block
constexpr int kRwPanelBytes = 128;          // packed bytes per row per panel (512 k, 4 groups)
constexpr int kRwStageBytes = kRwRows * kRwPanelBytes;
constexpr int kRwMaxStages = 8;
constexpr int kRwSmemBudget = 226 * 1024;   // 1 KB of the 227 KB is run-time alignment slack

enum : int { kErrRowWarpWaitTimeout = 2 };  // a weight panel never arrived

struct RowWarpParams {
    CUtensorMap tmap;       // uint8 [N, K/4], box [16 rows, 128 bytes], 128-byte swizzle
    GemvParams g;
};

struct RowWarpSmem {
    int invs_off, nb_off, act_off, act_stride, asum_off, xch_off, stage_off, stages, total;
};

// `pb` panels (1, 2 or 4) make one stage: they are requested back to back and complete on one
// mbarrier, so that DRAM sees pb * 128 contiguous bytes of each of the 16 rows at a time.
__host__ __device__ inline RowWarpSmem rowwarp_smem_layout(int W, int K, int warps, int pb) {
    RowWarpSmem L;
    const int ng = K / BM_GROUP;
    int off = kRwMaxWarps * kRwMaxStages * 8;         // mbarriers
    L.invs_off = off;
    off += 64;
    L.nb_off = off;                                   // int32 [ng][4][4]: C operand quads, -2 * group sum of A
    off += ng * 16 * 4;
    L.asum_off = off;                                 // int32 [8][ng] (natural-order staging)
    off += 8 * ng * 4;
    L.act_stride = K + kActPad;
    L.act_off = off;
    off += (W + 1) * L.act_stride;                    // row W is all zero (lanes without a token)
    off = (off + 15) & ~15;
    L.xch_off = off;                                  // K split: partial sums of the team's other warps, two buffers,
    off += 2 * kRwMaxWarps * 32 * 4 * 4 + 64;         // then one give-up flag per team
    off = (off + 1023) & ~1023;                       // the swizzle pattern is address based
    L.stage_off = off;
    int stages = (kRwSmemBudget - off) / (warps * pb * kRwStageBytes);
    if (stages > kRwMaxStages) stages = kRwMaxStages;
    L.stages = stages;
    L.total = off + (stages > 0 ? stages : 0) * warps * pb * kRwStageBytes;
    return L;
}

__device__ __forceinline__ void tma_panel_g2s(void *dst_smem, const CUtensorMap *tmap, int x, int y,
                                              uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst_smem)), "l"(tmap), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void mma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, int c0, int c1, int c2, int c3) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
}

// NTOK = 1: W == 1, only token 0 of a lane's token pair exists (half the accumulators).
// NTOK = 2: W <= 8.
// 4x4 byte transpose of a 16-run: out[4t+e] = in[4e+t] (the GEMV-ready order).
__device__ __forceinline__ uint4 transpose_run16(uint4 x) {
    const uint32_t lo01 = __byte_perm(x.x, x.y, 0x5140), lo23 = __byte_perm(x.z, x.w, 0x5140);
    const uint32_t hi01 = __byte_perm(x.x, x.y, 0x7362), hi23 = __byte_perm(x.z, x.w, 0x7362);
    return make_uint4(__byte_perm(lo01, lo23, 0x5410), __byte_perm(lo01, lo23, 0x7632),
                      __byte_perm(hi01, hi23, 0x5410), __byte_perm(hi01, hi23, 0x7632));
}

template <int NTOK, int PB, bool EMIT_G, int KS = 1>
__global__ void __launch_bounds__(kRwMaxWarps * 32, 1) t2_gemv_rowwarp_kernel(const __grid_constant__ RowWarpParams P) {
    static_assert(KS == 1 || (KS == 2 && PB == 2) || (KS == 4 && PB == 1), "panels per stage follow the split");
    extern __shared__ __align__(1024) unsigned char rw_smem[];
    unsigned char *const smem = rw_smem;
    const int THREADS = (int)blockDim.x, WARPS = THREADS >> 5;
    constexpr int kStage = PB * kRwStageBytes;
    constexpr int NA = 2 * NTOK;                      // accumulators per slot: rows g, g+8 x tokens
    constexpr int IL = 1;                             // groups issued in lock-step (measured: 1 is as fast as 4)
    const GemvParams &p = P.g;
    const int ng = p.K / BM_GROUP;
    const int panels = p.K / 512;
    const RowWarpSmem L = rowwarp_smem_layout(p.W, p.K, WARPS, PB);
    const int S = L.stages;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, q = lane & 3;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem) + warp * kRwMaxStages;
    // The swizzle pattern follows shared-memory address bits 4..9: align the rings at run time
    // (the launch asks for 1 KB more than the layout's total).
    unsigned char *ring0 = smem + L.stage_off;
    ring0 += (1024u - (smem_u32(ring0) & 1023u)) & 1023u;
    unsigned char *ring = ring0 + warp * S * kStage;

    // blocks of this warp's team: b = first + t * stride
    const int n_blocks = p.N / kRwRows;
    const int team = warp / KS, ks = warp % KS, TEAMS = WARPS / KS;
    const int first = team * (int)gridDim.x + (int)blockIdx.x;
    const int stride = TEAMS * (int)gridDim.x;
    const int my_blocks = first < n_blocks ? (n_blocks - first + stride - 1) / stride : 0;

    if (lane == 0) {
        for (int i = 0; i < S; ++i) mbar_init(&bars[i], 1);
        mbar_fence_init();
    }
    __syncwarp();
    // Producer state (lane 0): next stage to fill, next panel / row of the matrix, stages left.
    // this warp's panels: all of them (KS == 1), the pairs (4i + 2ks, 4i + 2ks + 1), or the singles 4i + ks
    const int pan0 = KS == 1 ? 0 : (KS == 2 ? 2 * ks : ks), pan_step = KS == 1 ? PB : 4;
    const int pgroups = KS == 1 ? (panels + PB - 1) / PB : panels / 4;       // stages per block of rows
    int ist = 0, iss_pan = pan0, iss_y = first * kRwRows, to_issue = my_blocks * pgroups;
    const int y_step = stride * kRwRows;
    auto issue_next = [&]() {
        const int np = panels - iss_pan < PB ? panels - iss_pan : PB;
        mbar_expect_tx(&bars[ist], (uint32_t)np * kRwStageBytes);
#pragma unroll
        for (int k = 0; k < PB; ++k)
            if (k < np)
                tma_panel_g2s(ring + ist * kStage + k * kRwStageBytes, &P.tmap, (iss_pan + k) * kRwPanelBytes, iss_y,
                              &bars[ist]);
        --to_issue;
        if (++ist == S) ist = 0;
        iss_pan += pan_step;
        if (iss_pan >= panels) { iss_pan = pan0; iss_y += y_step; }
    };
    // Weights do not depend on the previous kernel in the stream: request them first.
    if (lane == 0)
        for (int i = 0; i < S && to_issue > 0; ++i) issue_next();

    pdl_launch_dependents();
    if (p.pdl) pdl_wait();
    // ---- activations into shared memory.  Per 32-byte unit (two 16-runs, the part of a group
    // one lane feeds to the four MMAs) the words are interleaved {lo.x, hi.x, lo.y, hi.y, lo.z,
    // hi.z, lo.w, hi.w}, so that the B operand pair of every MMA is an aligned register pair of
    // one 16-byte load.  Row W is zero: lanes whose token does not exist read it.
    // All global reads of this prologue are issued before the first of them is used, so the
    // warps sit through one memory round trip, not three, while the rings fill.
    {
        float *invs_w = reinterpret_cast<float *>(smem + L.invs_off);
        int *asum_s = reinterpret_cast<int *>(smem + L.asum_off);
        int4 *nbq = reinterpret_cast<int4 *>(smem + L.nb_off);
        const bool prepared = p.asum != nullptr;
        const int units = p.K / 32, total_units = p.W * units;
        constexpr int kMaxUnits = 4;                       // units kept in registers per thread
        uint4 ulo[kMaxUnits], uhi[kMaxUnits];
#pragma unroll
        for (int k = 0; k < kMaxUnits; ++k) {
            const int i = threadIdx.x + k * THREADS;
            if (i < total_units) {
                const int m = i / units, u = i - m * units;
                const uint4 *src = reinterpret_cast<const uint4 *>(p.A + (size_t)m * p.K + 32 * u);
                ulo[k] = src[0];
                uhi[k] = src[1];
            }
        }
        float sval = 1.0f;
        if (threadIdx.x < 8 && threadIdx.x < p.W) sval = p.s[threadIdx.x];
        int pa0 = 0, pa1 = 0;                              // prepared: this thread's C quad entry
        if (prepared && threadIdx.x < ng * 4) {
            const int gg = threadIdx.x >> 2, qq = threadIdx.x & 3;
            if (2 * qq < p.W) pa0 = p.asum[(2 * qq) * ng + gg];
            if (2 * qq + 1 < p.W) pa1 = p.asum[(2 * qq + 1) * ng + gg];
        }
        // shared-memory initialisation while the loads are in flight
        if (!prepared)
            for (int i = threadIdx.x; i < 8 * ng; i += THREADS) asum_s[i] = 0;
        for (int i = threadIdx.x; i < L.act_stride / 16; i += THREADS)
            *reinterpret_cast<uint4 *>(smem + L.act_off + p.W * L.act_stride + 16 * i) = make_uint4(0u, 0u, 0u, 0u);
        if (KS > 1 && threadIdx.x < kRwMaxWarps)
            reinterpret_cast<int *>(smem + L.xch_off + 2 * kRwMaxWarps * 32 * 4 * 4)[threadIdx.x] = 0;
        __syncthreads();
        if (threadIdx.x < 8) invs_w[threadIdx.x] = threadIdx.x < p.W ? 1.0f / sval : 0.0f;
        if (prepared)
            for (int i = threadIdx.x; i < ng * 4; i += THREADS) {
                int v0 = pa0, v1 = pa1;
                if (i >= THREADS) {                        // more groups than threads / 4: late loads
                    const int gg = i >> 2, qq = i & 3;
                    v0 = 2 * qq < p.W ? p.asum[(2 * qq) * ng + gg] : 0;
                    v1 = 2 * qq + 1 < p.W ? p.asum[(2 * qq + 1) * ng + gg] : 0;
                }
                nbq[i] = make_int4(kGroupSumBias - 2 * v0, kGroupSumBias - 2 * v1, kGroupSumBias - 2 * v0, kGroupSumBias - 2 * v1);
            }
        for (int i0 = 0; i0 < total_units; i0 += kMaxUnits * THREADS) {
#pragma unroll
            for (int k = 0; k < kMaxUnits; ++k) {
                const int i = i0 + threadIdx.x + k * THREADS;
                if (i >= total_units) break;
                const int m = i / units, u = i - m * units;
                uint4 lo, hi;
                if (i0 == 0) {
                    lo = ulo[k];
                    hi = uhi[k];
                } else {
                    const uint4 *src = reinterpret_cast<const uint4 *>(p.A + (size_t)m * p.K + 32 * u);
                    lo = src[0];
                    hi = src[1];
                }
                if (!prepared) {
                    // natural order: group sum, then the 4x4 byte transpose per 16-run
                    int sum = __dp4a((int)lo.x, 0x01010101, 0);
                    sum = __dp4a((int)lo.y, 0x01010101, sum);
                    sum = __dp4a((int)lo.z, 0x01010101, sum);
                    sum = __dp4a((int)lo.w, 0x01010101, sum);
                    sum = __dp4a((int)hi.x, 0x01010101, sum);
                    sum = __dp4a((int)hi.y, 0x01010101, sum);
                    sum = __dp4a((int)hi.z, 0x01010101, sum);
                    sum = __dp4a((int)hi.w, 0x01010101, sum);
                    atomicAdd(&asum_s[m * ng + (u >> 2)], sum);
                    lo = transpose_run16(lo);
                    hi = transpose_run16(hi);
                }
                uint4 *dst = reinterpret_cast<uint4 *>(smem + L.act_off + m * L.act_stride + 32 * u);
                dst[0] = make_uint4(lo.x, hi.x, lo.y, hi.y);
                dst[1] = make_uint4(lo.z, hi.z, lo.w, hi.w);
            }
        }
        __syncthreads();
        if (!prepared) {
            for (int i = threadIdx.x; i < ng * 4; i += THREADS) {
                const int gg = i >> 2, qq = i & 3, t0 = 2 * qq, t1 = 2 * qq + 1;
                const int v0 = kGroupSumBias + (t0 < p.W ? -2 * asum_s[t0 * ng + gg] : 0);
                const int v1 = kGroupSumBias + (t1 < p.W ? -2 * asum_s[t1 * ng + gg] : 0);
                nbq[i] = make_int4(v0, v1, v0, v1);
            }
            __syncthreads();
        }
    }
    const float *invs = reinterpret_cast<const float *>(smem + L.invs_off);
    const unsigned char *nb_base = smem + L.nb_off + 16 * q;                  // C quad of group 0
    const unsigned char *arow0 = smem + L.act_off + (g < p.W ? g : p.W) * L.act_stride + 32 * q;  // token g or zeros
    // Swizzled position of this lane's 8 bytes of group j (0..3) of a panel, rows g and g+8:
    // 16-byte chunk (2j + q/2) is stored at chunk (2j + q/2) ^ (row & 7).
    int woff[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) woff[j] = g * kRwPanelBytes + (((2 * j + (q >> 1)) ^ g) << 4) + ((q & 1) << 3);

    int cst = 0;                                      // stage to consume next
    uint32_t cpar = 0;                                // its phase parity
    int waited = 0;                                   // panels consumed (error path only)
    bool ok = true;
    const uint16_t *sc0 = p.ws + (size_t)(first * kRwRows + g) * ng;   // scales of rows g and g+8
    const size_t sc_step = (size_t)stride * kRwRows * ng;
    int n0 = first * kRwRows;
    for (int t = 0; t < my_blocks && ok; ++t, n0 += stride * kRwRows, sc0 += sc_step) {
        const uint16_t *sc8 = sc0 + (size_t)8 * ng;
        float acc[BM_SLOTS][NA];
#pragma unroll
        for (int s = 0; s < BM_SLOTS; ++s)
#pragma unroll
            for (int e = 0; e < NA; ++e) acc[s][e] = 0.0f;
        uint2 nsc0 = *reinterpret_cast<const uint2 *>(sc0 + 4 * pan0), nsc8 = *reinterpret_cast<const uint2 *>(sc8 + 4 * pan0);

        for (int p4 = 0; p4 < panels && ok; p4 += 4) {
#pragma unroll
            for (int pp = 0; pp < 4; ++pp) {
                const int pan = p4 + pp;
                if (pan >= panels) break;                              // warp-uniform
                if (KS == 2 && (pp >> 1) != ks) continue;              // another warp of the team owns these slots
                if (KS == 4 && pp != ks) continue;
                const unsigned char *arow = arow0 + (size_t)pan * 4 * BM_GROUP, *nbp = nb_base + (size_t)pan * 4 * 64;
                const int G = 4 * pan;
                if (pp % PB == 0) {
                    ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bars[cst], cpar));
                    if (!ok) break;
                }
                const unsigned char *stage = ring + cst * kStage + (pp % PB) * kRwStageBytes;
                const uint2 csc0 = nsc0, csc8 = nsc8;
                const int nxt = KS == 1 ? pan + 1 : (KS == 2 ? ((pp & 1) ? pan + 3 : pan + 1) : pan + 4);   // next panel of this warp
                if (nxt < panels) {
                    nsc0 = *reinterpret_cast<const uint2 *>(sc0 + 4 * nxt);
                    nsc8 = *reinterpret_cast<const uint2 *>(sc8 + 4 * nxt);
                }
                // IL groups in lock-step: their four-MMA chains are independent of each other,
                // so consecutive MMAs never wait for the previous one's result.
#pragma unroll
                for (int j0 = 0; j0 < 4; j0 += IL) {
                    uint2 x[IL], y[IL];
                    uint4 b01[IL], b23[IL];
                    int d[IL][4];
                    constexpr uint32_t M3 = 0x03030303u;
#pragma unroll
                    for (int jj = 0; jj < IL; ++jj) {
                        const int j = j0 + jj;
                        x[jj] = *reinterpret_cast<const uint2 *>(stage + woff[j]);
                        y[jj] = *reinterpret_cast<const uint2 *>(stage + woff[j] + 8 * kRwPanelBytes);
                        b01[jj] = *reinterpret_cast<const uint4 *>(arow + BM_GROUP * j);        // steps 0, 1
                        b23[jj] = *reinterpret_cast<const uint4 *>(arow + BM_GROUP * j + 16);   // steps 2, 3
                    }
#pragma unroll
                    for (int jj = 0; jj < IL; ++jj) {
                        const int4 c = *reinterpret_cast<const int4 *>(nbp + 64 * (j0 + jj));
                        mma_u8s8(d[jj], x[jj].x & M3, y[jj].x & M3, x[jj].y & M3, y[jj].y & M3, b01[jj].x, b01[jj].y,
                                 c.x, c.y, c.z, c.w);
                    }
#pragma unroll
                    for (int jj = 0; jj < IL; ++jj)
                        mma_u8s8(d[jj], (x[jj].x >> 2) & M3, (y[jj].x >> 2) & M3, (x[jj].y >> 2) & M3,
                                 (y[jj].y >> 2) & M3, b01[jj].z, b01[jj].w, d[jj][0], d[jj][1], d[jj][2], d[jj][3]);
#pragma unroll
                    for (int jj = 0; jj < IL; ++jj)
                        mma_u8s8(d[jj], (x[jj].x >> 4) & M3, (y[jj].x >> 4) & M3, (x[jj].y >> 4) & M3,
                                 (y[jj].y >> 4) & M3, b23[jj].x, b23[jj].y, d[jj][0], d[jj][1], d[jj][2], d[jj][3]);
#pragma unroll
                    for (int jj = 0; jj < IL; ++jj)
                        mma_u8s8(d[jj], (x[jj].x >> 6) & M3, (y[jj].x >> 6) & M3, (x[jj].y >> 6) & M3,
                                 (y[jj].y >> 6) & M3, b23[jj].z, b23[jj].w, d[jj][0], d[jj][1], d[jj][2], d[jj][3]);
#pragma unroll
                    for (int jj = 0; jj < IL; ++jj) {
                        const int j = j0 + jj;
                        const uint32_t w0 = (j < 2) ? csc0.x : csc0.y, w8 = (j < 2) ? csc8.x : csc8.y;
                        const float s0 = (j & 1) ? __uint_as_float(w0 & 0xffff0000u) : __uint_as_float(w0 << 16);
                        const float s8 = (j & 1) ? __uint_as_float(w8 & 0xffff0000u) : __uint_as_float(w8 << 16);
                        float(&a)[NA] = acc[4 * pp + j];
                        if (NTOK == 2) {
                            a[0] = fmaf(group_sum_to_float(d[jj][0]), s0, a[0]);
                            a[1] = fmaf(group_sum_to_float(d[jj][1]), s0, a[1]);
                            a[2] = fmaf(group_sum_to_float(d[jj][2]), s8, a[2]);
                            a[3] = fmaf(group_sum_to_float(d[jj][3]), s8, a[3]);
                        } else {
                            a[0] = fmaf(group_sum_to_float(d[jj][0]), s0, a[0]);
                            a[1] = fmaf(group_sum_to_float(d[jj][2]), s8, a[1]);
                        }
                        if (EMIT_G) {
                            const int t0 = 2 * q, t1 = 2 * q + 1;
                            if (t0 < p.W) {
                                p.G[((size_t)t0 * p.N + n0 + g) * ng + G + j] = d[jj][0] - kGroupSumBias;
                                p.G[((size_t)t0 * p.N + n0 + g + 8) * ng + G + j] = d[jj][2] - kGroupSumBias;
                            }
                            if (t1 < p.W) {
                                p.G[((size_t)t1 * p.N + n0 + g) * ng + G + j] = d[jj][1] - kGroupSumBias;
                                p.G[((size_t)t1 * p.N + n0 + g + 8) * ng + G + j] = d[jj][3] - kGroupSumBias;
                            }
                        }
                    }
                }
                if (pp % PB == PB - 1 || pan == panels - 1) {
                    ++waited;
                    if (++cst == S) { cst = 0; cpar ^= 1u; }
                    __syncwarp();                                      // every lane is done with the stage
                    if (lane == 0 && to_issue > 0) issue_next();
                }
            }
        }
        if (KS == 1 && !ok) break;
        // Tree over the 16 slots (offsets 1, 2, 4, 8), reciprocal multiply, store.
        float yv[NA];
#pragma unroll
        for (int e = 0; e < NA; ++e) {
            const float s01 = acc[0][e] + acc[1][e], s23 = acc[2][e] + acc[3][e];
            const float s45 = acc[4][e] + acc[5][e], s67 = acc[6][e] + acc[7][e];
            const float s89 = acc[8][e] + acc[9][e], sab = acc[10][e] + acc[11][e];
            const float scd = acc[12][e] + acc[13][e], sef = acc[14][e] + acc[15][e];
            if (KS == 1) yv[e] = ((s01 + s23) + (s45 + s67)) + ((s89 + sab) + (scd + sef));
            else if (KS == 2) yv[e] = ks == 0 ? (s01 + s23) + (s45 + s67) : (s89 + sab) + (scd + sef);
            else yv[e] = ks == 0 ? s01 + s23 : (ks == 1 ? s45 + s67 : (ks == 2 ? s89 + sab : scd + sef));
        }
        if (KS > 1) {
            // the team's other warps hand their partial sums to warp 0, which adds them in tree order; two
            // buffers used in turn, so that one named barrier per block of rows is enough
            float *xch = reinterpret_cast<float *>(smem + L.xch_off) + (size_t)((t & 1) * kRwMaxWarps + team * KS) * 32 * 4;
            volatile int *tfail = reinterpret_cast<volatile int *>(smem + L.xch_off + 2 * kRwMaxWarps * 32 * 4 * 4) + team;
            if (!ok && lane == 0) *tfail = 1;          // a wait of this warp ran out: the whole team leaves after the barrier
            if (ks != 0) {
#pragma unroll
                for (int e = 0; e < NA; ++e) xch[((ks - 1) * 32 + lane) * 4 + e] = yv[e];
            }
            asm volatile("bar.sync %0, %1;" ::"r"(1 + team), "r"(KS * 32) : "memory");
            if (*tfail) { ok = false; break; }
            if (ks != 0) continue;
#pragma unroll
            for (int e = 0; e < NA; ++e) {
                const float p1 = xch[(0 * 32 + lane) * 4 + e];
                if (KS == 2) yv[e] = yv[e] + p1;
                else yv[e] = (yv[e] + p1) + (xch[(1 * 32 + lane) * 4 + e] + xch[(2 * 32 + lane) * 4 + e]);
            }
        }
        if (NTOK == 2) {
            const int t0 = 2 * q, t1 = 2 * q + 1;
            if (t0 < p.W) {
                const float is = invs[t0];
                gemv_store(p, t0, n0 + g, yv[0] * is);
                gemv_store(p, t0, n0 + g + 8, yv[2 % NA] * is);
            }
            if (t1 < p.W) {
                const float is = invs[t1];
                gemv_store(p, t1, n0 + g, yv[1] * is);
                gemv_store(p, t1, n0 + g + 8, yv[3 % NA] * is);
            }
        } else if (q == 0) {
            const float is = invs[0];
            gemv_store(p, 0, n0 + g, yv[0] * is);
            gemv_store(p, 0, n0 + g + 8, yv[1] * is);
        }
    }
    if (!ok) {
        // Give up: record it and give the copies still in flight a last bounded chance to
        // land in this warp's ring before the CTA's shared memory is released.
        if (lane == 0) {
            report_error(kErrRowWarpWaitTimeout);
            const int in_flight = my_blocks * pgroups - to_issue - waited;   // stages requested and not consumed
            for (int c = 0; c < in_flight; ++c) {
                for (int it = 0; it < (1 << 12); ++it)
                    if (mbar_try_wait(&bars[cst], cpar)) break;
                if (++cst == S) { cst = 0; cpar ^= 1u; }
            }
        }
    }
    gemv_peer_finish(p);
}

}  // namespace bm
