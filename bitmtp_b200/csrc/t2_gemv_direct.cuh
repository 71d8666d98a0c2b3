// T2-g128 GEMV for few tokens and few rows: a warp per output row, operands straight from
// global memory into registers.
//
// Replaces, for W <= 4 and layers of a few MB, t2g128_mfused of the reference
// (src/bonsai_sft/gpu/t2g128_kernels/t2g128_kernels.cu:29-92).  A launch over 0.5-6 MB of
// weights is bound by latency, not by bandwidth: what counts is the number of dependent memory
// round trips between the start of the grid and its last store.  The cooperative-tile and
// row-per-warp kernels stage operands in shared memory (barrier initialisation, bulk copies,
// an activation staging pass, a cross-warp reduction) and need four to five microseconds for
// any size; this kernel has one round trip: every lane requests its 16 bytes of packed weights,
// its scale and its 64 activations per token at once, then computes from registers.
//
// Work split: row n = one warp.  A pass covers 2048 elements of K in four steps q: lane l owns the
// 16-element run at k = 2048*pass + 512*q + 16*l, so a warp's activation loads are 512 contiguous
// bytes and its weight loads 128 (every sector fetched is used in full; with 64 contiguous elements per
// lane the activation sectors were fetched twice, which ncu showed as 299 K against 174 K sectors and a
// third more cycles).  Eight lanes share a group: their integer partial sums are added by shuffles,
// so every lane holds the exact group sum G of group 16*pass + 4*q + l/8.  fp32 order as in every other
// GEMV of this library (and bmo_t2_gemv of the CPU oracle): group g feeds slot g % 16 = 4*q + l/8 with
// fma((float)G, scale, slot) in ascending g (= ascending pass); the 16 slots are summed in the order
// of the xor butterfly with slot offsets 1, 2 (lane offsets 8, 16), 4, 8 (the q index, in registers);
// the sum is multiplied by 1/s[m].
//
// Activations: GEMV-ready (16-runs already in the order of the code registers `(word >> 2t) &
// 0x03030303`, group sums in p.asum), or natural order.  For one natural-order token the kernel
// transposes the token's 16-runs in registers and sums them with dp4a; for several it transposes
// the code registers instead and makes them signed, once for all tokens.
#pragma once

#include "t2_gemv.cuh"
#include "t2_gemv_rowwarp.cuh"

namespace bm {

constexpr int kDirectWarps = 8;          // rows per CTA
constexpr int kDirectMaxPasses = 5;      // K <= 10240
constexpr int kDirectMaxW = 4;

__host__ __device__ inline bool direct_fits(int W, int N, int K) {
    return W >= 1 && W <= kDirectMaxW && K >= 128 && (K % 128) == 0 && K <= 2048 * kDirectMaxPasses && N >= 1;
}

__device__ __forceinline__ int dp4a_s8_u8(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// The operands of a plain GEMV call only: a launch this short also pays for the size of its parameter block.
struct DirectParams {
    const int8_t *A;
    const int32_t *asum;
    const uint8_t *B;
    const uint16_t *ws;
    const float *s;
    void *C;
    int32_t *G;
    int W, N, K, ldc, out_kind, pdl;
};

__device__ __forceinline__ void direct_store(const DirectParams &p, int m, int n, float y) {
    if (p.out_kind == 0) reinterpret_cast<uint16_t *>(p.C)[(size_t)m * p.ldc + n] = bm_f32_to_bf16(y);
    else reinterpret_cast<float *>(p.C)[(size_t)m * p.ldc + n] = p.out_kind == 1 ? y : bm_bf16_rn(y);
}

// Sum over the eight lanes that share a group.
__device__ __forceinline__ int direct_group_sum(int v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    return v;
}

// The 16 slots (acc[q] of the four lane octets) summed in the canonical order.
__device__ __forceinline__ float direct_slot_tree(const float (&acc)[4]) {
    float t[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        t[q] = acc[q] + __shfl_xor_sync(0xffffffffu, acc[q], 8);
        t[q] = t[q] + __shfl_xor_sync(0xffffffffu, t[q], 16);
    }
    return (t[0] + t[1]) + (t[2] + t[3]);
}

// MAXP: passes the kernel is built for (K <= 2048 * MAXP); registers grow with it.
template <int WT, int MAXP>
__global__ void __launch_bounds__(kDirectWarps * 32) t2_gemv_direct_kernel(const DirectParams p) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = blockIdx.x * kDirectWarps + warp;
    pdl_launch_dependents();
    if (n >= p.N) return;
    const int ng = p.K >> 7;
    const int passes = (p.K + 2047) >> 11;
    const bool prepared = p.asum != nullptr;

    // Weights and scales do not depend on the previous kernel: request them first.
    uint32_t wv[MAXP][4];
    float sc[MAXP][4];
    const uint32_t *wrow = reinterpret_cast<const uint32_t *>(p.B + (size_t)n * (p.K >> 2));
#pragma unroll
    for (int ps = 0; ps < MAXP; ++ps)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int g = 16 * ps + 4 * q + (lane >> 3);
            const bool active = ps < passes && g < ng;
            wv[ps][q] = active ? __ldg(wrow + 128 * ps + 32 * q + lane) : 0u;
            sc[ps][q] = active ? bm_bf16_to_f32(__ldg(p.ws + (size_t)n * ng + g)) : 0.0f;
        }
    if (p.pdl) pdl_wait();
    // 1/s of the token this lane will store, requested with the activations
    const float inv_s = (lane < WT && lane < p.W) ? 1.0f / p.s[lane] : 0.0f;

    float acc[WT][4];
#pragma unroll
    for (int m = 0; m < WT; ++m)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[m][q] = 0.0f;

#pragma unroll
    for (int ps = 0; ps < MAXP; ++ps) {
        if (ps >= passes) break;                                   // uniform
        uint4 av[WT][4];
        int asum_g[WT][4];
#pragma unroll
        for (int m = 0; m < WT; ++m)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int g = 16 * ps + 4 * q + (lane >> 3);
                const bool on = g < ng && m < p.W;
                av[m][q] = on ? *reinterpret_cast<const uint4 *>(p.A + (size_t)m * p.K + 2048 * ps + 512 * q + 16 * lane)
                              : make_uint4(0u, 0u, 0u, 0u);
                asum_g[m][q] = (prepared && on) ? p.asum[m * ng + g] : 0;
            }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int g = 16 * ps + 4 * q + (lane >> 3);
            // codes of packed bytes 0..3 of this word: register t holds element t of each byte
            const uint32_t w = wv[ps][q];
            const uint32_t c0 = w & 0x03030303u, c1 = (w >> 2) & 0x03030303u, c2 = (w >> 4) & 0x03030303u,
                           c3 = (w >> 6) & 0x03030303u;
            int part[WT];
            if (prepared || WT == 1) {
#pragma unroll
                for (int m = 0; m < WT; ++m) {
                    uint4 a = av[m][q];
                    part[m] = 0;
                    if (!prepared) {
                        // one token: cheaper to bring its 16-run into the order of the code registers
                        int sum = __dp4a((int)a.x, 0x01010101, 0);
                        sum = __dp4a((int)a.y, 0x01010101, sum);
                        sum = __dp4a((int)a.z, 0x01010101, sum);
                        sum = __dp4a((int)a.w, 0x01010101, sum);
                        part[m] = -2 * sum;                        // codes are value + 2
                        a = transpose_run16(a);
                    }
                    part[m] = dp4a_s8_u8(a.x, c0, part[m]);
                    part[m] = dp4a_s8_u8(a.y, c1, part[m]);
                    part[m] = dp4a_s8_u8(a.z, c2, part[m]);
                    part[m] = dp4a_s8_u8(a.w, c3, part[m]);
                }
            } else {
                // several tokens in natural order: bring the codes into natural order once instead and
                // make them signed (code - 2 per byte, no borrow across bytes), shared by all tokens
                const uint4 nat = transpose_run16(make_uint4(c0, c1, c2, c3));
                const uint32_t s0 = ((nat.x | 0x80808080u) - 0x02020202u) ^ 0x80808080u;
                const uint32_t s1 = ((nat.y | 0x80808080u) - 0x02020202u) ^ 0x80808080u;
                const uint32_t s2 = ((nat.z | 0x80808080u) - 0x02020202u) ^ 0x80808080u;
                const uint32_t s3 = ((nat.w | 0x80808080u) - 0x02020202u) ^ 0x80808080u;
#pragma unroll
                for (int m = 0; m < WT; ++m) {
                    const uint4 a = av[m][q];
                    part[m] = __dp4a((int)a.x, (int)s0, 0);
                    part[m] = __dp4a((int)a.y, (int)s1, part[m]);
                    part[m] = __dp4a((int)a.z, (int)s2, part[m]);
                    part[m] = __dp4a((int)a.w, (int)s3, part[m]);
                }
            }
#pragma unroll
            for (int m = 0; m < WT; ++m) {
                const int G = direct_group_sum(part[m]) - 2 * asum_g[m][q];
                acc[m][q] = fmaf(group_sum_to_float(G + kGroupSumBias), sc[ps][q], acc[m][q]);
                if (p.G != nullptr && g < ng && (lane & 7) == 0 && m < p.W)
                    p.G[((size_t)m * p.N + n) * ng + g] = G;
            }
        }
    }
#pragma unroll
    for (int m = 0; m < WT; ++m) {
        const float v = direct_slot_tree(acc[m]);
        if (lane == m && m < p.W) direct_store(p, m, n, v * inv_s);
    }
}

// ---- width 1 with the activation row made in the kernel (src_mode 1 / 2) ------------------------
// The register-only GEMV for the projections of a width-1 replay: every CTA first turns the bf16 input
// row into GEMV-ready INT8 codes in shared memory (gemv_stage_row_from_bf16: known absmax, or residual
// add + RMSNorm, exactly as the cooperative kernel's prologue does), then each of its 8 warps computes
// one output column from registers.  SILU: a warp computes column n of the gate rows and of the up
// rows (B holds silu_F gate rows, then silu_F up rows) and stores bf16(silu(bf16 gate) * bf16 up); the
// row's max |output| goes to p.amax_out by atomic max.  Weight rows are requested before the wait on
// the previous kernel.  Same results as t2_gemv_mma_kernel with src_mode != 0, bit for bit.
constexpr int kDirectRowAsumOff = 2048 * kDirectMaxPasses;                 // int32 [K/128]
constexpr int kDirectRowInvsOff = kDirectRowAsumOff + 4 * 16 * kDirectMaxPasses;   // float [16]
constexpr int kDirectRowShOff = kDirectRowInvsOff + 64;                    // float [32]
constexpr int kDirectRowSmem = kDirectRowShOff + 128;

__host__ __device__ inline bool direct_row_fits(int N, int K) {
    return K >= 256 && (K % 256) == 0 && K <= 2048 * kDirectMaxPasses && N >= 8 && (N % 8) == 0;
}

template <bool SILU, int MAXP>
__global__ void __launch_bounds__(kGemvThreads) t2_gemv_direct_row_kernel(const GemvParams p) {
    __shared__ __align__(16) unsigned char smem[kDirectRowSmem];
    __shared__ unsigned int amax_sh;
    constexpr int NR = SILU ? 2 : 1;                    // weight rows per output column
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n = blockIdx.x * kDirectWarps + warp;     // output column; N % 8 == 0, so every warp has one
    const int ng = p.K >> 7;
    const int passes = (p.K + 2047) >> 11;
    pdl_launch_dependents();
    if (SILU && threadIdx.x == 0) amax_sh = 0u;

    uint32_t wv[NR][MAXP][4];
    float sc[NR][MAXP][4];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const size_t row = (size_t)n + (size_t)r * p.silu_F;
        const uint32_t *wrow = reinterpret_cast<const uint32_t *>(p.B + row * (p.K >> 2));
#pragma unroll
        for (int ps = 0; ps < MAXP; ++ps)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int g = 16 * ps + 4 * q + (lane >> 3);
                const bool active = ps < passes && g < ng;
                wv[r][ps][q] = active ? __ldg(wrow + 128 * ps + 32 * q + lane) : 0u;
                sc[r][ps][q] = active ? bm_bf16_to_f32(__ldg(p.ws + row * ng + g)) : 0.0f;
            }
    }
    if (p.pdl) pdl_wait();
    gemv_stage_row_from_bf16(p, smem, 0, kDirectRowAsumOff, kDirectRowInvsOff,
                             reinterpret_cast<float *>(smem + kDirectRowShOff));
    __syncthreads();
    const int *asum = reinterpret_cast<const int *>(smem + kDirectRowAsumOff);
    const float inv_s = reinterpret_cast<const float *>(smem + kDirectRowInvsOff)[0];

    float acc[NR][4];
#pragma unroll
    for (int r = 0; r < NR; ++r)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[r][q] = 0.0f;
#pragma unroll
    for (int ps = 0; ps < MAXP; ++ps) {
        if (ps >= passes) break;                                   // uniform
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int g = 16 * ps + 4 * q + (lane >> 3);
            const bool active = g < ng;
            const uint4 a = active ? *reinterpret_cast<const uint4 *>(smem + 2048 * ps + 512 * q + 16 * lane)
                                   : make_uint4(0u, 0u, 0u, 0u);
            const int nb = kGroupSumBias - 2 * (active ? asum[g] : 0);
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const uint32_t w = wv[r][ps][q];
                int part = dp4a_s8_u8(a.x, w & 0x03030303u, 0);
                part = dp4a_s8_u8(a.y, (w >> 2) & 0x03030303u, part);
                part = dp4a_s8_u8(a.z, (w >> 4) & 0x03030303u, part);
                part = dp4a_s8_u8(a.w, (w >> 6) & 0x03030303u, part);
                acc[r][q] = fmaf(group_sum_to_float(direct_group_sum(part) + nb), sc[r][ps][q], acc[r][q]);
            }
        }
    }
    float y[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) y[r] = direct_slot_tree(acc[r]) * inv_s;
    if (SILU) {
        if (lane == 0) {
            const float v = bm_bf16_rn(bm_silu_bf16(bm_bf16_rn(y[0])) * bm_bf16_rn(y[NR - 1]));
            reinterpret_cast<uint16_t *>(p.C)[n] = bm_f32_to_bf16(v);
            atomicMax(&amax_sh, __float_as_uint(fabsf(v)));
        }
        __syncthreads();
        if (threadIdx.x == 0 && amax_sh != 0u) atomicMax(&p.amax_out[0], amax_sh);
    } else if (lane == 0) {
        gemv_store(p, 0, n, y[0]);
    }
}

}  // namespace bm
