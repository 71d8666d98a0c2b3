// Dense tied head for the draft role: logits of up to 24 rows against the bf16 embedding table
// (`bf16_raw`) or against its per-tensor e4m3 copy (`fp8`).
//
// Replaces the two dense branches of Transformer._lm_head
// (src/bonsai_sft/gpu/model.py:1266-1282): `fp8` = per-tensor activation scale, e4m3 cast,
// torch._scaled_mm(h_fp8, W_fp8^T, scale_a, scale_b, out bf16) on the weight prepared by
// prepare_fp8_lm_head (model.py:1169-1194); `bf16_raw` = F.linear(h, W).  Both read the whole dense
// table once per call (311 MB / 622 MB for vocabulary 151936 x 2048), so the kernel is a stream over
// HBM: every warp owns blocks of 16 vocabulary rows and walks K with 16-byte loads straight from
// global memory into MMA fragments (no staging: a row's bytes are used once), the few activation
// rows wait in shared memory, products go through mma.sync m16n8k16 with fp32 accumulators (f16
// operands for the e4m3 table, whose values f16 holds exactly; bf16 operands for the bf16 table).
// The k order inside a fragment is permuted the same way on both operands (a dot product does not
// care), which is what lets a lane take 16 contiguous bytes of a row.
//
// Accumulation order is fixed (per output: k-blocks ascending inside the tensor-core adds) but, as
// for the cuBLASLt kernels it replaces, it is not the order of a CPU sum: parity for these two
// heads is a tolerance against an fp32 evaluation of the same quantised operands.
#pragma once

#include <cuda_fp16.h>

#include "bm_common.cuh"
#include "fused_ops.cuh"

namespace bm {

constexpr int kDenseThreads = 256;
constexpr int kDenseMaxRows = 24;              // activation rows per call (3 MMA column blocks)
// 16-bit elements of padding per staged activation row, chosen so that the fragment reads of a
// quarter warp fall into eight different 16-byte bank groups: the bf16 build reads one 16-byte piece per
// lane at (row g, 16t bytes) and wants the row stride = 64 mod 128 bytes; the e4m3 build reads two
// adjacent pieces per lane at (row g, 32t bytes) and wants 16 mod 128.
__host__ __device__ constexpr int dense_act_pad(bool fp8) { return fp8 ? 8 : 32; }

struct DenseHeadParams {
    const void *W;             // [N, K] bf16, or e4m3 when fp8
    const uint16_t *h;         // [R, K] bf16 normed rows
    const float *w_scale;      // fp8: per-tensor weight scale (device scalar)
    float *out;                // [R, ldc] fp32 holding bf16-rounded logits
    float *h_scale_out;        // fp8, optional: the activation scale this call derived
    int R, N, K, ldc, pdl;
};

__host__ __device__ inline size_t dense_head_smem(int R, int K, bool fp8) {
    const int rows = (R + 7) / 8 * 8;
    return (size_t)rows * (K + dense_act_pad(fp8)) * 2 + 64;
}

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1, bool f16) {
    if (f16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                     : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// two e4m3 bytes -> two f16 values (exact)
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint16_t v) {
    uint32_t r;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
    return r;
}

// fp32 -> e4m3 (round to nearest even, saturating to +-448 as the cast of an in-range value does)
__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(v));
    return (uint8_t)(r & 0xff);
}

// NB: MMA column blocks (8 activation rows each).  FP8: the table is e4m3 and the activations are cast
// to e4m3 with a per-tensor scale first.  grid: up to 2 CTAs per SM, 8 warps each; a warp takes
// 16-row blocks of the table round-robin.
template <int NB, bool FP8>
__global__ void __launch_bounds__(kDenseThreads, 2) dense_head_kernel(const DenseHeadParams p) {
    extern __shared__ __align__(16) unsigned char dyn[];
    __shared__ float red[kDenseThreads / 32];
    pdl_launch_dependents();
    if (p.pdl) pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int astride = p.K + dense_act_pad(FP8);                 // 16-bit elements per staged row
    uint16_t *As = reinterpret_cast<uint16_t *>(dyn);             // [NB*8][astride] f16 (FP8) or bf16
    float h_scale = 1.0f;
    if (FP8) {
        // per-tensor activation scale: bf16(amax / 448), at least 1e-12 (the reference divides a bf16
        // 0-dim tensor by a Python float, which stays bf16)
        float amax = 0.0f;
        for (int i = tid; i < p.R * (p.K / 8); i += kDenseThreads) {
            float f[8];
            unpack8(reinterpret_cast<const uint4 *>(p.h)[i], f);
#pragma unroll
            for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
        }
        amax = block_max(amax, red, lane, warp, kDenseThreads / 32);
        h_scale = fmaxf(bm_bf16_rn(amax / 448.0f), 1e-12f);
        if (blockIdx.x == 0 && tid == 0 && p.h_scale_out) *p.h_scale_out = h_scale;
    }
    // stage the activation rows: bf16 as they are, or e4m3(bf16(h / scale)) widened to f16; rows past R are zero
    for (int i = tid; i < NB * 8 * (p.K / 8); i += kDenseThreads) {
        const int r = i / (p.K / 8), u = i - r * (p.K / 8);
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < p.R) {
            v = reinterpret_cast<const uint4 *>(p.h + (size_t)r * p.K)[u];
            if (FP8) {
                float f[8];
                unpack8(v, f);
                uint32_t w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const uint16_t pair = (uint16_t)f32_to_e4m3(bm_bf16_rn(f[2 * e] / h_scale)) |
                                          ((uint16_t)f32_to_e4m3(bm_bf16_rn(f[2 * e + 1] / h_scale)) << 8);
                    w[e] = e4m3x2_to_f16x2(pair);
                }
                v = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        *reinterpret_cast<uint4 *>(As + (size_t)r * astride + 8 * u) = v;
    }
    __syncthreads();
    const float out_scale = FP8 ? h_scale * *p.w_scale : 1.0f;

    const int g = lane >> 2, t = lane & 3;
    const int nblocks = p.N / 16;
    const int wid = blockIdx.x * (kDenseThreads / 32) + warp, nwarps = gridDim.x * (kDenseThreads / 32);
    constexpr int KB = FP8 ? 64 : 32;          // k elements one lane-quad covers with 16-byte loads
    constexpr int UNROLL = 4;
    for (int nb = wid; nb < nblocks; nb += nwarps) {
        const int n0 = nb * 16;
        float acc[NB][4];
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[b][e] = 0.0f;
        const unsigned char *row0 = static_cast<const unsigned char *>(p.W) + (size_t)(n0 + g) * p.K * (FP8 ? 1 : 2) + 16 * t;
        const unsigned char *row8 = row0 + (size_t)8 * p.K * (FP8 ? 1 : 2);
        for (int k0 = 0; k0 < p.K; k0 += KB * UNROLL) {
            uint4 w0[UNROLL], w8[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int k = k0 + u * KB;
                if (k < p.K) {
                    w0[u] = __ldcs(reinterpret_cast<const uint4 *>(row0 + (size_t)k * (FP8 ? 1 : 2)));
                    w8[u] = __ldcs(reinterpret_cast<const uint4 *>(row8 + (size_t)k * (FP8 ? 1 : 2)));
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int k = k0 + u * KB;
                if (k >= p.K) break;
                if (FP8) {
                    // 16 e4m3 per row piece -> 8 f16x2 registers = four k16 steps
                    const uint32_t x0[4] = {w0[u].x, w0[u].y, w0[u].z, w0[u].w};
                    const uint32_t x8[4] = {w8[u].x, w8[u].y, w8[u].z, w8[u].w};
                    uint32_t a[4][4];
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        a[s][0] = e4m3x2_to_f16x2((uint16_t)(x0[s] & 0xffff));
                        a[s][2] = e4m3x2_to_f16x2((uint16_t)(x0[s] >> 16));
                        a[s][1] = e4m3x2_to_f16x2((uint16_t)(x8[s] & 0xffff));
                        a[s][3] = e4m3x2_to_f16x2((uint16_t)(x8[s] >> 16));
                    }
#pragma unroll
                    for (int b = 0; b < NB; ++b) {
                        const uint4 *bp = reinterpret_cast<const uint4 *>(As + (size_t)(8 * b + g) * astride + k + 16 * t);
                        const uint4 b01 = bp[0], b23 = bp[1];
                        mma_16816(acc[b], a[0][0], a[0][1], a[0][2], a[0][3], b01.x, b01.y, true);
                        mma_16816(acc[b], a[1][0], a[1][1], a[1][2], a[1][3], b01.z, b01.w, true);
                        mma_16816(acc[b], a[2][0], a[2][1], a[2][2], a[2][3], b23.x, b23.y, true);
                        mma_16816(acc[b], a[3][0], a[3][1], a[3][2], a[3][3], b23.z, b23.w, true);
                    }
                } else {
                    // 8 bf16 per row piece = two k16 steps
#pragma unroll
                    for (int b = 0; b < NB; ++b) {
                        const uint4 bb = *reinterpret_cast<const uint4 *>(As + (size_t)(8 * b + g) * astride + k + 8 * t);
                        mma_16816(acc[b], w0[u].x, w8[u].x, w0[u].y, w8[u].y, bb.x, bb.y, false);
                        mma_16816(acc[b], w0[u].z, w8[u].z, w0[u].w, w8[u].w, bb.z, bb.w, false);
                    }
                }
            }
        }
        // lane holds rows n0+g, n0+g+8 for activation rows 8b + 2t, 8b + 2t + 1
#pragma unroll
        for (int b = 0; b < NB; ++b) {
            const int r0 = 8 * b + 2 * t;
            if (r0 < p.R) {
                p.out[(size_t)r0 * p.ldc + n0 + g] = bm_bf16_rn(acc[b][0] * out_scale);
                p.out[(size_t)r0 * p.ldc + n0 + g + 8] = bm_bf16_rn(acc[b][2] * out_scale);
            }
            if (r0 + 1 < p.R) {
                p.out[(size_t)(r0 + 1) * p.ldc + n0 + g] = bm_bf16_rn(acc[b][1] * out_scale);
                p.out[(size_t)(r0 + 1) * p.ldc + n0 + g + 8] = bm_bf16_rn(acc[b][3] * out_scale);
            }
        }
    }
}

}  // namespace bm
