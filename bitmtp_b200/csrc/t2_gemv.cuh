// Packed T2-g128 ternary GEMV / skinny GEMM for sm_100a.
//
// Replaces the reference kernel t2g128_mfused and its dispatcher
// (src/bonsai_sft/gpu/t2g128_kernels/t2g128_kernels.cu:29-92, 94-148):
//   C[m, n] = ( sum_g  ws[n, g] * G[m, n, g] ) / s[m]
//   G[m, n, g] = sum_{k in group g} A[m, k] * (code[n, k] - 2)      (int32, exact)
// with A int8 [W, K], codes packed 4 per byte in natural order, ws bf16
// [N, K/128], s fp32 [W].
//
// Structure (one persistent CTA per SM slot, 8 warps):
//   * the weight matrix is cut into tiles of R = 8*RB consecutive output rows;
//     a tile is R contiguous rows of K/4 bytes plus R*K/128 bf16 scales, all
//     contiguous in global memory, so warp 0 fetches it with one bulk async
//     copy (TMA, untiled form) per row into a padded shared-memory row and one
//     copy for the scales, completion counted on an mbarrier.  STAGES tiles are
//     in flight per CTA; for the layer-sized matrices that is the CTA's whole
//     share, so every byte the kernel will read is requested before the first
//     one is consumed;
//   * the W activation rows are staged once per CTA into shared memory with a
//     4x4 byte transpose per 16 elements, so that the register produced by
//     `(word >> 2i) & 0x03030303` (codes 4e+i, e=0..3, of a 16-code word) meets
//     the four activations it multiplies in one 32-bit register.  Per-group
//     activation sums are kept too: codes are used unsigned (1,2,3) and
//     2*sum(A) is subtracted once per group, which removes the `code-2` from
//     the inner loop and keeps the group sum exact;
//   * two consumers share that frame:
//       lanes-across-K (dp4a): a warp owns rows, lane l owns the 64 weights of
//         one 16-byte piece; two lanes make a group.  Best for W <= 2.
//       tokens-as-MMA-rows (mma.sync m16n8k32 s8 x u8): a warp owns two of the
//         16 scale slots for all rows of the tile; the 16 tokens are the MMA's
//         M dimension, 8 output rows its N dimension, four MMAs cover a group
//         and the int32 fragment IS the group sum.  Cost is flat in W up to 16.
//
// fp32 order (shared with oracle/bm_oracle.c: bmo_t2_gemv): group g feeds slot
// g%16 with fma((float)G, scale, slot) in ascending g; the 16 slots are summed
// as a butterfly with offsets 1,2,4,8; the result is multiplied by the IEEE
// reciprocal 1/s[m] (the reference divides under --use_fast_math, i.e. by an
// approximate reciprocal; the exact one is within its error).  The order
// does not depend on W, on the consumer, or on the tile size, so a token's row
// is bit-identical at every replay width.
#pragma once

#include "bm_common.cuh"
#include "fused_ops.cuh"

namespace bm {

constexpr int kGemvThreads = 256;
constexpr int kGemvWarps = 8;
constexpr int kRowPad = 32;        // bytes appended to each staged weight row
constexpr int kActPad = 16;        // bytes appended to each staged activation row
constexpr int kMaxStages = 8;

struct GemvParams {
    const int8_t *A;        // [W, K]; natural order, or 4x4-transposed 16-runs when asum != nullptr
    const int32_t *asum;    // [W, K/128] group sums of A, or nullptr (the kernel then permutes and sums)
    const uint8_t *B;       // [N, K/4]
    const uint16_t *ws;     // [N, K/128] bf16 bits
    const float *s;         // [W]
    void *C;                // [W, ldc]  bf16 (out_kind 0) or fp32 (1, 2)
    int32_t *G;             // [W, N, K/128] or nullptr
    int W, N, K, ldc;
    int out_kind;           // 0 bf16, 1 fp32, 2 fp32 holding the bf16-rounded value
    int stages;             // tiles in flight per CTA
    int pdl;                // 1: wait for the previous grid before reading A / s
    // gate|up projection with SiLU(gate) * up in the epilogue (MMA consumer, bf16 output): B has
    // 2 * silu_F rows (gate rows, then up rows), N == silu_F output columns; a tile pairs 4*RB gate
    // rows with the 4*RB up rows of the same columns.  amax_out[m] receives, by atomic max, the bits of
    // max |output| of row m (zero before the launch).  silu_F == 0: plain projection.
    int silu_F;
    unsigned int *amax_out;
    // Width-1 launches that make their own activations (MMA consumer): instead of INT8 codes the
    // kernel is given the bf16 row and every CTA quantises it itself (a few thousand elements), which
    // removes a launch from the dependency chain of an AR replay.
    //   src_mode 1  x bf16 [K] + the bits of its absmax (amax_in[0]); amax_zero[0] is cleared
    //   src_mode 2  (gather | residual add) + RMSNorm of x (K == 2048 == 8 * threads), then the codes:
    //               the arithmetic of rmsnorm_kernel; CTA 0 stores the summed row to h_out
    int src_mode;
    const uint16_t *xb, *res, *norm_w;
    const int64_t *gather;
    int gather_rows;        // rows of xb when `gather` is given (the id is clamped into the table)
    uint16_t *h_out;
    float eps;
    const unsigned int *amax_in;
    unsigned int *amax_zero;
    // N-split over the GPUs of a node (bf16 output only): this launch computes rows of one shard;
    // every value is also stored into the same place of each peer's output buffer over NVLink, and
    // the last CTA to finish tells the peers and waits for their shards.  world <= 1: unused.
    int world, rank;
    uint16_t *peer_C[2][8];         // the two output buffers of every rank, used in turn ([b][rank] == C's twin)
    unsigned int *peer_flags[8];    // flag arrays [world] of the ranks; [rank] = the local one
    unsigned int *done;             // local: [0] counter of finished CTAs (zero between launches),
                                    //        [1] number of completed calls (the epoch; device-resident so
                                    //        that a captured graph can be replayed),
                                    //        [2] epoch of the last call whose wait for a peer ran out (0: none)
    unsigned int poll_limit;        // polls of one peer's flag before the wait is given up
};

struct GemvSmem {
    // Byte offsets into dynamic shared memory, computed identically on host and device.
    int act_stride, act_off, asum_off, stage_off, stage_bytes, row_stride, scale_off_in_stage,
        part_off, total;
};

__host__ __device__ inline GemvSmem gemv_smem_layout(int W, int K, int RB, int stages,
                                                     bool mma) {
    GemvSmem L;
    const int ng = K / BM_GROUP;
    const int R = 8 * RB;
    const int wrows = mma ? 16 : W;
    int off = 128;                                   // mbarriers live in the first 128 bytes
    L.act_stride = K + kActPad;
    L.act_off = off;
    off += wrows * L.act_stride;
    off = (off + 15) & ~15;
    L.asum_off = off;
    off += wrows * ng * 4;
    off = (off + 127) & ~127;
    L.row_stride = K / 4 + kRowPad;
    L.scale_off_in_stage = R * L.row_stride;
    L.stage_bytes = (L.scale_off_in_stage + R * ng * 2 + 127) & ~127;
    L.stage_off = off;
    off += stages * L.stage_bytes;
    L.part_off = off;
    if (mma) off += kGemvWarps * 16 * (R + 8) * 4;   // [warp][token][R+8] fp32 partials
    L.total = off;
    return L;
}

// ---- tile producer -----------------------------------------------------------
// Called by warp 0.  Rows [n0, n0 + rows) with rows a multiple of 8.
__device__ __forceinline__ void gemv_issue_tile(const GemvParams &p, unsigned char *stage,
                                                const GemvSmem &L, uint64_t *bar, int n0,
                                                int rows, int lane) {
    const int ng = p.K / BM_GROUP;
    const uint32_t row_bytes = (uint32_t)(p.K / 4);
    if (lane == 0) mbar_expect_tx(bar, (uint32_t)rows * row_bytes + (uint32_t)(rows * ng * 2));
    __syncwarp();
    if (p.silu_F == 0) {
        for (int r = lane; r < rows; r += 32)
            bulk_g2s(stage + r * L.row_stride, p.B + (size_t)(n0 + r) * row_bytes, row_bytes, bar);
        if (lane == 0)
            bulk_g2s(stage + L.scale_off_in_stage, p.ws + (size_t)n0 * ng, (uint32_t)(rows * ng * 2), bar);
    } else {
        // paired tile: rows [0, rows/2) are gate rows n0.., rows [rows/2, rows) the up rows of the same columns
        const int half = rows >> 1;
        for (int r = lane; r < rows; r += 32) {
            const size_t src = r < half ? (size_t)(n0 + r) : (size_t)(p.silu_F + n0 + r - half);
            bulk_g2s(stage + r * L.row_stride, p.B + src * row_bytes, row_bytes, bar);
        }
        if (lane == 0) {
            bulk_g2s(stage + L.scale_off_in_stage, p.ws + (size_t)n0 * ng, (uint32_t)(half * ng * 2), bar);
            bulk_g2s(stage + L.scale_off_in_stage + half * ng * 2, p.ws + (size_t)(p.silu_F + n0) * ng,
                     (uint32_t)(half * ng * 2), bar);
        }
    }
}

// ---- activation staging --------------------------------------------------------
// A (natural order, global) -> shared, 4x4 byte transpose per 16 elements, plus
// per-(token, group) sums.  `wrows` rows are written; rows >= W are zero.
__device__ __forceinline__ void gemv_stage_activations(const GemvParams &p, unsigned char *smem,
                                                       const GemvSmem &L, int wrows) {
    const int ng = p.K / BM_GROUP;
    int *asum = reinterpret_cast<int *>(smem + L.asum_off);
    for (int i = threadIdx.x; i < wrows * ng; i += blockDim.x) asum[i] = 0;
    __syncthreads();
    const int units = p.K / 16;
    for (int i = threadIdx.x; i < wrows * units; i += blockDim.x) {
        const int m = i / units, j = i - m * units;
        uint4 x = make_uint4(0u, 0u, 0u, 0u);
        if (m < p.W) x = *reinterpret_cast<const uint4 *>(p.A + (size_t)m * p.K + 16 * j);
        const uint32_t lo01 = __byte_perm(x.x, x.y, 0x5140), lo23 = __byte_perm(x.z, x.w, 0x5140);
        const uint32_t hi01 = __byte_perm(x.x, x.y, 0x7362), hi23 = __byte_perm(x.z, x.w, 0x7362);
        uint4 y;
        y.x = __byte_perm(lo01, lo23, 0x5410);
        y.y = __byte_perm(lo01, lo23, 0x7632);
        y.z = __byte_perm(hi01, hi23, 0x5410);
        y.w = __byte_perm(hi01, hi23, 0x7632);
        *reinterpret_cast<uint4 *>(smem + L.act_off + m * L.act_stride + 16 * j) = y;
        int sum = __dp4a((int)x.x, 0x01010101, 0);
        sum = __dp4a((int)x.y, 0x01010101, sum);
        sum = __dp4a((int)x.z, 0x01010101, sum);
        sum = __dp4a((int)x.w, 0x01010101, sum);
        if (m < p.W) atomicAdd(&asum[m * ng + (j >> 3)], sum);
    }
}

__device__ __forceinline__ void gemv_store(const GemvParams &p, int m, int n, float y) {
    if (p.out_kind == 0) {
        const uint16_t v = bm_f32_to_bf16(y);
        if (p.world > 1) {
            const int b = (int)((p.done[1] + 1u) & 1u);       // buffer of this call
            for (int r = 0; r < p.world; ++r) p.peer_C[b][r][(size_t)m * p.ldc + n] = v;
        } else {
            reinterpret_cast<uint16_t *>(p.C)[(size_t)m * p.ldc + n] = v;
        }
        return;
    }
    if (p.out_kind == 1)
        reinterpret_cast<float *>(p.C)[(size_t)m * p.ldc + n] = y;
    else
        reinterpret_cast<float *>(p.C)[(size_t)m * p.ldc + n] = bm_bf16_rn(y);
}

// ---- N-split hand-off ------------------------------------------------------------------------------
// Called by every CTA at the end of a launch with world > 1.  The last CTA to arrive knows that the
// whole shard has been stored (locally and into the peers' buffers), publishes `epoch` in its slot of
// every peer's flag array with system-scope release, and waits, with a limit, until every peer has
// published the same epoch here: when the kernel ends, the full output is in this GPU's buffer.
enum : int { kErrPeerWaitTimeout = 4 };

__device__ __forceinline__ void gemv_peer_finish(const GemvParams &p) {
    if (p.world <= 1) return;
    __syncthreads();
    if (threadIdx.x != 0) return;
    __threadfence_system();
    const unsigned int old = atomicAdd(&p.done[0], 1u);
    if (old != gridDim.x - 1) return;
    // last CTA: every other CTA has stored its part (and read the epoch) before it arrived
    atomicExch(&p.done[0], 0u);
    const unsigned int epoch = p.done[1] + 1u;
    __threadfence_system();
    for (int r = 0; r < p.world; ++r)
        if (r != p.rank)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.peer_flags[r] + p.rank), "r"(epoch) : "memory");
    for (int r = 0; r < p.world; ++r) {
        if (r == p.rank) continue;
        const unsigned int *flag = p.peer_flags[p.rank] + r;
        unsigned int spins = 0;
        for (;;) {
            unsigned int v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if ((int)(v - epoch) >= 0) break;
            if (++spins > p.poll_limit) {
                // give up: the caller finds the call number in done[2] (the output then holds stale
                // columns of that peer) and the device error word says why
                report_error(kErrPeerWaitTimeout);
                p.done[2] = epoch;
                break;
            }
            __nanosleep(100);
        }
    }
    p.done[1] = epoch;                               // the next launch (stream order) uses the other buffer
}

// =============================================================================
// Consumer 1: lanes across K, dp4a.  WB tokens per pass (W is covered in
// ceil(W/WB) passes over the staged tile), RB row-blocks of 8 rows per tile;
// warp w owns rows rb*8 + w.
// =============================================================================
template <int WB, int RB>
__global__ void __launch_bounds__(kGemvThreads) t2_gemv_dp4a_kernel(const GemvParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    const GemvSmem L = gemv_smem_layout(p.W, p.K, RB, p.stages, false);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ng = p.K / BM_GROUP;
    const int R = 8 * RB;
    const int n_tiles = (p.N + R - 1) / R;
    const int units = p.K / 64;                       // 16-byte pieces per row
    const int nch = (units + 31) / 32;                // 2048-element chunks

    if (threadIdx.x == 0) {
        for (int i = 0; i < p.stages; ++i) mbar_init(&bars[i], 1);
        mbar_fence_init();
    }
    __syncthreads();

    // Weights do not depend on the previous kernel: request them first.
    int my_tiles = 0;
    for (int t = blockIdx.x; t < n_tiles; t += gridDim.x) ++my_tiles;
    if (warp == 0) {
        for (int i = 0; i < p.stages - 1 && i < my_tiles; ++i) {
            const int n0 = (blockIdx.x + i * gridDim.x) * R;
            gemv_issue_tile(p, smem + L.stage_off + i * L.stage_bytes, L, &bars[i], n0,
                            min(R, p.N - n0), lane);
        }
    }
    pdl_launch_dependents();
    if (p.pdl) pdl_wait();
    gemv_stage_activations(p, smem, L, p.W);
    __syncthreads();

    const int *asum = reinterpret_cast<const int *>(smem + L.asum_off);
    const int slot_lane = lane >> 1;                  // slot this lane accumulates

    for (int i = 0; i < my_tiles; ++i) {
        const int st = i % p.stages;
        if (warp == 0) {
            const int nx = i + p.stages - 1;
            if (nx < my_tiles) {
                const int n0 = (blockIdx.x + nx * gridDim.x) * R;
                gemv_issue_tile(p, smem + L.stage_off + (nx % p.stages) * L.stage_bytes, L,
                                &bars[nx % p.stages], n0, min(R, p.N - n0), lane);
            }
        }
        const bool ok = mbar_wait_bounded(&bars[st], (uint32_t)((i / p.stages) & 1));
        if (__syncthreads_or(!ok)) {
            // Give up: record it, give copies still in flight a last bounded chance
            // to land in this CTA's shared memory, and leave.
            if (threadIdx.x == 0) {
                report_error(kErrGemvWaitTimeout);
                for (int j = i; j < my_tiles && j < i + p.stages - 1; ++j)
                    for (int it = 0; it < (1 << 12); ++it)
                        if (mbar_try_wait(&bars[j % p.stages], (uint32_t)((j / p.stages) & 1))) break;
            }
            break;
        }
        const unsigned char *stage = smem + L.stage_off + st * L.stage_bytes;
        const uint16_t *sc = reinterpret_cast<const uint16_t *>(stage + L.scale_off_in_stage);
        const int n0 = (blockIdx.x + i * gridDim.x) * R;
        const int rows = min(R, p.N - n0);

        for (int m0 = 0; m0 < p.W; m0 += WB) {
            float acc[RB][WB];
#pragma unroll
            for (int rb = 0; rb < RB; ++rb)
#pragma unroll
                for (int m = 0; m < WB; ++m) acc[rb][m] = 0.0f;

            for (int c = 0; c < nch; ++c) {
                const int u = c * 32 + lane;
                const bool active = u < units;
                const int g = u >> 1;
                uint4 a[WB][4];
#pragma unroll
                for (int m = 0; m < WB; ++m) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) a[m][j] = make_uint4(0u, 0u, 0u, 0u);
                    if (active && m0 + m < p.W) {
                        const uint4 *ap = reinterpret_cast<const uint4 *>(
                            smem + L.act_off + (m0 + m) * L.act_stride + 64 * u);
#pragma unroll
                        for (int j = 0; j < 4; ++j) a[m][j] = ap[j];
                    }
                }
#pragma unroll
                for (int rb = 0; rb < RB; ++rb) {
                    const int r = rb * 8 + warp;
                    if (r >= rows) continue;          // warp-uniform
                    uint4 w4 = make_uint4(0u, 0u, 0u, 0u);
                    if (active)
                        w4 = *reinterpret_cast<const uint4 *>(stage + r * L.row_stride + 16 * u);
                    const uint32_t wv[4] = {w4.x, w4.y, w4.z, w4.w};
                    int dot[WB];
#pragma unroll
                    for (int m = 0; m < WB; ++m) dot[m] = 0;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t c0 = wv[j] & 0x03030303u, c1 = (wv[j] >> 2) & 0x03030303u,
                                       c2 = (wv[j] >> 4) & 0x03030303u,
                                       c3 = (wv[j] >> 6) & 0x03030303u;
#pragma unroll
                        for (int m = 0; m < WB; ++m) {
                            const uint4 av = a[m][j];
                            dot[m] = __dp4a((int)av.x, (int)c0, dot[m]);
                            dot[m] = __dp4a((int)av.y, (int)c1, dot[m]);
                            dot[m] = __dp4a((int)av.z, (int)c2, dot[m]);
                            dot[m] = __dp4a((int)av.w, (int)c3, dot[m]);
                        }
                    }
                    const float scale = active ? bf16_bits_to_f32(sc[r * ng + g]) : 0.0f;
#pragma unroll
                    for (int m = 0; m < WB; ++m) {
                        const int both = dot[m] + __shfl_xor_sync(0xffffffffu, dot[m], 1);
                        if (active && m0 + m < p.W) {
                            const int G = both - 2 * asum[(m0 + m) * ng + g];
                            acc[rb][m] = fmaf((float)G, scale, acc[rb][m]);
                            if (p.G != nullptr && (lane & 1) == 0)
                                p.G[((size_t)(m0 + m) * p.N + n0 + r) * ng + g] = G;
                        }
                    }
                }
            }
            // Slot tree: lane bits 1..4 are slot bits 0..3.
#pragma unroll
            for (int rb = 0; rb < RB; ++rb) {
                const int r = rb * 8 + warp;
                if (r >= rows) continue;
#pragma unroll
                for (int m = 0; m < WB; ++m) {
                    float v = acc[rb][m];
                    v = v + __shfl_xor_sync(0xffffffffu, v, 2);
                    v = v + __shfl_xor_sync(0xffffffffu, v, 4);
                    v = v + __shfl_xor_sync(0xffffffffu, v, 8);
                    v = v + __shfl_xor_sync(0xffffffffu, v, 16);
                    if (lane == m && m0 + m < p.W) gemv_store(p, m0 + m, n0 + r, v * (1.0f / p.s[m0 + m]));
                }
            }
        }
        (void)slot_lane;
        __syncthreads();                              // stage st may be refilled next iteration
    }
}

// ---- width-1 activations made by the GEMV itself (src_mode 1 / 2) -------------------------------
// All kGemvThreads threads call this.  Leaves the GEMV-ready codes of token 0 in the staging row, its
// group sums and 1/s in shared memory.  `sh`: 32 floats of scratch.
__device__ __forceinline__ void gemv_stage_row_from_bf16(const GemvParams &p, unsigned char *smem, int act_off,
                                                         int asum_off, int invs_off, float *sh) {
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, nwarps = kGemvThreads / 32;
    const QuantSink sink{nullptr, reinterpret_cast<int8_t *>(smem + act_off), reinterpret_cast<int32_t *>(smem + asum_off)};
    float *invs = reinterpret_cast<float *>(smem + invs_off);
    float s;
    if (p.src_mode == 2) {
        const uint4 wraw = reinterpret_cast<const uint4 *>(p.norm_w)[t];
        const size_t src_row = p.gather ? gather_row(p.gather[0], p.gather_rows) : 0;
        float h[8];
        unpack8(reinterpret_cast<const uint4 *>(p.xb + src_row * p.K)[t], h);
        if (p.res) {
            float rr[8];
            unpack8(reinterpret_cast<const uint4 *>(p.res)[t], rr);
#pragma unroll
            for (int i = 0; i < 8; ++i) h[i] = bm_bf16_rn(h[i] + rr[i]);
        }
        if (blockIdx.x == 0 && p.h_out) reinterpret_cast<uint4 *>(p.h_out)[t] = pack8(h);
        float acc = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = fmaf(h[i], h[i], acc);
        const float total = block_sum_ordered(warp_sum_butterfly(acc), sh, lane, warp, nwarps);
        const float rs = bm_rsqrtf(total / (float)p.K + p.eps);
        float wv[8], n[8];
        unpack8(wraw, wv);
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            n[i] = bm_bf16_rn(wv[i] * bm_bf16_rn(h[i] * rs));
            amax = fmaxf(amax, fabsf(n[i]));
        }
        amax = block_max(amax, sh, lane, warp, nwarps);
        s = bm_act_scale(amax);
        emit_codes(sink, 0, p.K, t, quant8(n, s), true, lane);
    } else {
        s = bm_act_scale(__uint_as_float(p.amax_in[0]));
        for (int i = t; i < p.K / 8; i += kGemvThreads) {          // K % 256 == 0: whole warps
            float v[8];
            unpack8(reinterpret_cast<const uint4 *>(p.xb)[i], v);
            emit_codes(sink, 0, p.K, i, quant8(v, s), true, lane);
        }
        if (blockIdx.x == 0 && t == 0 && p.amax_zero) p.amax_zero[0] = 0u;
    }
    if (t < 16) invs[t] = t == 0 ? 1.0f / s : 0.0f;
}

// =============================================================================
// Consumer 2: tokens as the MMA rows, mma.sync.m16n8k32 s8 x u8 -> s32.
//
// Warp w owns scale slots 2w and 2w+1 (groups g with g%16 in {2w, 2w+1}) for
// every row of the tile; lane (r = lane/4, q = lane%4) supplies, per group, the
// 32 codes at k = 32q..32q+31 of output row n0 + rb*8 + r as the B fragment and
// the same 32 activations of tokens r and r+8 as the A fragment, and receives
// the group sums of tokens {r, r+8} x rows {2q, 2q+1}.  The first MMA of a
// group takes -2*sum(A) as its C operand, so the int32 fragment that comes out
// of the fourth MMA is the exact group sum of A * (code - 2).
//
// Everything that can be decided at compile time is: RB row-blocks per tile
// (N % (8*RB) == 0 is guaranteed by the host), HALF (W <= 8: tokens r+8 do not
// exist), ONECHUNK (K == 2048: one group per slot, activation fragments loaded
// once per CTA), EMIT_G (test build that also stores the group sums).  The
// profile of the first version showed the kernel bound by instruction issue,
// two thirds of it addressing and shape checks.
// Requires K % 256 == 0.
// =============================================================================
struct MmaSmem {
    int invs_off, act_stride, act_off, asum_off, stage_off, stage_bytes, row_stride,
        scale_off_in_stage, part_off, part_buf_floats, total;
};

__host__ __device__ inline MmaSmem mma_smem_layout(int K, int RB, int stages, bool half) {
    MmaSmem L;
    const int ng = K / BM_GROUP, R = 8 * RB, wrows = half ? 8 : 16;
    int off = 128;
    L.invs_off = off;
    off += 64;
    L.act_stride = K + kActPad;
    L.act_off = off;
    off += wrows * L.act_stride;
    off = (off + 15) & ~15;
    L.asum_off = off;
    off += wrows * ng * 4;
    off = (off + 127) & ~127;
    L.row_stride = K / 4 + kRowPad;
    L.scale_off_in_stage = R * L.row_stride;
    L.stage_bytes = (L.scale_off_in_stage + R * ng * 2 + 127) & ~127;
    L.stage_off = off;
    off += stages * L.stage_bytes;
    L.part_off = off;
    L.part_buf_floats = kGemvWarps * wrows * (R + 8);
    off += 2 * L.part_buf_floats * 4;                 // double-buffered partials
    L.total = off;
    return L;
}

__device__ __forceinline__ void mma_s8u8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1, int c0, int c1,
                                         int c2, int c3) {
    // Not volatile: the four MMAs of a group form a dependent chain, and the compiler must be
    // free to interleave the chains of different groups and row-blocks.
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
}

template <bool HALF>
struct AFrag {
    uint4 lo0, hi0;   // token r   : the four MMA steps' k-slots 4q.. and 16+4q..
    uint4 lo8, hi8;   // token r+8 (unused when HALF)
    int nb0, nb8;     // kGroupSumBias - 2 * sum(A) over the group, tokens r and r+8
};

// Fragments of group g for tokens r and r+8 from rows of `stride` bytes (shared-memory
// staging area, or the caller's GEMV-ready activations in global memory).  Tokens >= W
// give zeros.
template <bool HALF>
__device__ __forceinline__ void load_afrag(AFrag<HALF> &f, const unsigned char *rows, int stride,
                                           const int *asum, int W, int ng, int g, int r, int q) {
    f.lo0 = f.hi0 = f.lo8 = f.hi8 = make_uint4(0u, 0u, 0u, 0u);
    f.nb0 = f.nb8 = kGroupSumBias;
    if (r < W) {
        const uint4 *ap = reinterpret_cast<const uint4 *>(rows + (size_t)r * stride + BM_GROUP * g + 32 * q);
        f.lo0 = ap[0];
        f.hi0 = ap[1];
        f.nb0 = kGroupSumBias - 2 * asum[r * ng + g];
    }
    if (!HALF && r + 8 < W) {
        const uint4 *ap8 = reinterpret_cast<const uint4 *>(rows + (size_t)(r + 8) * stride + BM_GROUP * g + 32 * q);
        f.lo8 = ap8[0];
        f.hi8 = ap8[1];
        f.nb8 = kGroupSumBias - 2 * asum[(r + 8) * ng + g];
    }
}

// One group of one row-block: 4 MMAs, then acc += float(G) * scale.
template <bool HALF, bool EMIT_G>
__device__ __forceinline__ void mma_group_step(const AFrag<HALF> &f, uint2 w2, float s0, float s1,
                                               float (&acc)[4], int32_t *gdst0, int32_t *gdst8,
                                               int gstride) {
    constexpr uint32_t M3 = 0x03030303u;
    int d[4];
    mma_s8u8(d, f.lo0.x, f.lo8.x, f.hi0.x, f.hi8.x, w2.x & M3, w2.y & M3, f.nb0, f.nb0, f.nb8, f.nb8);
    mma_s8u8(d, f.lo0.y, f.lo8.y, f.hi0.y, f.hi8.y, (w2.x >> 2) & M3, (w2.y >> 2) & M3, d[0], d[1], d[2], d[3]);
    mma_s8u8(d, f.lo0.z, f.lo8.z, f.hi0.z, f.hi8.z, (w2.x >> 4) & M3, (w2.y >> 4) & M3, d[0], d[1], d[2], d[3]);
    mma_s8u8(d, f.lo0.w, f.lo8.w, f.hi0.w, f.hi8.w, (w2.x >> 6) & M3, (w2.y >> 6) & M3, d[0], d[1], d[2], d[3]);
    acc[0] = fmaf(group_sum_to_float(d[0]), s0, acc[0]);
    acc[1] = fmaf(group_sum_to_float(d[1]), s1, acc[1]);
    if (!HALF) {
        acc[2] = fmaf(group_sum_to_float(d[2]), s0, acc[2]);
        acc[3] = fmaf(group_sum_to_float(d[3]), s1, acc[3]);
    }
    if (EMIT_G) {
        if (gdst0) { gdst0[0] = d[0] - kGroupSumBias; gdst0[gstride] = d[1] - kGroupSumBias; }
        if (!HALF && gdst8) { gdst8[0] = d[2] - kGroupSumBias; gdst8[gstride] = d[3] - kGroupSumBias; }
    }
}

template <int RB, bool HALF, bool ONECHUNK, bool EMIT_G>
__global__ void __launch_bounds__(kGemvThreads, 2) t2_gemv_mma_kernel(const GemvParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int R = 8 * RB, RP = R + 8, WROWS = HALF ? 8 : 16;
    const int ng = p.K / BM_GROUP;
    const MmaSmem L = mma_smem_layout(p.K, RB, p.stages, HALF);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int r = lane >> 2, q = lane & 3;
    const int R_out = p.silu_F ? R / 2 : R;            // output columns per tile
    const int n_tiles = p.N / R_out;
    const int nch = ONECHUNK ? 1 : (ng + BM_SLOTS - 1) / BM_SLOTS;
    __shared__ unsigned int amax_sh[16];
    if (p.silu_F && threadIdx.x < 16) amax_sh[threadIdx.x] = 0u;

    if (threadIdx.x == 0) {
        for (int i = 0; i < p.stages; ++i) mbar_init(&bars[i], 1);
        mbar_init(&bars[kMaxStages], 1);              // activation rows (several-chunk, prepared)
        mbar_fence_init();
    }
    __syncthreads();

    // Weights do not depend on the previous kernel in the stream: request them first.
    const int my_tiles = (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    GemvSmem LS;                                      // the producer only needs these fields
    LS.row_stride = L.row_stride;
    LS.scale_off_in_stage = L.scale_off_in_stage;
    if (warp == 0) {
        for (int i = 0; i < p.stages && i < my_tiles; ++i)
            gemv_issue_tile(p, smem + L.stage_off + i * L.stage_bytes, LS, &bars[i],
                            (blockIdx.x + i * gridDim.x) * R_out, R, lane);
    }
    pdl_launch_dependents();
    if (p.pdl) pdl_wait();
    const bool prepared = p.asum != nullptr;
    // Where fragments come from: the caller's GEMV-ready rows (one chunk: straight from
    // global memory, nothing is staged), or the shared-memory staging area.
    const unsigned char *arows = smem + L.act_off;
    int astride = L.act_stride;
    const int *asum = reinterpret_cast<const int *>(smem + L.asum_off);
    uint64_t *abar = bars + kMaxStages;
    bool a_ok = true;
    {
        float *invs_w = reinterpret_cast<float *>(smem + L.invs_off);
        if (p.src_mode == 0 && threadIdx.x < 16) invs_w[threadIdx.x] = threadIdx.x < p.W ? 1.0f / p.s[threadIdx.x] : 0.0f;
        if (p.src_mode != 0) {
            __shared__ float stage_sh[32];
            gemv_stage_row_from_bf16(p, smem, L.act_off, L.asum_off, L.invs_off, stage_sh);
        } else if (!prepared) {
            GemvSmem LA;
            LA.act_off = L.act_off;
            LA.act_stride = L.act_stride;
            LA.asum_off = L.asum_off;
            gemv_stage_activations(p, smem, LA, WROWS);
        } else if (ONECHUNK) {
            arows = reinterpret_cast<const unsigned char *>(p.A);
            astride = p.K;
            asum = p.asum;
        } else {
            // several chunks: the rows are copied in bulk (no permutation left to do)
            if (warp == 1) {
                if (lane == 0) mbar_expect_tx(abar, (uint32_t)p.W * (uint32_t)p.K);
                __syncwarp();
                if (lane < p.W)
                    bulk_g2s(smem + L.act_off + lane * L.act_stride, p.A + (size_t)lane * p.K,
                             (uint32_t)p.K, abar);
            }
            int *as = reinterpret_cast<int *>(smem + L.asum_off);
            for (int i2 = threadIdx.x; i2 < p.W * ng; i2 += kGemvThreads) as[i2] = p.asum[i2];
            a_ok = mbar_wait_bounded(abar, 0u);
        }
    }
    __syncthreads();

    AFrag<HALF> fA, fB;
    if (ONECHUNK) {
        load_afrag<HALF>(fA, arows, astride, asum, p.W, ng, 2 * warp, r, q);
        load_afrag<HALF>(fB, arows, astride, asum, p.W, ng, 2 * warp + 1, r, q);
    }
    float *part = reinterpret_cast<float *>(smem + L.part_off);
    const float *invs = reinterpret_cast<const float *>(smem + L.invs_off);
    // Per-thread offsets inside a stage: weight bytes of row r at k-quarter q, and the
    // packed scale pair of rows 2q / 2q+1 for this warp's two slots.
    const int woff = r * L.row_stride + 8 * q + 64 * warp;
    const int soff = L.scale_off_in_stage + (2 * q * ng + 2 * warp) * 2;
    bool failed = false;

    for (int i = 0; i < my_tiles; ++i) {
        const int st = i % p.stages;
        const bool ok = mbar_wait_bounded(&bars[st], (uint32_t)((i / p.stages) & 1)) && a_ok;
        const unsigned char *stage = smem + L.stage_off + st * L.stage_bytes;
        const int n0 = (blockIdx.x + i * gridDim.x) * R_out;

        float acc[RB][2][4];
#pragma unroll
        for (int rb = 0; rb < RB; ++rb)
#pragma unroll
            for (int sl = 0; sl < 2; ++sl)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[rb][sl][e] = 0.0f;

        if (ok) {
            for (int c = 0; c < nch; ++c) {
                const int g0 = c * BM_SLOTS + 2 * warp;
                if (!ONECHUNK) {
                    if (g0 >= ng) break;              // warp-uniform
                    load_afrag<HALF>(fA, arows, astride, asum, p.W, ng, g0, r, q);
                    load_afrag<HALF>(fB, arows, astride, asum, p.W, ng, g0 + 1, r, q);
                }
                const unsigned char *wp = stage + woff + c * (32 * BM_SLOTS);
                const unsigned char *sp = stage + soff + c * (2 * BM_SLOTS);
#pragma unroll
                for (int rb = 0; rb < RB; ++rb) {
                    const uint2 wA = *reinterpret_cast<const uint2 *>(wp + rb * 8 * L.row_stride);
                    const uint2 wB = *reinterpret_cast<const uint2 *>(wp + rb * 8 * L.row_stride + 32);
                    const uint32_t x0 = *reinterpret_cast<const uint32_t *>(sp + rb * 8 * ng * 2);
                    const uint32_t x1 = *reinterpret_cast<const uint32_t *>(sp + rb * 8 * ng * 2 + ng * 2);
                    int32_t *g0p = nullptr, *g8p = nullptr;
                    if (EMIT_G) {
                        const size_t col = (size_t)(n0 + rb * 8 + 2 * q) * ng + g0;
                        if (r < p.W) g0p = p.G + (size_t)r * p.N * ng + col;
                        if (r + 8 < p.W) g8p = p.G + (size_t)(r + 8) * p.N * ng + col;
                    }
                    mma_group_step<HALF, EMIT_G>(fA, wA, __uint_as_float(x0 << 16),
                                                 __uint_as_float(x1 << 16), acc[rb][0], g0p, g8p, ng);
                    mma_group_step<HALF, EMIT_G>(fB, wB, __uint_as_float(x0 & 0xffff0000u),
                                                 __uint_as_float(x1 & 0xffff0000u), acc[rb][1],
                                                 g0p ? g0p + 1 : nullptr, g8p ? g8p + 1 : nullptr, ng);
                }
            }
        }
        // Slots 2w + (2w+1) inside the thread, the other three tree levels through
        // shared memory: part[buf][warp][token][row].
        float *pw = part + (i & 1) * L.part_buf_floats + warp * WROWS * RP;
#pragma unroll
        for (int rb = 0; rb < RB; ++rb) {
            const int row0 = rb * 8 + 2 * q;
            *reinterpret_cast<float2 *>(&pw[r * RP + row0]) =
                make_float2(acc[rb][0][0] + acc[rb][1][0], acc[rb][0][1] + acc[rb][1][1]);
            if (!HALF)
                *reinterpret_cast<float2 *>(&pw[(r + 8) * RP + row0]) =
                    make_float2(acc[rb][0][2] + acc[rb][1][2], acc[rb][0][3] + acc[rb][1][3]);
        }
        if (__syncthreads_or(!ok)) {
            // Give up: record it, give copies still in flight a last bounded chance to land
            // in this CTA's shared memory, and leave.
            failed = true;
            if (threadIdx.x == 0) {
                report_error(kErrGemvWaitTimeout);
                for (int j = i; j < my_tiles && j < i + p.stages; ++j)
                    for (int it = 0; it < (1 << 12); ++it)
                        if (mbar_try_wait(&bars[j % p.stages], (uint32_t)((j / p.stages) & 1))) break;
            }
            break;
        }
        // Every warp is done with stage `st`: refill it with the tile `stages` ahead.
        if (warp == 0 && i + p.stages < my_tiles)
            gemv_issue_tile(p, smem + L.stage_off + st * L.stage_bytes, LS, &bars[st],
                            (blockIdx.x + (i + p.stages) * gridDim.x) * R_out, R, lane);
        // Remaining tree levels, reciprocal multiply, store.  Thread = (token, 4 rows).
        const float *pr = part + (i & 1) * L.part_buf_floats;
        if (p.silu_F) {
            // rows [0, R/2) of the tile are gate rows, rows [R/2, R) the up rows of the same columns:
            // inner = bf16(silu(bf16 gate) * bf16 up), as the stand-alone SiLU kernel computes it from
            // the bf16 projection outputs
            // one output element per thread: the SiLU (own exp, IEEE division) is a long dependent chain
            for (int o = threadIdx.x; o < p.W * (R / 2); o += kGemvThreads) {
                const int m = o / (R / 2), c = o - m * (R / 2);
                float vg[kGemvWarps], vu[kGemvWarps];
#pragma unroll
                for (int w = 0; w < kGemvWarps; ++w) {
                    vg[w] = pr[(w * WROWS + m) * RP + c];
                    vu[w] = pr[(w * WROWS + m) * RP + R / 2 + c];
                }
                const float is = invs[m];
                const float g = (((vg[0] + vg[1]) + (vg[2] + vg[3])) + ((vg[4] + vg[5]) + (vg[6] + vg[7]))) * is;
                const float u = (((vu[0] + vu[1]) + (vu[2] + vu[3])) + ((vu[4] + vu[5]) + (vu[6] + vu[7]))) * is;
                const float v = bm_bf16_rn(bm_silu_bf16(bm_bf16_rn(g)) * bm_bf16_rn(u));
                reinterpret_cast<uint16_t *>(p.C)[(size_t)m * p.ldc + n0 + c] = bm_f32_to_bf16(v);
                atomicMax(&amax_sh[m], __float_as_uint(fabsf(v)));
            }
            continue;
        }
        for (int o = threadIdx.x; o < p.W * (R / 4); o += kGemvThreads) {
            const int m = o / (R / 4), rq = o - m * (R / 4);
            float4 v[kGemvWarps];
#pragma unroll
            for (int w = 0; w < kGemvWarps; ++w)
                v[w] = *reinterpret_cast<const float4 *>(&pr[(w * WROWS + m) * RP + 4 * rq]);
            const float is = invs[m];
            float y[4];
#define BM_TREE(F) (((v[0].F + v[1].F) + (v[2].F + v[3].F)) + ((v[4].F + v[5].F) + (v[6].F + v[7].F))) * is
            y[0] = BM_TREE(x); y[1] = BM_TREE(y); y[2] = BM_TREE(z); y[3] = BM_TREE(w);
#undef BM_TREE
            const size_t dst = (size_t)m * p.ldc + n0 + 4 * rq;
            if (p.out_kind == 0) {
                const uint32_t lo = (uint32_t)bm_f32_to_bf16(y[0]) | ((uint32_t)bm_f32_to_bf16(y[1]) << 16);
                const uint32_t hi = (uint32_t)bm_f32_to_bf16(y[2]) | ((uint32_t)bm_f32_to_bf16(y[3]) << 16);
                if (p.world > 1) {
                    const int b = (int)((p.done[1] + 1u) & 1u);   // buffer of this call
                    for (int pr = 0; pr < p.world; ++pr)
                        *reinterpret_cast<uint2 *>(p.peer_C[b][pr] + dst) = make_uint2(lo, hi);
                } else {
                    *reinterpret_cast<uint2 *>(reinterpret_cast<uint16_t *>(p.C) + dst) = make_uint2(lo, hi);
                }
            } else {
                if (p.out_kind == 2) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) y[e] = bm_bf16_rn(y[e]);
                }
                *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p.C) + dst) =
                    make_float4(y[0], y[1], y[2], y[3]);
            }
        }
    }
    (void)failed;
    if (p.silu_F) {
        __syncthreads();
        if (threadIdx.x < p.W && amax_sh[threadIdx.x] != 0u) atomicMax(&p.amax_out[threadIdx.x], amax_sh[threadIdx.x]);
    }
    gemv_peer_finish(p);
}

}  // namespace bm
