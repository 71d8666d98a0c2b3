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
// dimension (s8 activations as B); four MMAs cover a 128-group with bias - 2 * sum(a) as the first C
// operand, so the int32 fragment is the exact group sum plus the bias that turns it into a float.  The 2-bit -> 8-bit expansion happens in
// registers, once per group and warp, and is reused by the 32 prompt rows of the tile.
//
// fp32 order (the GEMV's, see the header of t2_gemv.cuh): group g -> slot g % 16, slot = fma(G,
// scale, slot) in ascending g, the 16 slots summed as a butterfly tree, times 1/s.  A wide tile cannot
// hold 16 slot accumulators per output, so the groups are visited SLOT BY SLOT (s, s+16, s+32, ...:
// one accumulator), and a finished slot is folded into a binary-counter tree (4 registers per output)
// whose additions are exactly the butterfly's.
//
// CTA = 8 warps = 128 weight rows x 32 prompt rows.  The groups are taken in the slot-major sequence
// (slot 0's groups, slot 1's, ...) in stages of kWideStageGroups: activations [32 rows][128 B per group]
// and codes [128 rows][32 B per group] arrive by 16-byte asynchronous copies into a ring of kWideStages
// buffers, the next stage loading while the current one is multiplied (one CTA barrier per stage); the
// bf16 scales of the CTA's 128 rows and the C operands (bias - 2 * sum(a)) of its 32 prompt rows are
// tables loaded once.  Two CTAs per SM.
#pragma once

#include "bm_common.cuh"
#include "t2_gemv_rowwarp.cuh"

namespace bm {

constexpr int kWideThreads = 256;
constexpr int kWideRows = 128;          // weight rows per CTA (16 per warp)
constexpr int kWideTokens = 32;         // prompt rows per CTA (4 MMA column blocks)
constexpr int kWideStageGroups = 4;     // groups per stage
constexpr int kWideStages = 2;          // stage buffers
// Strides chosen so that the fragment reads are free of bank conflicts: activation rows (16-byte reads of
// 8 rows x 4 quarters) want an odd number of 16-byte units, code rows (8-byte reads of 4 rows x 4
// quarters) 32 or 96 mod 128 bytes, the C-operand table (8-byte reads, stores along the group index) 34 words.
constexpr int kWideActStride = kWideStageGroups * 128 + 16;
constexpr int kWideCodeStride = kWideStageGroups * 32 + 32;
constexpr int kWideStageBytes = kWideTokens * kWideActStride + kWideRows * kWideCodeStride;
constexpr int kWideNbStride = kWideTokens + 2;
static_assert((kWideActStride / 16) % 2 == 1 && (kWideCodeStride % 128 == 32 || kWideCodeStride % 128 == 96),
              "bank-conflict-free strides");

struct WideParams {
    const int8_t *A;        // [T, K] GEMV-ready INT8 rows
    const int32_t *asum;    // [T, K/128]
    const float *s;         // [T]
    const uint8_t *B;       // [N, K/4]
    const uint16_t *ws;     // [N, K/128] bf16
    uint16_t *C;            // [T, ldc] bf16
    int T, N, K, ldc, pdl;
};

// Scale-table row stride in bf16 elements: ng + 2 makes the 32-bit word stride odd when ng % 4 == 0.
__host__ __device__ inline int wide_scale_stride(int ng) { return ng + 2; }

// `park`: the K = 2048 build parks the sum of slots 0-7 of every output in shared memory while slots 8-15 are
// multiplied (16 registers fewer where the tree is fullest).
__host__ __device__ inline size_t wide_smem_bytes(int ng, bool park = false) {
    size_t off = (size_t)kWideStages * kWideStageBytes;
    off += ((size_t)kWideRows * wide_scale_stride(ng) * 2 + 15) & ~(size_t)15;
    off += ((size_t)ng * kWideNbStride * 4 + 15) & ~(size_t)15;
    if (park) off += (size_t)kWideThreads * 16 * 4;
    return off;
}

// Position in the slot-major sequence of groups: slot s (0..15), term c; slot s has ceil((ng - s) / 16)
// groups s, s + 16, ...  `step` moves to the next position (warp-uniform integer work, no division).
struct WideSeq {
    int s, c;
    __device__ __forceinline__ int group() const { return s + BM_SLOTS * c; }
    __device__ __forceinline__ static int terms(int slot, int ng) { return (ng - slot + BM_SLOTS - 1) >> 4; }
    __device__ __forceinline__ bool step(int ng) {             // true when the slot was finished by this step
        if (++c < terms(s, ng)) return false;
        c = 0;
        ++s;
        return true;
    }
};

// Folds the finished slot S (compile-time) into the binary-counter tree of one output: level l holds the
// sum of a finished block of 2^l slots whose partner has not arrived yet; `left + right` with the earlier
// block on the left, which is the butterfly order ((s0+s1)+(s2+s3))+... of the GEMV.  Straight-line code:
// a run-time slot number here costs dozens of register moves per slot where the branches meet.
template <int S>
__device__ __forceinline__ void wide_tree_push(float (&tree)[4], float v) {
    if (S & 1) { v = tree[0] + v; } else { tree[0] = v; return; }
    if (S & 2) { v = tree[1] + v; } else { tree[1] = v; return; }
    if (S & 4) { v = tree[2] + v; } else { tree[2] = v; return; }
    if (S & 8) { v = tree[3] + v; } else { tree[3] = v; return; }
    tree[3] = v;            // S == 15: the total
}

// Shared-memory loads by 32-bit shared address (the multiply loop keeps its addresses in 32-bit registers
// with constant offsets instead of 64-bit generic pointers).
__device__ __forceinline__ uint2 wide_lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ uint4 wide_lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ float wide_lds_bf16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a) : "memory");
    return __uint_as_float((uint32_t)v << 16);
}

// One 128-group for this warp's 16 weight rows x the CTA's 32 prompt rows: unpack the codes once, then
// per block of 8 prompt rows four MMAs and `acc = fma((float)G, scale, acc)`.
//   wts   this lane's code bytes of the group (row g of the warp's 16; row g + 8 is 8 rows further)
//   act   this lane's activation bytes of the group (prompt row g of block 0)
//   nb    this lane's C operands of the group (prompt rows 2q, 2q + 1 of block 0)
__device__ __forceinline__ void wide_group(uint32_t wts, uint32_t act, uint32_t nb, float s0, float s8, float (&acc)[4][4]) {
    constexpr uint32_t M3 = 0x03030303u;
    const uint2 x = wide_lds64(wts);
    const uint2 y = wide_lds64(wts + 8 * kWideCodeStride);
    // A operands of the four MMAs.  Bit plane t of a code word (codes 4e + t of its 16-code runs) meets
    // activation word t of the same run; which two (plane, word) pairs share an MMA does not change the
    // integer sum, so they are paired such that every B operand is an aligned register pair of one
    // 16-byte activation load: (lo.x, lo.y), (lo.z, lo.w), (hi.x, hi.y), (hi.z, hi.w).
    uint32_t a[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t xw = j < 2 ? x.x : x.y, yw = j < 2 ? y.x : y.y;
        const int t = 2 * (j & 1);
        a[j][0] = (xw >> (2 * t)) & M3;
        a[j][1] = (yw >> (2 * t)) & M3;
        a[j][2] = (xw >> (2 * t + 2)) & M3;
        a[j][3] = (yw >> (2 * t + 2)) & M3;
    }
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const uint4 lo = wide_lds128(act + 8 * b * kWideActStride);
        const uint4 hi = wide_lds128(act + 8 * b * kWideActStride + 16);
        const uint2 c = wide_lds64(nb + 32 * b);
        int d[4];
        mma_u8s8(d, a[0][0], a[0][1], a[0][2], a[0][3], lo.x, lo.y, (int)c.x, (int)c.y, (int)c.x, (int)c.y);
        mma_u8s8(d, a[1][0], a[1][1], a[1][2], a[1][3], lo.z, lo.w, d[0], d[1], d[2], d[3]);
        mma_u8s8(d, a[2][0], a[2][1], a[2][2], a[2][3], hi.x, hi.y, d[0], d[1], d[2], d[3]);
        mma_u8s8(d, a[3][0], a[3][1], a[3][2], a[3][3], hi.z, hi.w, d[0], d[1], d[2], d[3]);
        acc[b][0] = fmaf(group_sum_to_float(d[0]), s0, acc[b][0]);
        acc[b][1] = fmaf(group_sum_to_float(d[1]), s0, acc[b][1]);
        acc[b][2] = fmaf(group_sum_to_float(d[2]), s8, acc[b][2]);
        acc[b][3] = fmaf(group_sum_to_float(d[3]), s8, acc[b][3]);
    }
}

// Requests of one group into position li of a stage buffer: every thread copies one 16-byte half of one
// code row (128 rows x 2) and one 16-byte piece of one prompt row (32 rows x 8).
__device__ __forceinline__ void wide_issue_codes(unsigned char *buf, int li, const uint8_t *src_row, int grp, int tid) {
    cp_async16(buf + kWideTokens * kWideActStride + (tid >> 1) * kWideCodeStride + li * 32 + 16 * (tid & 1), src_row + grp * 32);
}
__device__ __forceinline__ void wide_issue_row(unsigned char *buf, int li, const int8_t *src_row, int grp, int tid) {
    unsigned char *dst = buf + (tid >> 3) * kWideActStride + li * 128 + 16 * (tid & 7);
    if (src_row != nullptr) cp_async16(dst, src_row + grp * 128);
    else *reinterpret_cast<uint4 *>(dst) = make_uint4(0u, 0u, 0u, 0u);
}

// State of the copy pipeline.  Before the first group of stage st: the stage has landed - kWideStages
// batches are out at stage 0, kWideStages - 1 + st later, and only the ones after batch st may still be in
// flight; once every warp is past the barrier the buffer of stage st - 1 is free and takes stage
// st - 1 + kWideStages.
struct WidePipe {
    unsigned char *ring;
    const uint8_t *code_src;      // this thread's half of a code row, group 0
    const int8_t *row_src;        // this thread's piece of a prompt row, group 0 (null: past T)
    WideSeq prod;                 // next group to request
    int requested, ng;
};
__device__ __forceinline__ void wide_enter_stage(WidePipe &pp, int st) {
    const int tid = threadIdx.x;
    if (st == 0) cp_async_wait_batches<kWideStages - 1>();
    else cp_async_wait_batches<kWideStages - 2>();
    __syncthreads();
    if (st > 0) {
        unsigned char *buf = pp.ring + ((st - 1) % kWideStages) * kWideStageBytes;
        for (int li = 0; li < kWideStageGroups && pp.requested < pp.ng; ++li, ++pp.requested, pp.prod.step(pp.ng)) {
            wide_issue_codes(buf, li, pp.code_src, pp.prod.group(), tid);
            wide_issue_row(buf, li, pp.row_src, pp.prod.group(), tid);
        }
        cp_async_commit();
    }
}

// grid (N / 128, ceil(T / 32)), 256 threads.  K % 128 == 0, N % 128 == 0.
// ONE: K == 2048, one group per slot - the position in the sequence, its stage and its place in the stage are
// compile-time constants and the loop over a slot's groups disappears.
template <bool ONE>
__global__ void __launch_bounds__(kWideThreads, 2) t2_gemm_wide_kernel(const WideParams p) {
    extern __shared__ __align__(16) unsigned char wsm[];
    pdl_launch_dependents();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, q = lane & 3;
    const int ng = p.K / BM_GROUP, scs = wide_scale_stride(ng);
    const int n0 = blockIdx.x * kWideRows, t0 = blockIdx.y * kWideTokens;
    unsigned char *ring = wsm;
    uint16_t *sc_tab = reinterpret_cast<uint16_t *>(wsm + kWideStages * kWideStageBytes);
    int *nb_tab = reinterpret_cast<int *>(wsm + kWideStages * kWideStageBytes + (((size_t)kWideRows * scs * 2 + 15) & ~(size_t)15));
    float4 *parked = reinterpret_cast<float4 *>(reinterpret_cast<unsigned char *>(nb_tab) + (((size_t)ng * kWideNbStride * 4 + 15) & ~(size_t)15));
    // what this thread copies of every group: its half of a code row, its piece of a prompt row (null: past T)
    const uint8_t *code_src = p.B + (size_t)(n0 + (tid >> 1)) * (p.K / 4) + 16 * (tid & 1);
    const int8_t *row_src = t0 + (tid >> 3) < p.T ? p.A + (size_t)(t0 + (tid >> 3)) * p.K + 16 * (tid & 7) : nullptr;

    // Weights first: the codes of the whole ring and the scales do not depend on the previous kernel in
    // the stream.  Batch st of the asynchronous copies holds (at least) everything of stage st.
    {
        WideSeq w = {0, 0};
        for (int i = 0; i < kWideStages * kWideStageGroups && i < ng; ++i, w.step(ng))
            wide_issue_codes(ring + (i / kWideStageGroups) * kWideStageBytes, i % kWideStageGroups, code_src, w.group(), tid);
    }
    // (eight lanes walk one row's groups: no division by the run-time group count anywhere in this kernel)
#pragma unroll
    for (int j = 0; j < kWideRows / 32; ++j) {
        const int r = (tid >> 3) + 32 * j;
        for (int grp = tid & 7; grp < ng; grp += 8) sc_tab[r * scs + grp] = p.ws[(size_t)(n0 + r) * ng + grp];
    }
    if (p.pdl) pdl_wait();
    WidePipe pp = {ring, code_src, row_src, {0, 0}, 0, ng};
#pragma unroll
    for (int st = 0; st < kWideStages; ++st) {
        for (int li = 0; li < kWideStageGroups && pp.requested < ng; ++li, ++pp.requested, pp.prod.step(ng))
            wide_issue_row(ring + st * kWideStageBytes, li, row_src, pp.prod.group(), tid);
        cp_async_commit();
    }
    {
        const int r = tid >> 3;                                      // 32 prompt rows x 8 lanes
        const bool live = t0 + r < p.T;
        for (int grp = tid & 7; grp < ng; grp += 8)
            nb_tab[grp * kWideNbStride + r] = kGroupSumBias - 2 * (live ? p.asum[(size_t)(t0 + r) * ng + grp] : 0);
    }

    // 32-bit shared addresses of this lane's pieces: scales of rows g / g + 8, C operands of prompt rows
    // 2q / 2q + 1, code bytes and activation bytes of group 0 of stage buffer 0
    const uint32_t ring_s = (uint32_t)__cvta_generic_to_shared(ring);
    const uint32_t sc0 = (uint32_t)__cvta_generic_to_shared(sc_tab + (16 * warp + g) * scs), sc8 = sc0 + 16 * scs;
    const uint32_t nb0 = (uint32_t)__cvta_generic_to_shared(nb_tab + 2 * q);
    const uint32_t wbase = ring_s + kWideTokens * kWideActStride + (16 * warp + g) * kWideCodeStride + 8 * q;
    const uint32_t abase = ring_s + g * kWideActStride + 32 * q;
    int seq = 0;                             // position of the group being multiplied
    float tree[4][4][4];                     // [token block][fragment element][level]
    // The slots in ascending order, the slot number a compile-time constant for the tree; one copy of the
    // multiply per slot, its groups (s, s + 16, ...) in a run-time loop.
#define BM_WIDE_SLOT(S_)                                                                                          \
    {                                                                                                             \
        float acc[4][4];                                                                                          \
        _Pragma("unroll") for (int b = 0; b < 4; ++b)                                                             \
            _Pragma("unroll") for (int e = 0; e < 4; ++e) acc[b][e] = 0.0f;                                       \
        if (ONE) {                                                                                                \
            constexpr int st = S_ / kWideStageGroups, li = S_ % kWideStageGroups;                                 \
            constexpr uint32_t boff = (st % kWideStages) * kWideStageBytes;                                       \
            if (li == 0) wide_enter_stage(pp, st);                                                                \
            wide_group(wbase + boff + li * 32, abase + boff + li * 128, nb0 + S_ * (4 * kWideNbStride),           \
                       wide_lds_bf16(sc0 + 2 * S_), wide_lds_bf16(sc8 + 2 * S_), acc);                            \
        } else {                                                                                                  \
            const int nt = WideSeq::terms(S_, ng);                                                                \
            for (int c = 0; c < nt; ++c, ++seq) {                                                                 \
                const int st = seq / kWideStageGroups, li = seq % kWideStageGroups;                               \
                if (li == 0) wide_enter_stage(pp, st);                                                            \
                const uint32_t boff = (st % kWideStages) * kWideStageBytes;                                       \
                const int grp = S_ + BM_SLOTS * c;                                                                \
                wide_group(wbase + boff + li * 32, abase + boff + li * 128, nb0 + grp * (4 * kWideNbStride),      \
                           wide_lds_bf16(sc0 + 2 * grp), wide_lds_bf16(sc8 + 2 * grp), acc);                      \
            }                                                                                                     \
        }                                                                                                         \
        if (ONE && S_ == 15) {                                                                                    \
            _Pragma("unroll") for (int b = 0; b < 4; ++b) {                                                       \
                const float4 low = parked[b * kWideThreads + tid];                                                \
                tree[b][0][3] = low.x; tree[b][1][3] = low.y; tree[b][2][3] = low.z; tree[b][3][3] = low.w;       \
            }                                                                                                     \
        }                                                                                                         \
        _Pragma("unroll") for (int b = 0; b < 4; ++b)                                                             \
            _Pragma("unroll") for (int e = 0; e < 4; ++e) wide_tree_push<S_>(tree[b][e], acc[b][e]);              \
        if (ONE && S_ == 7) {                                                                                     \
            _Pragma("unroll") for (int b = 0; b < 4; ++b)                                                         \
                parked[b * kWideThreads + tid] = make_float4(tree[b][0][3], tree[b][1][3], tree[b][2][3], tree[b][3][3]); \
        }                                                                                                         \
    }
    BM_WIDE_SLOT(0) BM_WIDE_SLOT(1) BM_WIDE_SLOT(2) BM_WIDE_SLOT(3) BM_WIDE_SLOT(4) BM_WIDE_SLOT(5) BM_WIDE_SLOT(6)
    BM_WIDE_SLOT(7) BM_WIDE_SLOT(8) BM_WIDE_SLOT(9) BM_WIDE_SLOT(10) BM_WIDE_SLOT(11) BM_WIDE_SLOT(12)
    BM_WIDE_SLOT(13) BM_WIDE_SLOT(14) BM_WIDE_SLOT(15)
#undef BM_WIDE_SLOT
    // times 1/s of the prompt row, to bf16
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
