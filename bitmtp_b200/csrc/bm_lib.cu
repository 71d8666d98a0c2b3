// libbitmtp_b200.so: single translation unit holding every kernel and the C ABI
// declared in include/bitmtp_b200.h.  Host code here only validates arguments,
// picks a launch geometry and enqueues; it allocates nothing.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>
#include <mutex>

#include "../../include/bitmtp_b200.h"
#include "bm_common.cuh"

#include "t2_gemv.cuh"
#include "fused_ops.cuh"
#include "verify_attn.cuh"
#include "t2_gemv_rowwarp.cuh"
#include "t2_gemv_direct.cuh"
#include "dense_head.cuh"
#include "t2_gemm_wide.cuh"

#include <cudaTypedefs.h>
#include <map>
#include <tuple>

namespace {

constexpr int kMaxSmemPerCta = 227 * 1024;

struct DeviceInfo {
    int device = -1;
    int sm_count = 0;
};

DeviceInfo current_device() {
    static thread_local DeviceInfo cached;
    int dev = 0;
    cudaGetDevice(&dev);
    if (cached.device != dev) {
        cached.device = dev;
        cudaDeviceGetAttribute(&cached.sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (cached.sm_count <= 0) cached.sm_count = 148;
    }
    return cached;
}

inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? BM_OK : BM_ECUDA_BASE + (int)e; }

// Kernel launches issued by this library since it was loaded (launches recorded into a
// stream capture count once, at capture).  Diagnostic only: read through bm_launch_count.
std::atomic<unsigned long long> g_launches{0};
inline void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

// Generic launch with the optional programmatic-serialisation attribute.
template <typename Kernel, typename... Args>
int launch_ex(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int pdl,
              Args... args) {
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_status(e);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    count_launch();
    return cuda_status(cudaLaunchKernelEx(&cfg, kernel, args...));
}

template <typename Kernel>
int launch(Kernel kernel, int grid, int block, int smem, cudaStream_t stream, int pdl,
           const bm::GemvParams &p) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return cuda_status(e);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)block, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    count_launch();
    return cuda_status(cudaLaunchKernelEx(&cfg, kernel, p));
}

// Rows per tile: the largest of 32/16/8 that still leaves two tiles per SM, so
// that the tail of the last wave stays short.
int pick_rb(int N, int sms) {
    for (int rb = 4; rb > 1; rb >>= 1)
        if (N / (8 * rb) >= 2 * sms) return rb;
    return 1;
}

struct Plan {
    int rb, stages, grid, smem;
};

bool make_plan(int W, int N, int K, bool mma, int sms, Plan *out) {
    int rb = pick_rb(N, sms);
    for (; rb >= 1; rb >>= 1) {
        const int tiles = (N + 8 * rb - 1) / (8 * rb);
        // Two CTAs per SM when both fit; otherwise one.
        for (int per_sm = 2; per_sm >= 1; --per_sm) {
            const int grid = tiles < sms * per_sm ? tiles : sms * per_sm;
            const int tiles_per_cta = (tiles + grid - 1) / grid;
            const int budget = per_sm == 2 ? (kMaxSmemPerCta - 2048) / 2 : kMaxSmemPerCta;
            int stages = tiles_per_cta + 1 < bm::kMaxStages ? tiles_per_cta + 1 : bm::kMaxStages;
            if (stages < 2) stages = 2;
            for (; stages >= 2; --stages) {
                const bm::GemvSmem L = bm::gemv_smem_layout(W, K, rb, stages, mma);
                if (L.total <= budget) {
                    out->rb = rb;
                    out->stages = stages;
                    out->grid = grid;
                    out->smem = L.total;
                    return true;
                }
            }
        }
    }
    return false;
}

int gemv_launch_dp4a(const bm::GemvParams &p0, int sms, int pdl, cudaStream_t stream) {
    Plan pl;
    if (!make_plan(p0.W, p0.N, p0.K, false, sms, &pl)) return BM_EINVAL;
    bm::GemvParams p = p0;
    p.stages = pl.stages;
    p.pdl = pdl;
    const int wb = p.W == 1 ? 1 : (p.W == 2 ? 2 : 4);
#define BM_DP4A_CASE(WB_, RB_)                                                               \
    if (wb == WB_ && pl.rb == RB_)                                                           \
        return launch(bm::t2_gemv_dp4a_kernel<WB_, RB_>, pl.grid, bm::kGemvThreads, pl.smem, \
                      stream, pdl, p);
    BM_DP4A_CASE(1, 1) BM_DP4A_CASE(1, 2) BM_DP4A_CASE(1, 4)
    BM_DP4A_CASE(2, 1) BM_DP4A_CASE(2, 2) BM_DP4A_CASE(2, 4)
    BM_DP4A_CASE(4, 1) BM_DP4A_CASE(4, 2) BM_DP4A_CASE(4, 4)
#undef BM_DP4A_CASE
    return BM_EINVAL;
}

constexpr size_t kDirectMaxBytes = 8u << 20;   // packed weights up to which AUTO prefers the direct kernel

// Row-per-warp kernel without shared-memory staging, for W <= 4 (t2_gemv_direct.cuh).
int gemv_launch_direct(const bm::GemvParams &p0, int pdl, cudaStream_t stream) {
    if (!bm::direct_fits(p0.W, p0.N, p0.K) || p0.world > 1 || p0.silu_F != 0 || p0.src_mode != 0) return BM_EINVAL;
    const bm::DirectParams p{p0.A, p0.asum, p0.B, p0.ws, p0.s, p0.C, p0.G, p0.W, p0.N, p0.K, p0.ldc, p0.out_kind, pdl};
    const dim3 grid((unsigned)((p.N + bm::kDirectWarps - 1) / bm::kDirectWarps)), block(bm::kDirectWarps * 32);
    const int maxp = p.K <= 2048 ? 1 : (p.K <= 6144 ? 3 : 5);
    const int wt = p.W == 1 ? 1 : (p.W == 2 ? 2 : 4);
#define BM_DIRECT_CASE(WT_, MP_) \
    if (wt == WT_ && maxp == MP_) return launch_ex(bm::t2_gemv_direct_kernel<WT_, MP_>, grid, block, 0, stream, pdl, p);
    BM_DIRECT_CASE(1, 1) BM_DIRECT_CASE(1, 3) BM_DIRECT_CASE(1, 5)
    BM_DIRECT_CASE(2, 1) BM_DIRECT_CASE(2, 3) BM_DIRECT_CASE(2, 5)
    BM_DIRECT_CASE(4, 1) BM_DIRECT_CASE(4, 3) BM_DIRECT_CASE(4, 5)
#undef BM_DIRECT_CASE
    return BM_EINVAL;
}

struct MmaPlan {
    int rb, stages, grid, smem;
};

// Launch geometry of the MMA consumer.  Rows per tile grow with N so that large
// matrices amortise the per-tile barrier and merge; CTAs per SM are bounded by
// shared memory (activations + partials + at least two weight stages).
bool make_mma_plan(int N, int K, bool half, int sms, int force_rb, MmaPlan *out) {
    // Two CTAs of 8 warps per SM (128 registers per thread); each gets half the shared
    // memory.  Among the tile heights that divide N, take the one that keeps the most
    // weight bytes in flight per CTA, larger tiles winning ties (fewer hand-offs per byte);
    // small matrices keep 8-row tiles so that every SM gets work.
    const int per_sm = 2;
    const int budget = (kMaxSmemPerCta + 1024) / per_sm - 1024;
    int best_rb = 0, best_stages = 0, best_grid = 0, best_smem = 0;
    long best_flight = -1;
    for (int rb = 4; rb >= 1; rb >>= 1) {
        if (force_rb && rb != force_rb) continue;
        if ((N % (8 * rb)) != 0) continue;
        const int tiles = N / (8 * rb);
        // 16-row tiles already pay with one tile per SM (measured on 4096 x 2048 at widths 9 and 16: 4.0 -> 3.6 us
        // per launch inside a replay); 32-row tiles only when every CTA slot gets two of them
        if (!force_rb && rb > 1 && tiles < (rb == 2 ? sms : 2 * per_sm * sms)) continue;
        const int grid = tiles < sms * per_sm ? tiles : sms * per_sm;
        const int tiles_per_cta = (tiles + grid - 1) / grid;
        const int want = tiles_per_cta < bm::kMaxStages ? tiles_per_cta : bm::kMaxStages;
        for (int stages = want; stages >= 1; --stages) {
            const bm::MmaSmem L = bm::mma_smem_layout(K, rb, stages, half);
            if (L.total > budget) continue;
            const long flight = (long)stages * L.stage_bytes;
            if (flight > best_flight) {
                best_flight = flight;
                best_rb = rb; best_stages = stages; best_grid = grid; best_smem = L.total;
            }
            break;
        }
    }
    if (best_rb == 0) {
        // Nothing fits twice per SM (very long K): one CTA per SM with the whole budget.
        // 16-row tiles when they give every CTA one tile where 8-row tiles would give some CTAs two
        // (2048 rows: 128 tiles on 128 SMs instead of 256 on 148).
        for (int rb = 2; rb >= 1; --rb) {
            if (force_rb && rb != force_rb && force_rb <= 2) continue;
            if ((N % (8 * rb)) != 0) continue;
            const int tiles = N / (8 * rb);
            if (rb == 2 && !force_rb && !(tiles <= sms && 2 * tiles > sms)) continue;
            const int grid = tiles < sms ? tiles : sms;
            for (int stages = 2; stages >= 1; --stages) {
                const bm::MmaSmem L = bm::mma_smem_layout(K, rb, stages, half);
                if (L.total <= kMaxSmemPerCta) {
                    out->rb = rb; out->stages = stages; out->grid = grid; out->smem = L.total;
                    return true;
                }
            }
        }
        return false;
    }
    out->rb = best_rb; out->stages = best_stages; out->grid = best_grid; out->smem = best_smem;
    return true;
}

template <int RB, bool HALF, bool ONECHUNK, bool EMIT_G>
int launch_mma_inst(const MmaPlan &pl, cudaStream_t stream, int pdl, const bm::GemvParams &p) {
    return launch(bm::t2_gemv_mma_kernel<RB, HALF, ONECHUNK, EMIT_G>, pl.grid, bm::kGemvThreads, pl.smem, stream,
                  pdl, p);
}

template <bool HALF, bool ONECHUNK>
int launch_mma_rb(const MmaPlan &pl, cudaStream_t stream, int pdl, const bm::GemvParams &p) {
    if (p.G != nullptr) return launch_mma_inst<1, HALF, ONECHUNK, true>(pl, stream, pdl, p);
    if (pl.rb == 4) return launch_mma_inst<4, HALF, ONECHUNK, false>(pl, stream, pdl, p);
    if (pl.rb == 2) return launch_mma_inst<2, HALF, ONECHUNK, false>(pl, stream, pdl, p);
    return launch_mma_inst<1, HALF, ONECHUNK, false>(pl, stream, pdl, p);
}

int gemv_launch_mma(const bm::GemvParams &p0, int sms, int pdl, int force_rb, cudaStream_t stream) {
    // Tokens beyond 16 go through a second launch over the remaining rows.
    for (int m0 = 0; m0 < p0.W; m0 += 16) {
        bm::GemvParams p = p0;
        p.W = p0.W - m0 < 16 ? p0.W - m0 : 16;
        p.A = p0.A + (size_t)m0 * p0.K;
        if (p0.asum) p.asum = p0.asum + (size_t)m0 * (p0.K / BM_GROUP);
        p.s = p0.s + m0;
        const size_t esz = p0.out_kind == BM_OUT_BF16 ? 2 : 4;
        p.C = static_cast<char *>(p0.C) + (size_t)m0 * p0.ldc * esz;
        if (p0.G) p.G = p0.G + (size_t)m0 * p0.N * (p0.K / BM_GROUP);
        const bool half = p.W <= 8, one = p.K == 2048;
        MmaPlan pl;
        if (!make_mma_plan(p.N, p.K, half, sms, force_rb, &pl)) return BM_EINVAL;
        if (p.G != nullptr) {                         // the group-sum build exists for RB = 1 only
            pl.rb = 1;
            pl.grid = p.N / 8 < pl.grid ? p.N / 8 : pl.grid;
            pl.stages = 1;
            pl.smem = bm::mma_smem_layout(p.K, 1, 1, half).total;
        }
        p.stages = pl.stages;
        const int use_pdl = (m0 == 0) ? pdl : 0;
        p.pdl = use_pdl;
        int rc;
        if (half) rc = one ? launch_mma_rb<true, true>(pl, stream, use_pdl, p) : launch_mma_rb<true, false>(pl, stream, use_pdl, p);
        else rc = one ? launch_mma_rb<false, true>(pl, stream, use_pdl, p) : launch_mma_rb<false, false>(pl, stream, use_pdl, p);
        if (rc != BM_OK) return rc;
    }
    return BM_OK;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- row-per-warp GEMV: tensor maps ------------------------------------------------
// A tiled TMA copy needs a 128-byte descriptor of the weight matrix.  It is encoded by the
// driver on first use of a (device, pointer, N, K) and kept; the encode routine is looked up
// through the runtime, so the library does not link against libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

int weight_tensor_map(const void *B, int N, int K, CUtensorMap *out) {
    static std::mutex mu;
    static EncodeTiledFn encode = nullptr;
    static std::map<std::tuple<int, const void *, int, int>, CUtensorMap> cache;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_status(e);
    std::lock_guard<std::mutex> lock(mu);
    const auto key = std::make_tuple(dev, B, N, K);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return BM_OK; }
    if (encode == nullptr) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess) return cuda_status(e);
        if (fn == nullptr || qres != cudaDriverEntryPointSuccess) return BM_EINVAL;
        encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    CUtensorMap tm;
    const cuuint64_t dims[2] = {(cuuint64_t)(K / 4), (cuuint64_t)N};
    const cuuint64_t strides[1] = {(cuuint64_t)(K / 4)};
    const cuuint32_t box[2] = {(cuuint32_t)bm::kRwPanelBytes, (cuuint32_t)bm::kRwRows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(&tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(B), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return BM_ECUDA_BASE + 999;
    if (cache.size() > 4096) cache.clear();
    cache[key] = tm;
    *out = tm;
    return BM_OK;
}

// Warps per CTA, panels per stage and K split of the row-per-warp kernel.  The split (2 or 4 warps per
// 16-row block) is taken when the matrix has too few blocks to give every warp of every SM one.
struct RowWarpCfg { int warps, pb, ks; };

inline int rowwarp_ksplit(int N, int K, int sms) {
    const int blocks = N / bm::kRwRows;
    if ((K % 2048) != 0 || blocks >= 8 * sms) return 1;
    return 2 * blocks >= 8 * sms ? 2 : 4;
}

inline RowWarpCfg rowwarp_cfg(int W, int K, int ks = 1) {
    RowWarpCfg c;
    c.ks = ks;
    c.pb = ks == 4 ? 1 : 2;
    int warps = bm::kRwMaxWarps;
    // keep at least two stages per warp
    while (warps > 4 && bm::rowwarp_smem_layout(W, K, warps, c.pb).stages < 2) --warps;
    c.warps = warps;
    return c;
}

bool rowwarp_fits(int W, int N, int K) {
    if (W > 8 || (K % 512) != 0 || (N % bm::kRwRows) != 0) return false;
    const RowWarpCfg c = rowwarp_cfg(W, K);
    return bm::rowwarp_smem_layout(W, K, c.warps, c.pb).stages >= 2;
}

template <int NTOK, int PB, int KS>
int launch_rowwarp(const bm::RowWarpParams &P, int warps, int sms, int pdl, cudaStream_t stream) {
    const bm::RowWarpSmem L = bm::rowwarp_smem_layout(P.g.W, P.g.K, warps, PB);
    const int blocks = P.g.N / bm::kRwRows, teams = warps / KS;
    int grid = (blocks + teams - 1) / teams;
    if (grid > sms) grid = sms;
    const size_t smem = (size_t)L.total + 1024;
    if (P.g.G != nullptr)
        return launch_ex(bm::t2_gemv_rowwarp_kernel<NTOK, PB, true, KS>, dim3(grid), dim3(warps * 32), smem, stream, pdl, P);
    return launch_ex(bm::t2_gemv_rowwarp_kernel<NTOK, PB, false, KS>, dim3(grid), dim3(warps * 32), smem, stream, pdl, P);
}

int gemv_launch_rowwarp(const bm::GemvParams &p0, int sms, int pdl, cudaStream_t stream) {
    if (!rowwarp_fits(p0.W, p0.N, p0.K)) return BM_EINVAL;
    const int ks = rowwarp_ksplit(p0.N, p0.K, sms);
    bm::RowWarpParams P;
    const int rc = weight_tensor_map(p0.B, p0.N, p0.K, &P.tmap);
    if (rc != BM_OK) return rc;
    P.g = p0;
    P.g.pdl = pdl;
    const RowWarpCfg c = rowwarp_cfg(p0.W, p0.K, ks);
    if (c.warps % ks) return BM_EINVAL;
    if (p0.W == 1) {
        if (ks == 1) return launch_rowwarp<1, 2, 1>(P, c.warps, sms, pdl, stream);
        if (ks == 2) return launch_rowwarp<1, 2, 2>(P, c.warps, sms, pdl, stream);
        return launch_rowwarp<1, 1, 4>(P, c.warps, sms, pdl, stream);
    }
    if (ks == 1) return launch_rowwarp<2, 2, 1>(P, c.warps, sms, pdl, stream);
    if (ks == 2) return launch_rowwarp<2, 2, 2>(P, c.warps, sms, pdl, stream);
    return launch_rowwarp<2, 1, 4>(P, c.warps, sms, pdl, stream);
}

}  // namespace

extern "C" {

const char *bm_version(void) { return "bitmtp_b200 0.1 (sm_100a)"; }

int bm_sm_count(void) { return current_device().sm_count; }

unsigned long long bm_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int bm_device_error(void) {
    int v = 0;
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    if (cudaMemcpyFromSymbol(&v, bm::g_dev_err, sizeof(int)) != cudaSuccess) return -1;
    if (v != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(bm::g_dev_err, &zero, sizeof(int));
    }
    return v;
}

int64_t bm_t2_gemv_bytes(int W, int N, int K, int out_kind) {
    const int64_t esz = out_kind == BM_OUT_BF16 ? 2 : 4;
    return (int64_t)N * K / 4 + (int64_t)N * (K / 128) * 2 + (int64_t)W * K + 4 * (int64_t)W +
           esz * W * N;
}

struct PeerArgs {
    int world, rank;
    void *const *peer_C0;      // first output buffer of every rank
    void *const *peer_C1;      // second output buffer of every rank
    void *const *peer_flags;
    void *done;                // uint32 [4]
    unsigned int poll_limit;   // 0: default
};

static int gemv_common(const void *A, const void *a_sums, const void *B, void *C, const void *s, const void *ws,
                       int W, int N, int K, int ldc, int out_kind, int path, void *G_out, int pdl, void *stream,
                       const PeerArgs *peer = nullptr);

int bm_t2_gemv(const void *A, const void *B, void *C, const void *s, const void *ws, int W, int N,
               int K, int ldc, int out_kind, int path, void *G_out, int pdl, void *stream) {
    return gemv_common(A, nullptr, B, C, s, ws, W, N, K, ldc, out_kind, path, G_out, pdl, stream);
}

int bm_t2_gemv_prepared(const void *A_prep, const void *a_sums, const void *B, void *C, const void *s,
                        const void *ws, int W, int N, int K, int ldc, int out_kind, int pdl, void *stream) {
    if (!a_sums || (K % 256) != 0) return BM_EINVAL;
    return gemv_common(A_prep, a_sums, B, C, s, ws, W, N, K, ldc, out_kind, BM_PATH_AUTO, nullptr, pdl, stream);
}

static int gemv_common(const void *A, const void *a_sums, const void *B, void *C, const void *s, const void *ws,
                       int W, int N, int K, int ldc, int out_kind, int path, void *G_out, int pdl, void *stream,
                       const PeerArgs *peer) {
    if (!A || !B || !C || !s || !ws) return BM_EINVAL;
    if (W < 1 || W > BM_MAX_W || N < 8 || (N % 8) != 0 || K < 128 || (K % 128) != 0) return BM_EINVAL;
    if (ldc < N || (ldc % 4) != 0 || out_kind < 0 || out_kind > 2) return BM_EINVAL;
    if (!aligned16(A) || !aligned16(B) || !aligned16(ws) || !aligned16(C)) return BM_EINVAL;
    bm::GemvParams p;
    p.A = static_cast<const int8_t *>(A);
    p.asum = static_cast<const int32_t *>(a_sums);
    p.B = static_cast<const uint8_t *>(B);
    p.ws = static_cast<const uint16_t *>(ws);
    p.s = static_cast<const float *>(s);
    p.C = C;
    p.G = static_cast<int32_t *>(G_out);
    p.W = W;
    p.N = N;
    p.K = K;
    p.ldc = ldc;
    p.out_kind = out_kind;
    p.stages = 2;
    p.pdl = 0;
    p.silu_F = 0;
    p.amax_out = nullptr;
    p.src_mode = 0;
    p.xb = p.res = p.norm_w = nullptr;
    p.gather = nullptr;
    p.gather_rows = 0;
    p.h_out = nullptr;
    p.eps = 0.0f;
    p.amax_in = nullptr;
    p.amax_zero = nullptr;
    p.world = 0;
    p.rank = 0;
    p.done = nullptr;
    p.poll_limit = 0;
    for (int i = 0; i < 8; ++i) { p.peer_C[0][i] = p.peer_C[1][i] = nullptr; p.peer_flags[i] = nullptr; }
    if (peer != nullptr && peer->world > 1) {
        if (peer->world > 8 || peer->rank < 0 || peer->rank >= peer->world || out_kind != BM_OUT_BF16 || G_out != nullptr ||
            W > 16 || (K % 256) != 0 || !peer->peer_C0 || !peer->peer_C1 || !peer->peer_flags || !peer->done)
            return BM_EINVAL;
        p.world = peer->world;
        p.rank = peer->rank;
        p.done = static_cast<unsigned int *>(peer->done);
        p.poll_limit = peer->poll_limit ? peer->poll_limit : (1u << 22);
        for (int i = 0; i < peer->world; ++i) {
            if (!peer->peer_C0[i] || !peer->peer_C1[i] || !peer->peer_flags[i]) return BM_EINVAL;
            p.peer_C[0][i] = static_cast<uint16_t *>(peer->peer_C0[i]);
            p.peer_C[1][i] = static_cast<uint16_t *>(peer->peer_C1[i]);
            p.peer_flags[i] = static_cast<unsigned int *>(peer->peer_flags[i]);
        }
    }
    const int sms = current_device().sm_count;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The MMA consumer needs an even number of groups (K % 256 == 0); every model shape
    // has it.  Odd group counts go to the lanes-across-K consumer.
    if (path < BM_PATH_AUTO || path > BM_PATH_DIRECT) return BM_EINVAL;
    const int force_rb = 0;                           // tile height chosen by make_mma_plan
    if (path == BM_PATH_AUTO) {
        // Measured on B200 (one call after the other over weights that rotate through more than L2):
        //  * many rows and at most 8 tokens: every warp streams its own 16-row blocks (row-per-warp kernel);
        //  * one token over up to 4 MB of weights (two over up to 2 MB): the launch is latency-bound and the
        //    kernel with a single memory round trip wins (3.3-5.3 us against 5.2-8.4 us); for three or four
        //    tokens it still does up to 1 MB (2048 x 2048: 5.2 against 5.6 us, 1024 x 2048: 4.4 against 5.6 us);
        //  * otherwise, up to 8 tokens and K a multiple of 2048: the row-per-warp kernel with two or four warps
        //    sharing a block (2048 x 6144 at W = 8: 9.7 against 11.2 us; a 14336 x 8192 shard: 14.7 against 28.8 us);
        //  * everything else (more than 8 tokens, odd K): the cooperative tiles.
        const bool rw = rowwarp_fits(W, N, K);
        const size_t wbytes = (size_t)N * K / 4;
        const bool direct_ok = p.world <= 1 && bm::direct_fits(W, N, K) &&
                               wbytes <= (W == 1 ? (size_t)4 << 20 : (W == 2 ? (size_t)2 << 20 : (size_t)1 << 20));
        if (rw && N / bm::kRwRows >= 8 * sms) path = BM_PATH_ROWWARP;
        else if (direct_ok) path = BM_PATH_DIRECT;
        else if (rw && (K % 2048) == 0) path = BM_PATH_ROWWARP;
        else path = (K % 256) == 0 ? BM_PATH_MMA : BM_PATH_DP4A;
    }
    if (path == BM_PATH_DIRECT) return gemv_launch_direct(p, pdl, st);
    if (path == BM_PATH_ROWWARP) return gemv_launch_rowwarp(p, sms, pdl, st);
    if (path == BM_PATH_DP4A) return gemv_launch_dp4a(p, sms, pdl, st);
    if (path == BM_PATH_MMA) return (K % 256) == 0 ? gemv_launch_mma(p, sms, pdl, force_rb, st) : BM_EINVAL;
    return BM_EINVAL;
}

void t2g128_int8xint2_linear(int8_t *A, int8_t *B, void *C, float *s, void *ws, int M, int N,
                             int K, void *stream) {
    const int rc = bm_t2_gemv(A, B, C, s, ws, M, N, K, N, BM_OUT_BF16, BM_PATH_AUTO, nullptr, 0, stream);
    if (rc != BM_OK) fprintf(stderr, "[t2g128] unsupported shape M=%d N=%d K=%d (status %d)\n", M, N, K, rc);
}

// ---------------------------------------------------------------------------- fused operators
int bm_quant_rows(const void *x, int M, int K, void *q, void *q_prep, void *asum, void *s, int pdl, void *stream) {
    if (!x || !s || (!q && !q_prep) || M < 1 || K < 8 || (K % 8) != 0 || !aligned16(x)) return BM_EINVAL;
    if ((q_prep == nullptr) != (asum == nullptr) || (q_prep && (K % BM_GROUP) != 0)) return BM_EINVAL;
    if ((reinterpret_cast<uintptr_t>(q) & 7u) || (reinterpret_cast<uintptr_t>(q_prep) & 7u)) return BM_EINVAL;
    bm::QuantSink sink{static_cast<int8_t *>(q), static_cast<int8_t *>(q_prep), static_cast<int32_t *>(asum)};
    return launch_ex(bm::quant_rows_kernel, dim3(M), dim3(bm::kRowThreads), 0, static_cast<cudaStream_t>(stream), pdl,
                     static_cast<const uint16_t *>(x), K, sink, static_cast<float *>(s), pdl);
}

int bm_rmsnorm_fused(const void *x, const void *gather, int gather_rows, const void *res, const void *w, float eps,
                     int M, int dim, int row0, void *h_out, void *q, void *q_prep, void *asum, void *s, void *n_out,
                     int pdl, void *stream) {
    if (!x || !w || M < 1 || dim < 256 || (dim % 256) != 0 || dim > 8192) return BM_EINVAL;
    if (gather && gather_rows < 1) return BM_EINVAL;
    if (((q != nullptr) || (q_prep != nullptr)) != (s != nullptr)) return BM_EINVAL;
    if ((q_prep == nullptr) != (asum == nullptr)) return BM_EINVAL;
    if (!aligned16(x) || !aligned16(w) || (res && !aligned16(res))) return BM_EINVAL;
    bm::NormParams p;
    p.x = static_cast<const uint16_t *>(x);
    p.gather = static_cast<const int64_t *>(gather);
    p.gather_rows = gather_rows;
    p.res = static_cast<const uint16_t *>(res);
    p.w = static_cast<const uint16_t *>(w);
    p.h_out = static_cast<uint16_t *>(h_out);
    p.q = bm::QuantSink{static_cast<int8_t *>(q), static_cast<int8_t *>(q_prep), static_cast<int32_t *>(asum)};
    p.s = static_cast<float *>(s);
    p.n_out = static_cast<uint16_t *>(n_out);
    p.eps = eps;
    p.dim = dim;
    p.row0 = row0;
    p.pdl = pdl;
    return launch_ex(bm::rmsnorm_kernel, dim3(M), dim3(dim / 8), 0, static_cast<cudaStream_t>(stream), pdl, p);
}

int bm_t2_gemv_gate_up_silu(const void *A_prep, const void *a_sums, const void *B, const void *ws, const void *s, int W,
                            int F, int K, void *inner_out, void *amax_out, int pdl, void *stream) {
    if (!A_prep || !a_sums || !B || !ws || !s || !inner_out || !amax_out) return BM_EINVAL;
    if (W < 1 || W > 16 || F < 16 || (F % 16) != 0 || (K % 256) != 0 || K < 256) return BM_EINVAL;
    if (!aligned16(A_prep) || !aligned16(B) || !aligned16(ws) || !aligned16(inner_out)) return BM_EINVAL;
    bm::GemvParams p;
    p.A = static_cast<const int8_t *>(A_prep);
    p.asum = static_cast<const int32_t *>(a_sums);
    p.B = static_cast<const uint8_t *>(B);
    p.ws = static_cast<const uint16_t *>(ws);
    p.s = static_cast<const float *>(s);
    p.C = inner_out;
    p.G = nullptr;
    p.W = W;
    p.N = F;
    p.K = K;
    p.ldc = F;
    p.out_kind = BM_OUT_BF16;
    p.pdl = pdl;
    p.silu_F = F;
    p.amax_out = static_cast<unsigned int *>(amax_out);
    p.src_mode = 0;
    p.xb = p.res = p.norm_w = nullptr;
    p.gather = nullptr;
    p.gather_rows = 0;
    p.h_out = nullptr;
    p.eps = 0.0f;
    p.amax_in = nullptr;
    p.amax_zero = nullptr;
    p.world = 0;
    p.rank = 0;
    p.done = nullptr;
    p.poll_limit = 0;
    for (int i = 0; i < 8; ++i) { p.peer_C[0][i] = p.peer_C[1][i] = nullptr; p.peer_flags[i] = nullptr; }
    const int sms = current_device().sm_count;
    const bool half = W <= 8, one = K == 2048;
    MmaPlan pl;
    // the planner sees the 2F weight rows; a tile of 8*RB rows is 4*RB gate rows and their 4*RB up rows
    if (!make_mma_plan(2 * F, K, half, sms, 0, &pl)) return BM_EINVAL;
    if (pl.rb < 2 || (F % (4 * pl.rb)) != 0) {
        if (!make_mma_plan(2 * F, K, half, sms, 2, &pl) || (F % 8) != 0) return BM_EINVAL;
    }
    p.stages = pl.stages;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (half) return one ? launch_mma_rb<true, true>(pl, st, pdl, p) : launch_mma_rb<true, false>(pl, st, pdl, p);
    return one ? launch_mma_rb<false, true>(pl, st, pdl, p) : launch_mma_rb<false, false>(pl, st, pdl, p);
}

int bm_stage_replay_inputs(int kind, const void *src_a, const void *src_b, int n_pend, int cache_len, int M, int D,
                           long long mask_id, int role, int P, void *tok, void *pos, void *state, void *stream) {
    if (kind < 0 || kind > 3 || !src_a || !tok || !pos || !state || M < 1 || M > BM_MAX_W) return BM_EINVAL;
    if (kind == 0 && (n_pend < 1 || n_pend > P || P + D != M)) return BM_EINVAL;
    if (kind == 1 && (!src_b || n_pend < 1 || M != D + 1)) return BM_EINVAL;
    if (kind == 2 && M != 1) return BM_EINVAL;
    if (kind == 3 && (n_pend < 1 || n_pend > M)) return BM_EINVAL;
    int sp = n_pend < 0 ? 0 : n_pend;
    const int pmax = P > 0 ? P : 0;
    if (sp > pmax) sp = pmax;
    if (kind != 0) sp = 0;
    count_launch();
    bm::stage_replay_inputs_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        kind, static_cast<const int64_t *>(src_a), static_cast<const int64_t *>(src_b), n_pend, cache_len, M, D,
        (int64_t)mask_id, role, P, sp, static_cast<int64_t *>(tok), static_cast<int64_t *>(pos),
        static_cast<bm::StepState *>(state));
    return cuda_status(cudaGetLastError());
}

int bm_commit_stage_draft(const void *src, int n_commit, int verified, void *gen_dst, void *pending, int stage,
                          int cache_len, int M, int D, long long mask_id, int role, int P, void *tok, void *pos,
                          void *state, void *stream) {
    if (!src || !gen_dst || !pending || n_commit < 1 || n_commit > 32) return BM_EINVAL;
    if (stage) {
        const int n_pend = verified ? 1 : n_commit;
        if (!tok || !pos || !state || M < 1 || M > BM_MAX_W || P + D != M || n_pend > P) return BM_EINVAL;
    }
    count_launch();
    bm::commit_stage_draft_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const int64_t *>(src), n_commit, verified, static_cast<int64_t *>(gen_dst),
        static_cast<int64_t *>(pending), stage, cache_len, M, D, (int64_t)mask_id, role, P, static_cast<int64_t *>(tok),
        static_cast<int64_t *>(pos), static_cast<bm::StepState *>(state));
    return cuda_status(cudaGetLastError());
}

int bm_t2_gemv_row_fused(int src_mode, const void *x, const void *gather, int gather_rows, const void *res,
                         const void *norm_w, float eps,
                         void *h_out, const void *amax_in, void *amax_zero, const void *B, const void *ws, int N, int K,
                         void *C, int ldc, int out_kind, int silu, void *amax_out, int pdl, void *stream) {
    if ((src_mode != 1 && src_mode != 2) || !x || !B || !ws || !C || N < 8 || (N % 8) != 0 || (K % 256) != 0 || K < 256)
        return BM_EINVAL;
    const bool staged = (pdl & BM_PDL_STAGED) != 0;     // testing aid: keep to the shared-memory-staged kernel
    pdl &= BM_PDL_OVERLAP;
    if (src_mode == 1 && !amax_in) return BM_EINVAL;
    if (gather && gather_rows < 1) return BM_EINVAL;
    if (src_mode == 2 && (!norm_w || K != 8 * bm::kGemvThreads)) return BM_EINVAL;
    if (silu && (!amax_out || out_kind != BM_OUT_BF16 || (N % 16) != 0)) return BM_EINVAL;
    if (ldc < N || (ldc % 4) != 0 || out_kind < 0 || out_kind > 2) return BM_EINVAL;
    if (!aligned16(x) || !aligned16(B) || !aligned16(ws) || !aligned16(C) || (res && !aligned16(res)) ||
        (norm_w && !aligned16(norm_w)) || (h_out && !aligned16(h_out)))
        return BM_EINVAL;
    bm::GemvParams p;
    p.A = nullptr;
    p.asum = nullptr;
    p.B = static_cast<const uint8_t *>(B);
    p.ws = static_cast<const uint16_t *>(ws);
    p.s = nullptr;
    p.C = C;
    p.G = nullptr;
    p.W = 1;
    p.N = N;
    p.K = K;
    p.ldc = ldc;
    p.out_kind = out_kind;
    p.pdl = pdl;
    p.silu_F = silu ? N : 0;
    p.amax_out = static_cast<unsigned int *>(amax_out);
    p.src_mode = src_mode;
    p.xb = static_cast<const uint16_t *>(x);
    p.res = static_cast<const uint16_t *>(res);
    p.norm_w = static_cast<const uint16_t *>(norm_w);
    p.gather = static_cast<const int64_t *>(gather);
    p.gather_rows = gather_rows;
    p.h_out = static_cast<uint16_t *>(h_out);
    p.eps = eps;
    p.amax_in = static_cast<const unsigned int *>(amax_in);
    p.amax_zero = static_cast<unsigned int *>(amax_zero);
    p.world = 0;
    p.rank = 0;
    p.done = nullptr;
    p.poll_limit = 0;
    for (int i = 0; i < 8; ++i) { p.peer_C[0][i] = p.peer_C[1][i] = nullptr; p.peer_flags[i] = nullptr; }
    const int sms = current_device().sm_count;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // A few MB of weights: the register-only kernel (one memory round trip after the row is staged).
    if (!staged && bm::direct_row_fits(N, K) && (size_t)(silu ? 2 : 1) * N * K / 4 <= kDirectMaxBytes) {
        const dim3 grid((unsigned)(N / bm::kDirectWarps)), block(bm::kGemvThreads);
        const int maxp = K <= 2048 ? 1 : (K <= 6144 ? 3 : 5);
#define BM_ROW_CASE(S_, MP_) \
        if (silu == S_ && maxp == MP_) return launch_ex(bm::t2_gemv_direct_row_kernel<S_, MP_>, grid, block, 0, st, pdl, p);
        BM_ROW_CASE(false, 1) BM_ROW_CASE(false, 3) BM_ROW_CASE(false, 5)
        BM_ROW_CASE(true, 1) BM_ROW_CASE(true, 3) BM_ROW_CASE(true, 5)
#undef BM_ROW_CASE
    }
    const bool one = K == 2048;
    MmaPlan pl;
    if (!make_mma_plan(silu ? 2 * N : N, K, true, sms, 0, &pl)) return BM_EINVAL;
    if (silu && (N % (4 * pl.rb)) != 0 && !make_mma_plan(2 * N, K, true, sms, 1, &pl)) return BM_EINVAL;
    p.stages = pl.stages;
    return one ? launch_mma_rb<true, true>(pl, st, pdl, p) : launch_mma_rb<true, false>(pl, st, pdl, p);
}

int bm_zero_words(void *p, int n, void *stream) {
    if (!p || n < 1) return BM_EINVAL;
    return cuda_status(cudaMemsetAsync(p, 0, (size_t)n * 4, static_cast<cudaStream_t>(stream)));
}

int bm_quant_rows_amax(const void *x, const void *amax_in, void *amax_zero, int M, int K, void *q, void *q_prep,
                       void *asum, void *s, int pdl, void *stream) {
    if (!x || !amax_in || !s || (!q && !q_prep) || M < 1 || M > 65535 || K < 256 || (K % 256) != 0 || !aligned16(x))
        return BM_EINVAL;
    if ((q_prep == nullptr) != (asum == nullptr) || amax_zero == amax_in) return BM_EINVAL;
    bm::QuantSink sink{static_cast<int8_t *>(q), static_cast<int8_t *>(q_prep), static_cast<int32_t *>(asum)};
    const int units = M * (K / 8);
    const int grid = (units + bm::kQuantAmaxThreads - 1) / bm::kQuantAmaxThreads;
    return launch_ex(bm::quant_rows_amax_kernel, dim3(grid), dim3(bm::kQuantAmaxThreads), 0,
                     static_cast<cudaStream_t>(stream), pdl, static_cast<const uint16_t *>(x),
                     static_cast<const unsigned int *>(amax_in), static_cast<unsigned int *>(amax_zero), M, K, sink,
                     static_cast<float *>(s), pdl);
}

int bm_silu_mul_quant(const void *gu, int M, int F, void *q, void *q_prep, void *asum, void *s, void *inner_out,
                      int pdl, void *stream) {
    if (!gu || !s || (!q && !q_prep) || M < 1 || F < 8 || (F % 8) != 0 || !aligned16(gu)) return BM_EINVAL;
    if ((q_prep == nullptr) != (asum == nullptr) || (q_prep && (F % BM_GROUP) != 0)) return BM_EINVAL;
    const size_t smem = (size_t)F * 2;
    if (smem > 200 * 1024) return BM_EINVAL;
    bm::QuantSink sink{static_cast<int8_t *>(q), static_cast<int8_t *>(q_prep), static_cast<int32_t *>(asum)};
    return launch_ex(bm::silu_mul_quant_kernel, dim3(M), dim3(bm::kRowThreads), smem, static_cast<cudaStream_t>(stream),
                     pdl, static_cast<const uint16_t *>(gu), F, sink, static_cast<float *>(s),
                     static_cast<uint16_t *>(inner_out), pdl);
}

int bm_qknorm_rope_kvappend(const void *xqkv, const void *q_w, const void *k_w, float eps, const void *cos_t,
                            const void *sin_t, const void *positions, int M, int H, int Hkv, void *k_base,
                            void *v_base, int kv_rows, int sigma, void *q_out, int pdl, void *stream) {
    if (!xqkv || !q_w || !k_w || !cos_t || !sin_t || !positions || !k_base || !v_base || !q_out) return BM_EINVAL;
    if (M < 1 || M > 65535 || H < 1 || Hkv < 1 || (H % Hkv) != 0 || sigma < 0 || sigma + M > kv_rows) return BM_EINVAL;
    bm::RopeParams p;
    p.xqkv = static_cast<const uint16_t *>(xqkv);
    p.q_w = static_cast<const uint16_t *>(q_w);
    p.k_w = static_cast<const uint16_t *>(k_w);
    p.cos_t = static_cast<const uint16_t *>(cos_t);
    p.sin_t = static_cast<const uint16_t *>(sin_t);
    p.positions = static_cast<const int64_t *>(positions);
    p.k_base = static_cast<uint16_t *>(k_base);
    p.v_base = static_cast<uint16_t *>(v_base);
    p.q_out = static_cast<uint16_t *>(q_out);
    p.eps = eps;
    p.M = M; p.H = H; p.Hkv = Hkv; p.kv_rows = kv_rows; p.sigma = sigma; p.pdl = pdl;
    const int heads = H + 2 * Hkv;
    return launch_ex(bm::qknorm_rope_kvappend_kernel, dim3((heads + 3) / 4, M), dim3(128), 0,
                     static_cast<cudaStream_t>(stream), pdl, p);
}

int bm_set_step_state(void *state, int cache_len, int n_pend, int role, int P, void *stream) {
    if (!state || cache_len < 0 || role < 0 || role > 2) return BM_EINVAL;
    count_launch();
    bm::set_step_state_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<bm::StepState *>(state), cache_len, n_pend, role, P);
    return cuda_status(cudaGetLastError());
}

int bm_kv_copy_rows(void *kv, int planes, int kv_rows, int src_row, int dst_row, int n, void *stream) {
    if (!kv || planes < 1 || n < 0 || src_row < 0 || dst_row < 0 || src_row + n > kv_rows || dst_row + n > kv_rows)
        return BM_EINVAL;
    if (n == 0) return BM_OK;
    if (!(src_row >= dst_row + n || dst_row >= src_row + n)) return BM_EINVAL;   // ranges must not overlap
    count_launch();
    bm::kv_copy_rows_kernel<<<planes, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<uint16_t *>(kv), planes, kv_rows, src_row, dst_row, n);
    return cuda_status(cudaGetLastError());
}

int64_t bm_verify_attention_scratch_bytes(int M, int H, int sigma) {
    return (int64_t)bm::attn_scratch_bytes(M, H, sigma);
}

}  // extern "C"

namespace {
// Inputs of the attention kernel with the q/k norm, RoPE and KV append folded in (null: rotated queries in `q`).
struct RopeInputs {
    const void *xqkv, *q_w, *k_w, *cos_t, *sin_t, *positions;
    float eps;
};

// Launch of the cluster build of the attention kernel: the grid's x extent is one thread-block cluster.
// Returns -1 (and launches nothing) unless the device holds all of the grid's clusters at once - a
// cluster that has to wait for a place costs more than the shorter merge saves - so that the caller takes
// the ticket build; the device is asked once per kernel, cluster size and device.
template <void (*kernel)(const bm::AttnParams)>
int launch_attention_cluster(dim3 grid, size_t smem, cudaStream_t st, int pdl, const bm::AttnParams &p) {
    static std::atomic<int> resident[bm::kAttnMaxCluster + 1][8];    // clusters the device holds, +1 (0: not asked yet)
    const int dev = current_device().device;
    if (grid.x > (unsigned)bm::kAttnMaxCluster || dev < 0 || dev >= 8) return -1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(bm::kAttnThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = grid.x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    std::atomic<int> &known = resident[grid.x][dev];
    int held = known.load(std::memory_order_relaxed) - 1;
    if (held < 0) {
        int clusters = 0;
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess && grid.x > 8)
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        cfg.numAttrs = 1;
        if (e == cudaSuccess) e = cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg);
        if (e != cudaSuccess) cudaGetLastError();                     // an unsupported size is an answer, not a failure
        held = e == cudaSuccess && clusters > 0 ? clusters : 0;
        known.store(held + 1, std::memory_order_relaxed);
    }
    if ((int)(grid.y * grid.z) > held) return -1;
    cfg.numAttrs = pdl ? 2 : 1;
    count_launch();
    return cuda_status(cudaLaunchKernelEx(&cfg, kernel, p));
}

template <bool ROPE>
int launch_attention(int nq, dim3 grid, size_t smem, cudaStream_t st, int pdl, const bm::AttnParams &p) {
    const dim3 block(bm::kAttnThreads);
    // Cluster build where a (kv head, query group)'s super-chunks fit one cluster.  Same arithmetic, same order.
    if (p.slab_rows == 0 && p.slots > 0 && grid.x <= (unsigned)bm::kAttnMaxCluster) {
        int rc;
        switch (nq) {
            case 1: rc = launch_attention_cluster<bm::attn_fused_kernel<1, ROPE, true>>(grid, smem, st, pdl, p); break;
            case 2: rc = launch_attention_cluster<bm::attn_fused_kernel<2, ROPE, true>>(grid, smem, st, pdl, p); break;
            case 3: rc = launch_attention_cluster<bm::attn_fused_kernel<3, ROPE, true>>(grid, smem, st, pdl, p); break;
            default: rc = launch_attention_cluster<bm::attn_fused_kernel<4, ROPE, true>>(grid, smem, st, pdl, p); break;
        }
        if (rc >= 0) return rc;
    }
    switch (nq) {
        case 1: return launch_ex(bm::attn_fused_kernel<1, ROPE>, grid, block, smem, st, pdl, p);
        case 2: return launch_ex(bm::attn_fused_kernel<2, ROPE>, grid, block, smem, st, pdl, p);
        case 3: return launch_ex(bm::attn_fused_kernel<3, ROPE>, grid, block, smem, st, pdl, p);
        default: return launch_ex(bm::attn_fused_kernel<4, ROPE>, grid, block, smem, st, pdl, p);
    }
}

// One attention launch (scores, softmax, numerators, merge: bf16 rows + row absmax bits), followed by the
// flat quantisation launch unless the caller asked for rows only (`amax_rows` != null).
int verify_attention_impl(const void *q, const RopeInputs *rope, const void *k_base, const void *v_base, int M, int H,
                          int Hkv, int kv_rows, int sigma, const void *state, void *scratch, void *att_out,
                          void *q_out, void *q_prep, void *asum, void *s_out, int pdl, void *stream,
                          void *amax_rows = nullptr) {
    if (amax_rows != nullptr) {
        if (!att_out) return BM_EINVAL;
    } else {
        if ((!q_out && !q_prep) || !s_out || (q_prep == nullptr) != (asum == nullptr)) return BM_EINVAL;
    }
    if (rope != nullptr) {
        if (!rope->xqkv || !rope->q_w || !rope->k_w || !rope->cos_t || !rope->sin_t || !rope->positions) return BM_EINVAL;
        if ((reinterpret_cast<uintptr_t>(rope->xqkv) & 7u) || (reinterpret_cast<uintptr_t>(rope->cos_t) & 7u) ||
            (reinterpret_cast<uintptr_t>(rope->sin_t) & 7u) || (reinterpret_cast<uintptr_t>(rope->q_w) & 7u) ||
            (reinterpret_cast<uintptr_t>(rope->k_w) & 7u))
            return BM_EINVAL;
        q = rope->xqkv;                               // only for the null / alignment checks below
    }
    if (!q || !k_base || !v_base || !state || !scratch) return BM_EINVAL;
    if (M < 1 || M > BM_MAX_W || H < 1 || Hkv < 1 || (H % Hkv) != 0) return BM_EINVAL;
    if (sigma < 0 || sigma + M > kv_rows || !aligned16(q) || !aligned16(k_base) || !aligned16(v_base) ||
        !aligned16(scratch) || (att_out && !aligned16(att_out)))
        return BM_EINVAL;
    const int NJ = (sigma + BM_ATTN_SUPER - 1) / BM_ATTN_SUPER + 1;
    if (NJ > bm::kAttnMaxNJ) return BM_EINVAL;
    const int G = H / Hkv, QV = G * M;
    int nq = 1, Z = 1;
    bm::attn_query_split(QV, &nq, &Z);
    // more z-slices than the coarse split needs: every CTA picks the split for the history length it reads
    Z = bm::attn_zmax(QV, nq);
    if (Hkv * Z > bm::kAttnTickets) return BM_EINVAL;
    if ((H * 128) % 256 != 0 && amax_rows == nullptr) return BM_EINVAL;   // the flat quantisation wants K % 256 == 0
    bm::AttnParams p = {};
    p.slots = 2 * current_device().sm_count;                     // two CTAs of this kernel per SM (shared memory)
    p.q = static_cast<const uint16_t *>(q);
    p.k_base = static_cast<const uint16_t *>(k_base);
    p.v_base = static_cast<const uint16_t *>(v_base);
    p.state = static_cast<const bm::StepState *>(state);
    p.M = M; p.H = H; p.Hkv = Hkv; p.kv_rows = kv_rows; p.sigma = sigma; p.NJ = NJ;
    char *sc = static_cast<char *>(scratch);
    p.tickets = reinterpret_cast<unsigned int *>(sc);
    unsigned int *own_amax = reinterpret_cast<unsigned int *>(sc) + bm::kAttnTickets;
    p.pm = reinterpret_cast<float *>(sc + bm::kAttnHeaderBytes);
    p.pl = p.pm + (size_t)M * H * NJ;
    p.po = p.pl + (size_t)M * H * NJ;
    uint16_t *own_rows = reinterpret_cast<uint16_t *>(p.po + (size_t)M * H * NJ * 128);
    p.att = att_out ? static_cast<uint16_t *>(att_out) : own_rows;
    p.amax = amax_rows ? static_cast<unsigned int *>(amax_rows) : own_amax;
    p.pdl = pdl & (BM_PDL_OVERLAP | BM_PDL_STABLE_STATE);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (amax_rows == nullptr) {
        // this call gathers the row absmax in the scratch header: clear it first (stream-ordered)
        const cudaError_t e = cudaMemsetAsync(own_amax, 0, BM_MAX_W * sizeof(unsigned int), st);
        if (e != cudaSuccess) return cuda_status(e);
    }
    const size_t smem = bm::attn_smem_bytes(nq);
    const dim3 grid(NJ, Hkv, Z);
    // after a memset node the launch cannot overlap its predecessor programmatically
    const int attn_pdl = amax_rows ? (pdl & BM_PDL_OVERLAP) : 0;
    if (amax_rows == nullptr) p.pdl = 0;
    int rc;
    if (rope != nullptr) {
        p.xqkv = static_cast<const uint16_t *>(rope->xqkv);
        p.q_w = static_cast<const uint16_t *>(rope->q_w);
        p.k_w = static_cast<const uint16_t *>(rope->k_w);
        p.cos_t = static_cast<const uint16_t *>(rope->cos_t);
        p.sin_t = static_cast<const uint16_t *>(rope->sin_t);
        p.positions = static_cast<const int64_t *>(rope->positions);
        p.k_out = const_cast<uint16_t *>(p.k_base);
        p.v_out = const_cast<uint16_t *>(p.v_base);
        p.eps = rope->eps;
        rc = launch_attention<true>(nq, grid, smem, st, attn_pdl, p);
    } else {
        rc = launch_attention<false>(nq, grid, smem, st, attn_pdl, p);
    }
    if (rc != BM_OK || amax_rows != nullptr) return rc;
    // INT8 codes of the rows from the flat grid, with the absmax the merge gathered
    bm::QuantSink sink{static_cast<int8_t *>(q_out), static_cast<int8_t *>(q_prep), static_cast<int32_t *>(asum)};
    const int K = H * 128, units = M * (K / 8);
    const int qgrid = (units + bm::kQuantAmaxThreads - 1) / bm::kQuantAmaxThreads;
    return launch_ex(bm::quant_rows_amax_kernel, dim3(qgrid), dim3(bm::kQuantAmaxThreads), 0, st, pdl & BM_PDL_OVERLAP,
                     static_cast<const uint16_t *>(p.att), static_cast<const unsigned int *>(own_amax),
                     static_cast<unsigned int *>(nullptr), M, K, sink, static_cast<float *>(s_out), pdl & BM_PDL_OVERLAP);
}
}  // namespace

extern "C" {

int bm_verify_attention(const void *q, const void *k_base, const void *v_base, int M, int H, int Hkv, int kv_rows,
                        int sigma, const void *state, void *scratch, void *att_out, void *q_out, void *q_prep,
                        void *asum, void *s_out, int pdl, void *stream) {
    return verify_attention_impl(q, nullptr, k_base, v_base, M, H, Hkv, kv_rows, sigma, state, scratch, att_out, q_out,
                                 q_prep, asum, s_out, pdl, stream);
}

int bm_rope_verify_attention_rows(const void *xqkv, const void *q_w, const void *k_w, float eps, const void *cos_t,
                                  const void *sin_t, const void *positions, void *k_base, void *v_base, int M, int H,
                                  int Hkv, int kv_rows, int sigma, const void *state, void *scratch, void *att_out,
                                  void *amax_out, int pdl, void *stream) {
    if (!amax_out) return BM_EINVAL;
    const RopeInputs rope{xqkv, q_w, k_w, cos_t, sin_t, positions, eps};
    return verify_attention_impl(nullptr, &rope, k_base, v_base, M, H, Hkv, kv_rows, sigma, state, scratch, att_out,
                                 nullptr, nullptr, nullptr, nullptr, pdl, stream, amax_out);
}

int bm_rope_verify_attention(const void *xqkv, const void *q_w, const void *k_w, float eps, const void *cos_t,
                             const void *sin_t, const void *positions, void *k_base, void *v_base, int M, int H,
                             int Hkv, int kv_rows, int sigma, const void *state, void *scratch, void *att_out,
                             void *q_out, void *q_prep, void *asum, void *s_out, int pdl, void *stream) {
    const RopeInputs rope{xqkv, q_w, k_w, cos_t, sin_t, positions, eps};
    return verify_attention_impl(nullptr, &rope, k_base, v_base, M, H, Hkv, kv_rows, sigma, state, scratch, att_out,
                                 q_out, q_prep, asum, s_out, pdl, stream);
}

// ---------------------------------------------------------------------------- logits
int bm_argmax_rows(const void *logits, int rows, int vocab, int ld, void *idx, void *max_out, void *stream) {
    if (!logits || !idx || rows < 1 || vocab < 1 || ld < vocab) return BM_EINVAL;
    count_launch();
    bm::argmax_rows_kernel<<<rows, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float *>(logits), vocab, ld, static_cast<int64_t *>(idx), static_cast<float *>(max_out));
    return cuda_status(cudaGetLastError());
}

int bm_draft_chain(const void *logits, int D, int vocab, int ld, float tau, void *idx, void *max_buf, void *conf,
                   void *n_out, void *stream) {
    if (!logits || !idx || !max_buf || !conf || !n_out || D < 1 || D > BM_MAX_W || vocab < 1 || ld < vocab ||
        vocab > bm::kConfMaxChunks * 256)
        return BM_EINVAL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    count_launch();
    bm::argmax_rows_kernel<<<D, 1024, 0, st>>>(static_cast<const float *>(logits), vocab, ld,
                                               static_cast<int64_t *>(idx), static_cast<float *>(max_buf));
    count_launch();
    bm::row_confidence_kernel<<<D, 256, 0, st>>>(static_cast<const float *>(logits), vocab, ld,
                                                 static_cast<const float *>(max_buf), static_cast<float *>(conf));
    count_launch();
    bm::chain_length_kernel<<<1, 32, 0, st>>>(static_cast<const float *>(conf), D, tau, static_cast<int *>(n_out));
    return cuda_status(cudaGetLastError());
}

long long bm_logit_scratch_bytes(void) { return (long long)sizeof(bm::LogitScratch); }

int bm_argmax_rows_split(const void *logits, int rows, int vocab, int ld, void *idx, void *max_out, void *scratch,
                         void *stream) {
    if (!logits || !idx || !scratch || rows < 1 || rows > bm::kLogitMaxRows || vocab < 1 || ld < vocab ||
        !aligned16(scratch))
        return BM_EINVAL;
    count_launch();
    bm::argmax_split_kernel<<<dim3(bm::logit_splits(rows), rows), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float *>(logits), vocab, ld, static_cast<int64_t *>(idx), static_cast<float *>(max_out),
        static_cast<bm::LogitScratch *>(scratch));
    return cuda_status(cudaGetLastError());
}

int bm_draft_chain_split(const void *logits, int D, int vocab, int ld, float tau, void *idx, void *max_buf, void *conf,
                         void *n_out, void *scratch, void *stream) {
    if (!logits || !idx || !max_buf || !conf || !n_out || !scratch || D < 1 || D > bm::kLogitMaxRows || vocab < 1 ||
        ld < vocab || vocab > bm::kConfMaxChunks * 256 || !aligned16(scratch))
        return BM_EINVAL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    bm::LogitScratch *sc = static_cast<bm::LogitScratch *>(scratch);
    {
        // One launch with a cluster per row when the device holds all D clusters at once; else the two launches below.
        static std::atomic<int> held[8];                              // clusters the device holds, +1 (0: not asked yet)
        const int dev = current_device().device;
        const int nchunks = (vocab + 255) / 256, per = (nchunks + bm::kDraftClusterCtas - 1) / bm::kDraftClusterCtas;
        const size_t smem = (size_t)per * 256 * sizeof(float);
        if (dev >= 0 && dev < 8 && smem <= 96 * 1024) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(bm::kDraftClusterCtas, D);
            cfg.blockDim = dim3(256);
            cfg.dynamicSmemBytes = smem;
            cfg.stream = st;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = bm::kDraftClusterCtas;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            cudaError_t e = cudaFuncSetAttribute(bm::draft_chain_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)(96 * 1024));
            int n = held[dev].load(std::memory_order_relaxed) - 1;
            if (e == cudaSuccess && n < 0) {
                int clusters = 0;
                e = cudaFuncSetAttribute(bm::draft_chain_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
                cudaLaunchConfig_t probe = cfg;
                probe.gridDim = dim3(bm::kDraftClusterCtas, bm::kLogitMaxRows);
                probe.dynamicSmemBytes = 96 * 1024;
                if (e == cudaSuccess) e = cudaOccupancyMaxActiveClusters(&clusters, bm::draft_chain_cluster_kernel, &probe);
                if (e != cudaSuccess) cudaGetLastError();             // an unsupported size is an answer, not a failure
                n = e == cudaSuccess && clusters > 0 ? clusters : 0;
                held[dev].store(n + 1, std::memory_order_relaxed);
                e = cudaSuccess;
            }
            if (e == cudaSuccess && D <= n) {
                count_launch();
                return cuda_status(cudaLaunchKernelEx(&cfg, bm::draft_chain_cluster_kernel, static_cast<const float *>(logits),
                                                      vocab, ld, static_cast<int64_t *>(idx), static_cast<float *>(max_buf),
                                                      static_cast<float *>(conf), D, tau, static_cast<int *>(n_out), sc));
            }
        }
    }
    count_launch();
    bm::argmax_split_kernel<<<dim3(bm::logit_splits(D), D), 256, 0, st>>>(
        static_cast<const float *>(logits), vocab, ld, static_cast<int64_t *>(idx), static_cast<float *>(max_buf), sc);
    count_launch();
    bm::confidence_split_kernel<<<dim3(bm::logit_splits(D), D), 256, 0, st>>>(
        static_cast<const float *>(logits), vocab, ld, static_cast<const float *>(max_buf), static_cast<float *>(conf), D,
        tau, static_cast<int *>(n_out), sc);
    return cuda_status(cudaGetLastError());
}

int bm_verify_accept(const void *draft, const void *verify, int D, void *n_out, void *stream) {
    if (!draft || !verify || !n_out || D < 1) return BM_EINVAL;
    count_launch();
    bm::verify_accept_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const int64_t *>(draft), static_cast<const int64_t *>(verify), D, static_cast<int *>(n_out));
    return cuda_status(cudaGetLastError());
}

// ---------------------------------------------------------------------------- converter
int bm_pack_t2_g128(const void *w, int N, int K, void *packed, void *scale, void *frozen, void *stream) {
    if (!w || !packed || !scale || N < 1 || K < BM_GROUP || (K % BM_GROUP) != 0) return BM_EINVAL;
    if (!aligned16(w) || (frozen && !aligned16(frozen)) || (reinterpret_cast<uintptr_t>(packed) & 1u)) return BM_EINVAL;
    const long long units = (long long)N * (K / BM_GROUP);
    const long long blocks = (units + 15) / 16;                     // two (row, group) units per warp
    if (blocks > 0x7fffffffLL) return BM_EINVAL;
    count_launch();
    bm::pack_t2_g128_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t *>(w), N, K, static_cast<uint8_t *>(packed), static_cast<uint16_t *>(scale),
        static_cast<uint16_t *>(frozen));
    return cuda_status(cudaGetLastError());
}

// ---------------------------------------------------------------------------- prompt (many-row) path
int bm_t2_gemm_wide(const void *A_prep, const void *a_sums, const void *B, void *C, const void *s, const void *ws, int T,
                    int N, int K, int ldc, int pdl, void *stream) {
    if (!A_prep || !a_sums || !B || !C || !s || !ws || T < 1 || N < bm::kWideRows || (N % bm::kWideRows) != 0 ||
        K < BM_GROUP || (K % BM_GROUP) != 0 || ldc < N)
        return BM_EINVAL;
    if (!aligned16(A_prep) || !aligned16(B)) return BM_EINVAL;
    const size_t smem = bm::wide_smem_bytes(K / BM_GROUP, K == BM_SLOTS * BM_GROUP);
    if (smem > (size_t)kMaxSmemPerCta) return BM_EINVAL;
    bm::WideParams p;
    p.A = static_cast<const int8_t *>(A_prep);
    p.asum = static_cast<const int32_t *>(a_sums);
    p.s = static_cast<const float *>(s);
    p.B = static_cast<const uint8_t *>(B);
    p.ws = static_cast<const uint16_t *>(ws);
    p.C = static_cast<uint16_t *>(C);
    p.T = T; p.N = N; p.K = K; p.ldc = ldc; p.pdl = pdl & BM_PDL_OVERLAP;
    const dim3 grid(N / bm::kWideRows, (T + bm::kWideTokens - 1) / bm::kWideTokens);
    if (grid.y > 65535) return BM_EINVAL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (K == BM_SLOTS * BM_GROUP) return launch_ex(bm::t2_gemm_wide_kernel<true>, grid, dim3(bm::kWideThreads), smem, st, p.pdl, p);
    return launch_ex(bm::t2_gemm_wide_kernel<false>, grid, dim3(bm::kWideThreads), smem, st, p.pdl, p);
}

namespace {
// Slabs, grid.x and scratch layout of the prompt-mode attention.
struct PromptAttnPlan { int n_slabs, units, NJ, nq, Z; size_t ticket_bytes, total; };
bool prompt_attn_plan(int T, int hist0, int slab_rows, int H, int Hkv, PromptAttnPlan *pl) {
    if (T < 1 || hist0 < 0 || slab_rows < 1 || slab_rows > BM_MAX_W || H < 1 || Hkv < 1 || (H % Hkv) != 0) return false;
    pl->n_slabs = (T + slab_rows - 1) / slab_rows;
    pl->units = 0;
    for (int s = 0; s < pl->n_slabs; ++s) pl->units += (hist0 + s * slab_rows + BM_ATTN_SUPER - 1) / BM_ATTN_SUPER + 1;
    pl->NJ = (hist0 + T + BM_ATTN_SUPER - 1) / BM_ATTN_SUPER + 1;
    bm::attn_query_split((H / Hkv) * slab_rows, &pl->nq, &pl->Z);
    pl->ticket_bytes = ((size_t)pl->n_slabs * Hkv * pl->Z * 4 + 1023) / 1024 * 1024;
    pl->total = pl->ticket_bytes + (size_t)T * H * pl->NJ * 4 * 2 + (size_t)T * H * pl->NJ * 128 * 4;
    return pl->NJ <= bm::kAttnMaxNJ;
}
}  // namespace

long long bm_prompt_attention_scratch_bytes(int T, int hist0, int slab_rows, int H, int Hkv) {
    PromptAttnPlan pl;
    return prompt_attn_plan(T, hist0, slab_rows, H, Hkv, &pl) ? (long long)pl.total : -1;
}

int bm_prompt_attention(const void *q, const void *k_base, const void *v_base, int T, int hist0, int slab_rows, int H,
                        int Hkv, int kv_rows, void *scratch, void *att_out, void *amax_out, int pdl, void *stream) {
    PromptAttnPlan pl;
    if (!q || !k_base || !v_base || !scratch || !att_out || !amax_out) return BM_EINVAL;
    if (!prompt_attn_plan(T, hist0, slab_rows, H, Hkv, &pl) || hist0 + T > kv_rows) return BM_EINVAL;
    if (!aligned16(q) || !aligned16(k_base) || !aligned16(v_base) || !aligned16(scratch) || !aligned16(att_out)) return BM_EINVAL;
    bm::AttnParams p = {};
    p.q = static_cast<const uint16_t *>(q);
    p.k_base = static_cast<const uint16_t *>(k_base);
    p.v_base = static_cast<const uint16_t *>(v_base);
    p.state = nullptr;
    p.M = T; p.H = H; p.Hkv = Hkv; p.kv_rows = kv_rows; p.sigma = hist0; p.NJ = pl.NJ;
    char *sc = static_cast<char *>(scratch);
    p.tickets = reinterpret_cast<unsigned int *>(sc);
    p.pm = reinterpret_cast<float *>(sc + pl.ticket_bytes);
    p.pl = p.pm + (size_t)T * H * pl.NJ;
    p.po = p.pl + (size_t)T * H * pl.NJ;
    p.att = static_cast<uint16_t *>(att_out);
    p.amax = static_cast<unsigned int *>(amax_out);
    p.pdl = pdl & BM_PDL_OVERLAP;
    p.slab_rows = slab_rows;
    p.slab_hist0 = hist0;
    const dim3 grid(pl.units, Hkv, pl.Z);
    return launch_attention<false>(pl.nq, grid, bm::attn_smem_bytes(pl.nq), static_cast<cudaStream_t>(stream), p.pdl, p);
}

// ---------------------------------------------------------------------------- dense draft heads
int bm_dense_head(const void *h, const void *W, int fp8, const void *w_scale, int R, int N, int K, void *out, int ldc,
                  void *h_scale_out, int pdl, void *stream) {
    if (!h || !W || !out || R < 1 || R > bm::kDenseMaxRows || N < 16 || (N % 16) != 0 || K < 256 || (K % 256) != 0)
        return BM_EINVAL;
    if (ldc < N || (fp8 && !w_scale) || !aligned16(h) || !aligned16(W)) return BM_EINVAL;
    bm::DenseHeadParams p;
    p.W = W;
    p.h = static_cast<const uint16_t *>(h);
    p.w_scale = static_cast<const float *>(w_scale);
    p.out = static_cast<float *>(out);
    p.h_scale_out = static_cast<float *>(h_scale_out);
    p.R = R; p.N = N; p.K = K; p.ldc = ldc; p.pdl = pdl & BM_PDL_OVERLAP;
    const size_t smem = bm::dense_head_smem(R, K, fp8 != 0);
    if (smem > (size_t)kMaxSmemPerCta) return BM_EINVAL;
    const int sms = current_device().sm_count;
    const int blocks = N / 16;
    int grid = (smem <= (size_t)(kMaxSmemPerCta - 2048) / 2 ? 2 : 1) * sms;   // two CTAs per SM when the rows fit twice
    if (grid * (bm::kDenseThreads / 32) > blocks) grid = (blocks + bm::kDenseThreads / 32 - 1) / (bm::kDenseThreads / 32);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const dim3 g(grid), b(bm::kDenseThreads);
    const int nb = (R + 7) / 8;
#define BM_DENSE_CASE(NB_) \
    if (nb == NB_) return fp8 ? launch_ex(bm::dense_head_kernel<NB_, true>, g, b, smem, st, p.pdl, p) \
                             : launch_ex(bm::dense_head_kernel<NB_, false>, g, b, smem, st, p.pdl, p);
    BM_DENSE_CASE(1) BM_DENSE_CASE(2) BM_DENSE_CASE(3)
#undef BM_DENSE_CASE
    return BM_EINVAL;
}

// ---------------------------------------------------------------------------- N-split GEMV
int bm_t2_gemv_nsplit(const void *A, const void *B, const void *s, const void *ws, int W, int N_shard, int K, int ldc,
                      int col0, int world, int rank, void *const *peer_C0, void *const *peer_C1,
                      void *const *peer_flags, void *state, int poll_limit, int pdl, void *stream) {
    if (poll_limit < 0) return BM_EINVAL;
    if (world < 2 || world > 8 || rank < 0 || rank >= world || col0 < 0 || (col0 % 8) != 0 || col0 + N_shard > ldc ||
        !peer_C0 || !peer_C1 || !peer_flags || !state)
        return BM_EINVAL;
    // every rank writes columns [col0, col0 + N_shard) of every rank's [W, ldc] buffers
    void *s0[8], *s1[8];
    for (int i = 0; i < world; ++i) {
        if (!peer_C0[i] || !peer_C1[i]) return BM_EINVAL;
        s0[i] = static_cast<uint16_t *>(peer_C0[i]) + col0;
        s1[i] = static_cast<uint16_t *>(peer_C1[i]) + col0;
    }
    PeerArgs peer{world, rank, s0, s1, peer_flags, state, (unsigned int)poll_limit};
    return gemv_common(A, nullptr, B, s0[rank], s, ws, W, N_shard, K, ldc, BM_OUT_BF16, BM_PATH_AUTO, nullptr, pdl,
                       stream, &peer);
}

// ---------------------------------------------------------- attention without allocation
// Some hosts cannot give the attention a scratch buffer: a C or Go service that owns no
// device allocator of its own, a plugin that runs where the embedding runtime has handed
// all free device memory to its pool, or a latency-critical loop in which a device
// allocation is unwelcome because it synchronises the whole device.  For them the partial
// results of the split-KV attention go into a fixed array that is part of the loaded module,
// so nothing is allocated or freed by the call, by this library or by a library under it.
//
// The array is shared by every call on a device: two calls whose execution can overlap
// (different streams, or different host threads) race on it and must be serialised by the
// caller.  It starts as zeros when the module is loaded, which is what the counters in its
// first KiB need; every call leaves them zero again and writes every other word it reads.
constexpr size_t kStaticAttnScratchBytes = BM_STATIC_ATTN_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_attn_scratch[kStaticAttnScratchBytes];

constexpr int kMaxDevices = 64;
static void *g_static_attn_ptr[kMaxDevices];      // device address of the array, per device
static std::mutex g_static_attn_mutex;

// Looks the array's address up on the current device, once per device.  The look-up is a
// runtime call, so it is refused while `stream` is capturing: the first call on a device has to be
// made outside stream capture.
static int static_attn_scratch(void **out, cudaStream_t stream) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_status(e);
    if (dev < 0 || dev >= kMaxDevices) return BM_EINVAL;
    std::lock_guard<std::mutex> lock(g_static_attn_mutex);
    if (g_static_attn_ptr[dev] == nullptr) {
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
            fprintf(stderr, "bm_verify_attention_static: first call on device %d while its stream is capturing; "
                            "call it once outside capture\n", dev);
            return BM_ECAPTURE;
        }
        void *ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_attn_scratch);
        if (e != cudaSuccess) return cuda_status(e);
        if (ptr == nullptr) return BM_EINVAL;
        g_static_attn_ptr[dev] = ptr;
    }
    *out = g_static_attn_ptr[dev];
    return BM_OK;
}

int bm_verify_attention_static(const void *q, const void *k_base, const void *v_base, int M, int H, int Hkv,
                               int kv_rows, int sigma, const void *state, void *att_out, void *q_out,
                               void *q_prep, void *asum, void *s_out, int pdl, void *stream) {
    if (M < 1 || H < 1 || sigma < 0) return BM_EINVAL;
    const size_t need = bm::attn_scratch_bytes(M, H, sigma);
    if (need > kStaticAttnScratchBytes) {
        fprintf(stderr,
                "bm_verify_attention_static: M=%d H=%d sigma=%d needs %zu scratch bytes, the built-in array "
                "holds %zu; use bm_verify_attention with caller scratch\n",
                M, H, sigma, need, kStaticAttnScratchBytes);
        return BM_ETOOBIG;
    }
    void *scratch = nullptr;
    const int rc = static_attn_scratch(&scratch, static_cast<cudaStream_t>(stream));
    if (rc != BM_OK) return rc;
    return bm_verify_attention(q, k_base, v_base, M, H, Hkv, kv_rows, sigma, state, scratch, att_out, q_out,
                               q_prep, asum, s_out, pdl, stream);
}

}  // extern "C"
