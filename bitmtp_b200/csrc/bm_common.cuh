// Device-side helpers shared by every kernel file: error reporting, mbarrier /
// bulk-copy wrappers with bounded waits, warp reductions.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "bm_math.h"

namespace bm {

// ---- error word ------------------------------------------------------------
// One int per device.  A kernel that gives up on a wait stores a code here and
// returns; bm_device_error() reads and clears it.  0 = no error.
enum DevErr : int {
    kErrNone = 0,
    kErrGemvWaitTimeout = 1,   // a weight tile never arrived in shared memory
};

// The library is one translation unit, so the definition lives here.
__device__ int g_dev_err = 0;

__device__ __forceinline__ void report_error(int code) { atomicCAS(&g_dev_err, 0, code); }

// ---- shared-memory addresses ------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier + bulk async copy (TMA, untiled form) -------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

// Global -> shared bulk copy.  Both addresses 16-byte aligned, bytes a multiple
// of 16.  Completion is signalled on `bar` as transaction bytes.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes,
                                         uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Wait for a phase with an iteration limit.  Returns false when the limit runs
// out; the caller then reports an error and leaves instead of spinning forever.
// try_wait itself blocks for a hardware-defined slice, so 1<<22 polls is on the
// order of seconds, far beyond any healthy copy.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity) {
    for (int it = 0; it < (1 << 22); ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it > 64) __nanosleep(64);
    }
    return false;
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Same, but gives up at once when another warp of the CTA has already given up
// (`*abort_flag` != 0), so that one lost copy does not make every warp of the CTA sit
// out its own full limit in turn.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity,
                                                  volatile int *abort_flag) {
    for (int it = 0; it < (1 << 22); ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if (it > 32) {
            if (*abort_flag) return false;
            __nanosleep(32);
        }
    }
    *abort_flag = 1;
    return false;
}

// ---- programmatic dependent launch ------------------------------------------
// wait: block until every grid this one depends on has finished and its writes
// are visible.  launch_dependents: allow the next grid in the stream to start
// its own prologue.  Both are no-ops for a kernel launched without the
// programmatic-serialisation attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// 16-byte asynchronous copy global -> shared (both addresses 16-byte aligned), and the wait for all of a
// thread's outstanding ones.
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
// Batches of such copies: commit closes the batch issued so far, wait_batches<N> returns when at most
// N of this thread's most recent batches are still in flight.
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_batches() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ---- thread-block clusters ----------------------------------------------------
// One barrier phase = arrive + wait by every
// thread of every CTA of the cluster that has not exited (a hardware barrier, no polling of memory), and
// reads of another CTA's shared memory through its cluster-wide address.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t cluster_map(const void *own_shared, uint32_t rank) {
    uint32_t mapped;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                 : "=r"(mapped) : "r"((uint32_t)__cvta_generic_to_shared(own_shared)), "r"(rank));
    return mapped;
}
__device__ __forceinline__ float4 cluster_ld4(uint32_t a) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ float2 cluster_ld2(uint32_t a) {
    float2 v;
    asm volatile("ld.shared::cluster.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ void cluster_st_f32(uint32_t a, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_st_s32(uint32_t a, int v) {
    asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}

// ---- warp reductions in the oracle's butterfly order -------------------------
// Exact int32 -> fp32 of a group sum without the conversion unit.  A group sum is at most 128 * 127 * 3
// in magnitude, so kGroupSumBias + G is the bit pattern of the float 1.5 * 2^23 + G; subtracting 1.5 * 2^23
// (exact: both operands and the result are integers below 2^24) gives (float)G.  The bias is added for free
// by starting the MMA accumulator at bias - 2 * sum(A) instead of -2 * sum(A).
constexpr int kGroupSumBias = 0x4B400000;
__device__ __forceinline__ float group_sum_to_float(int biased) { return __int_as_float(biased) - 12582912.0f; }

__device__ __forceinline__ float warp_sum_butterfly(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = v + __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

__device__ __forceinline__ float bf16_bits_to_f32(uint16_t h) {
    return __uint_as_float(((uint32_t)h) << 16);
}

}  // namespace bm
