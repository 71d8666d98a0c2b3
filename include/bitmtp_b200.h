/* C ABI of libbitmtp_b200.so: the B200 (sm_100a) replacement for the native
 * operator behind BitMTP's packed T2-g128 decode path.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller unless a comment says
 *     host; the library allocates nothing and keeps no per-call state;
 *   - `stream` is a cudaStream_t passed as void*; calls only enqueue work and are
 *     legal inside stream capture;
 *   - bf16 tensors are passed as raw 16-bit patterns;
 *   - functions return 0 on success, BM_EINVAL for a shape / alignment the
 *     kernels do not take, or 1000 + the cudaError_t of a failed launch.
 */
#ifndef BITMTP_B200_H_
#define BITMTP_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BM_OK 0
#define BM_EINVAL 22
#define BM_ECUDA_BASE 1000

/* out_kind for bm_t2_gemv */
#define BM_OUT_BF16 0          /* C is bf16 [W, ldc]                               */
#define BM_OUT_F32 1           /* C is fp32 [W, ldc]                               */
#define BM_OUT_F32_OF_BF16 2   /* C is fp32 holding the bf16-rounded value (logits) */

/* consumer selection for bm_t2_gemv */
#define BM_PATH_AUTO 0
#define BM_PATH_DP4A 1
#define BM_PATH_MMA 2

/* Library / build identification: returns a static string. */
const char *bm_version(void);

/* Number of SMs the launch heuristics were sized for on the current device. */
int bm_sm_count(void);

/* Reads and clears the per-device error word that kernels set when a bounded
 * wait runs out (0 = none, 1 = a GEMV weight tile never arrived). Synchronises
 * the device. */
int bm_device_error(void);

/* Drop-in for the reference's only native symbol
 * (src/bonsai_sft/gpu/t2g128_kernels/t2g128_kernels.cu:123-148, bound with
 * ctypes in src/bonsai_sft/gpu/model.py:206-219):
 *   C[M,N] (bf16) = ((A int8 [M,K]) x (B 2-bit codes [N,K/4]) per-group scaled by
 *   ws bf16 [N,K/128]) / s fp32 [M].
 * Same argument order and types.  Unlike the reference it takes every
 * 1 <= M <= 32, K % 128 == 0, N % 8 == 0; an unsupported shape prints to stderr
 * and returns without writing C, as the reference does. */
void t2g128_int8xint2_linear(int8_t *A, int8_t *B, void *C, float *s, void *ws, int M, int N,
                             int K, void *stream);

/* Status-returning form of the same operator (replaces the same reference
 * lines), with the extras the tests and the runtime need:
 *   ldc       row stride of C in elements (>= N)
 *   out_kind  BM_OUT_*
 *   path      BM_PATH_*  (AUTO: dp4a for W <= 2, MMA above)
 *   G_out     int32 [W, N, K/128] exact group sums, or NULL
 *   pdl       1 = launch with programmatic stream serialisation: the kernel
 *             requests its weight tiles at once and waits for the previous
 *             kernel in the stream only before it reads A and s */
int bm_t2_gemv(const void *A, const void *B, void *C, const void *s, const void *ws, int W, int N,
               int K, int ldc, int out_kind, int path, void *G_out, int pdl, void *stream);

/* Algorithmic bytes one bm_t2_gemv call moves (codes + scales + A + s + C), the
 * numerator of the roofline figure. Host-only arithmetic. */
int64_t bm_t2_gemv_bytes(int W, int N, int K, int out_kind);

#ifdef __cplusplus
}
#endif

#endif /* BITMTP_B200_H_ */
