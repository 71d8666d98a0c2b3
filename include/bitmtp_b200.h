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
#define BM_ETOOBIG 27          /* the request exceeds a built-in limit               */
#define BM_ECAPTURE 16         /* set-up that cannot run while the stream is capturing */
#define BM_ECUDA_BASE 1000

/* out_kind for bm_t2_gemv */
#define BM_OUT_BF16 0          /* C is bf16 [W, ldc]                               */
#define BM_OUT_F32 1           /* C is fp32 [W, ldc]                               */
#define BM_OUT_F32_OF_BF16 2   /* C is fp32 holding the bf16-rounded value (logits) */

/* consumer selection for bm_t2_gemv */
/* `pdl` values (bit mask).  BM_PDL_OVERLAP: the launch may start before the previous kernel
 * of the stream has finished and waits for it on the device before reading its output.
 * BM_PDL_STABLE_STATE (bm_verify_attention only, with BM_PDL_OVERLAP): the caller promises
 * that the step record and the history rows [0, cache_len) were written by launches that
 * completed before the current run of overlapped launches began (true for a captured
 * replay whose record is set before the graph launch), so they are read without waiting. */
#define BM_PDL_OVERLAP 1
#define BM_PDL_STABLE_STATE 2
#define BM_PDL_STAGED 4        /* bm_t2_gemv_row_fused only: use the shared-memory-staged kernel at every size */

#define BM_PATH_AUTO 0
#define BM_PATH_DP4A 1
#define BM_PATH_MMA 2
#define BM_PATH_ROWWARP 3      /* W <= 8, K % 512 == 0, N % 16 == 0: a warp per 16-row block */
#define BM_PATH_DIRECT 4       /* W <= 4, K <= 10240: a warp per row, operands straight into registers */

/* Library / build identification: returns a static string. */
const char *bm_version(void);

/* Number of SMs the launch heuristics were sized for on the current device. */
int bm_sm_count(void);

/* Kernel launches this library has issued in this process (a launch recorded into a
 * stream capture counts once, at capture time; replays of the graph are the caller's to
 * count).  Host-side diagnostic counter; no reference counterpart. */
unsigned long long bm_launch_count(void);

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
 *   path      BM_PATH_*  (AUTO: the MMA consumer whenever K % 256 == 0, which
 *             covers every model shape; the lanes-across-K dp4a consumer otherwise.
 *             BM_PATH_MMA with K % 256 != 0 is BM_EINVAL; any other value is BM_EINVAL)
 *   C         16-byte aligned, ldc a multiple of 4
 *   G_out     int32 [W, N, K/128] exact group sums, or NULL
 *   pdl       1 = launch with programmatic stream serialisation: the kernel
 *             requests its weight tiles at once and waits for the previous
 *             kernel in the stream only before it reads A and s */
int bm_t2_gemv(const void *A, const void *B, void *C, const void *s, const void *ws, int W, int N,
               int K, int ldc, int out_kind, int path, void *G_out, int pdl, void *stream);

/* The same product on GEMV-ready activations (q_prep / asum of the quantising operators):
 * the kernel then skips its own byte permutation and group sums, and for K == 2048 reads
 * its fragments straight from A_prep without staging them.  K % 256 == 0.  Results are
 * bit-identical to bm_t2_gemv on the natural-order codes.  No counterpart in the
 * reference, whose kernel re-reads natural-order activations from global memory for
 * every output row. */
int bm_t2_gemv_prepared(const void *A_prep, const void *a_sums, const void *B, void *C, const void *s,
                        const void *ws, int W, int N, int K, int ldc, int out_kind, int pdl,
                        void *stream);

/* Algorithmic bytes one bm_t2_gemv call moves (codes + scales + A + s + C), the
 * numerator of the roofline figure. Host-only arithmetic. */
int64_t bm_t2_gemv_bytes(int W, int N, int K, int out_kind);

/* ------------------------------------------------------------------ fused operators
 * `pdl` on every call below has the meaning given at bm_t2_gemv: the kernel is
 * launched with programmatic stream serialisation and waits for its
 * predecessor before its first read of a tensor the predecessor writes. */

/* Per-row absmax INT8 quantisation: x bf16 [M, K] -> q int8 [M, K], s fp32 [M]
 * with s = 127 / max(absmax, 1e-5), q = clamp(rint(x * s), -128, 127).
 * Replaces T2LinearKernel.quant_input (src/bonsai_sft/gpu/model.py:632-636).
 *
 * Every quantising operator below takes the same trio of outputs, any of which may be
 * NULL (at least one of q / q_prep must be given; q_prep and asum go together):
 *   q       int8 [M, K] in natural order, what the reference's operator returns
 *   q_prep  int8 [M, K] GEMV-ready: each run of 16 codes stored as its 4x4 byte
 *           transpose (q_prep[4t+e] = q[4e+t]), the order bm_t2_gemv_prepared consumes
 *   asum    int32 [M, K/128]: the sum of the codes of each 128-group (K % 128 == 0) */
int bm_quant_rows(const void *x, int M, int K, void *q, void *q_prep, void *asum, void *s, int pdl,
                  void *stream);

/* (gather | residual add) + RMSNorm + (INT8 quantisation | bf16 store), one row per CTA.
 *   x       bf16 [*, dim]; row m is x[gather[m]] when gather (int64 [M]) is given,
 *           else x[row0 + m].  gather_rows = rows of x: an id outside [0, gather_rows)
 *           reads the nearest valid row instead of memory outside the table
 *   res     optional bf16 [*, dim], read at row0 + m: h = bf16(x + res)
 *   w       bf16 [dim] norm weight;  dim a multiple of 256, <= 8192
 *   h_out   optional bf16 [M, dim]: the row before the norm
 *   q, q_prep, asum, s   optional quantised outputs (see bm_quant_rows) + fp32 [M]
 *   n_out   optional bf16 [M, dim]: the normed row
 * Replaces _fused_norm_quant, _fused_add_norm_quant, RMSNorm.forward on the logit
 * rows and the embedding gather (src/bonsai_sft/gpu/model.py:307-336, 290-295,
 * 1386, 1401-1402). */
int bm_rmsnorm_fused(const void *x, const void *gather, int gather_rows, const void *res, const void *w,
                     float eps, int M, int dim, int row0, void *h_out, void *q, void *q_prep, void *asum, void *s,
                     void *n_out, int pdl, void *stream);

/* inner = bf16(bf16(silu(gate)) * up), then the quantisation of bm_quant_rows.
 * gu bf16 [M, 2F] = gate | up; q int8 [M, F]; s fp32 [M]; inner_out optional bf16 [M, F].
 * Replaces src/bonsai_sft/gpu/model.py:1059-1061. */
int bm_silu_mul_quant(const void *gu, int M, int F, void *q, void *q_prep, void *asum, void *s,
                      void *inner_out, int pdl, void *stream);

/* Split qkv, per-head RMSNorm of q and k, RoPE from bf16 tables, append K / V rows.
 *   xqkv bf16 [M, (H + 2*Hkv)*128]; q_w, k_w bf16 [128]; cos_t, sin_t bf16 [max_pos, 128];
 *   positions int64 [M]; k_base, v_base bf16 [Hkv, kv_rows, 128] (one layer of the shared
 *   buffer), rows [sigma, sigma + M) are written; q_out bf16 [M, H, 128].
 * Replaces _fused_qkv_qknorm_rope_kv_write (src/bonsai_sft/gpu/model.py:388-436). */
int bm_qknorm_rope_kvappend(const void *xqkv, const void *q_w, const void *k_w, float eps,
                            const void *cos_t, const void *sin_t, const void *positions, int M,
                            int H, int Hkv, void *k_base, void *v_base, int kv_rows, int sigma,
                            void *q_out, int pdl, void *stream);

/* Writes {cache_len, n_pend, role, P} into the 16-byte device record the attention
 * reads.  role: 0 draft, 1 verify, 2 ar.  Takes the place of the host-side mask
 * rebuild GraphAtlas.prepare_step (src/bonsai_sft/gpu/fast_runtime.py:391-465). */
int bm_set_step_state(void *state, int cache_len, int n_pend, int role, int P, void *stream);

/* Copies rows [src_row, src_row + n) onto [dst_row, dst_row + n) in each of `planes`
 * planes of a bf16 [planes, kv_rows, 128] buffer (non-overlapping ranges).
 * Replaces GraphAtlas.commit_kv / commit_kv_from_verify
 * (src/bonsai_sft/gpu/fast_runtime.py:467-508). */
int bm_kv_copy_rows(void *kv, int planes, int kv_rows, int src_row, int dst_row, int n,
                    void *stream);

/* Scratch bytes bm_verify_attention needs for (M, H, sigma): a 1 KiB header of counters, the
 * split-KV partials (one per 128 keys, query row and head) and one bf16 copy of the output rows.
 * Host-only arithmetic. */
int64_t bm_verify_attention_scratch_bytes(int M, int H, int sigma);

/* Block-verify attention of one layer + INT8 quantisation of its output rows.
 *   q bf16 [M, H, 128]; k_base, v_base bf16 [Hkv, kv_rows, 128]; history rows are
 *   [0, cache_len), the M rows of this replay sit at [sigma, sigma + M);
 *   state: the record written by bm_set_step_state;
 *   scratch: bm_verify_attention_scratch_bytes bytes, 16-byte aligned, ZERO before its
 *   first use (its first KiB holds counters that every call leaves zero again); not
 *   shared by calls that may execute at the same time;
 *   att_out bf16 [M, H*128] or NULL; q_out / q_prep / asum: the quantised rows (see
 *   bm_quant_rows); s_out fp32 [M].  H*128 a multiple of 256; sigma <= 8064.
 * Two launches: the attention itself (scores, softmax, numerators and the merge of the
 * split-KV partials - by the last CTA to finish, or, where the device holds the whole grid
 * as thread-block clusters, through distributed shared memory; same order, same bits) and
 * the flat quantisation of its rows.
 * Visibility follows the reference's draft / verify / ar masks.  Replaces the
 * attention and o-projection input quantisation of
 * Attention.forward_sdlm_graph_kernel (src/bonsai_sft/gpu/model.py:989-1005) and the
 * mask tensors of src/bonsai_sft/gpu/fast_runtime.py:345-372, 423-465. */
int bm_verify_attention(const void *q, const void *k_base, const void *v_base, int M, int H,
                        int Hkv, int kv_rows, int sigma, const void *state, void *scratch,
                        void *att_out, void *q_out, void *q_prep, void *asum, void *s_out, int pdl,
                        void *stream);

/* bm_verify_attention for callers that cannot provide scratch memory; it has no
 * counterpart in the reference.  Same arguments without `scratch`: the split-KV partials go to
 * an array built into the library (BM_STATIC_ATTN_SCRATCH_BYTES per device), so the call
 * allocates and frees nothing.  Requests whose
 * bm_verify_attention_scratch_bytes(M, H, sigma) exceeds that size return BM_ETOOBIG
 * (16 rows x 16 heads fit up to sigma = 7808, 32 rows x 32 heads up to sigma = 1792); every
 * shape is also bound by bm_verify_attention's own sigma <= 8064 (BM_EINVAL beyond it).
 * The first call on a device looks the array's address up, which is a runtime call: make it
 * before any stream capture on that device.  A first call on a capturing stream returns
 * BM_ECAPTURE and enqueues nothing.  All calls on a device share the one array: calls that
 * may execute at the same time must be serialised by the caller. */
#define BM_STATIC_ATTN_SCRATCH_BYTES (8u << 20)
int bm_verify_attention_static(const void *q, const void *k_base, const void *v_base, int M, int H,
                               int Hkv, int kv_rows, int sigma, const void *state, void *att_out,
                               void *q_out, void *q_prep, void *asum, void *s_out, int pdl,
                               void *stream);

/* gate|up projection with SiLU(gate) * up in the epilogue: B [2F, K/4] holds the gate rows, then the
 * up rows (scales ws [2F, K/128] likewise); inner_out bf16 [W, F] = bf16(silu(bf16 g) * bf16 u), the value
 * bm_silu_mul_quant forms from the bf16 projection outputs; amax_out uint32 [W] receives, by atomic
 * max, the bits of max |inner| per row and must be zero on entry.  GEMV-ready activations as for
 * bm_t2_gemv_prepared; W <= 16.  With bm_quant_rows_amax it replaces the gate/up projections and
 * `F.silu(g) * u` + quant_input of FeedForward (src/bonsai_sft/gpu/model.py:1053-1064), bit for bit. */
int bm_t2_gemv_gate_up_silu(const void *A_prep, const void *a_sums, const void *B, const void *ws,
                            const void *s, int W, int F, int K, void *inner_out, void *amax_out, int pdl,
                            void *stream);

/* Token ids, positions and the step record of one replay in one launch.
 *   kind 0 (draft, M = P + D): tok = pending[0..n_pend) | 0 .. | pending[n_pend-1] at row P | mask_id ..;
 *           pos = cache_len + i (pending rows), 0 (padding rows), cache_len + n_pend - 1 + k (block rows);
 *   kind 1 (verify, M = D + 1): tok = pending[n_pend-1] | draft[0..D); pos = cache_len - 1 + i;
 *   kind 2 (AR, M = 1): tok = src_a[0], pos = cache_len;
 *   kind 3 (prompt slab of width M, n_pend real rows): tok = src_a[0..n_pend) | 0 ..; pos = cache_len + i | 0 ...
 * src_a = pending tokens (int64; the slab's prompt ids for kind 3), src_b = draft tokens (kind 1); tok, pos int64 [M]; state as written by
 * bm_set_step_state (n_pend clamped to [0, P] for a draft, 0 otherwise).  Replaces the per-step tensor
 * fills of src/bonsai_sft/gpu/fast_generate.py:1015-1055, 247-256 and fast_runtime.prepare_step. */
int bm_stage_replay_inputs(int kind, const void *src_a, const void *src_b, int n_pend, int cache_len, int M, int D,
                           long long mask_id, int role, int P, void *tok, void *pos, void *state, void *stream);

/* End of one decode step and start of the next in one launch: gen_dst[0..n_commit) = src[0..n_commit) (the
 * committed ids into the output buffer); pending[0..n_commit) = the same ids after a confidence commit
 * (verified == 0), pending[0] = src[n_commit-1] after a verified step; then, if stage != 0, the draft inputs of
 * width M = P + D are staged from the pending ids as bm_stage_replay_inputs kind 0 does (n_pend = n_commit or 1).
 * Replaces the copies of src/bonsai_sft/gpu/fast_generate.py:1121-1140 and the fills of :1015-1037. */
int bm_commit_stage_draft(const void *src, int n_commit, int verified, void *gen_dst, void *pending, int stage,
                          int cache_len, int M, int D, long long mask_id, int role, int P, void *tok, void *pos,
                          void *state, void *stream);

/* Width-1 GEMV that makes its own INT8 activations from a bf16 row, for the AR replay (one launch per
 * projection instead of two): every CTA quantises the row itself.
 *   src_mode 1: x bf16 [K] with the bits of its absmax in amax_in[0] (as left by
 *               bm_rope_verify_attention_rows or bm_t2_gemv_gate_up_silu); amax_zero[0] (optional, another
 *               word) is cleared.  Equals bm_quant_rows_amax + bm_t2_gemv_prepared.
 *   src_mode 2: h = bf16(x_row + res) (x_row = x[gather[0]] when gather is given, the id clamped to
 *               [0, gather_rows); res optional), stored to
 *               h_out [K] (must not alias x or res), then RMSNorm with norm_w and eps and the codes.
 *               K == 2048.  Equals bm_rmsnorm_fused + bm_t2_gemv_prepared.
 *   silu != 0: B holds 2N rows (gate, then up), C bf16 [N] = bf16(silu(g) * u), amax_out[0] gathers its
 *               absmax (zero on entry), as bm_t2_gemv_gate_up_silu.
 * Other arguments as bm_t2_gemv.  Bit-identical to the chains named above. */
int bm_t2_gemv_row_fused(int src_mode, const void *x, const void *gather, int gather_rows, const void *res,
                         const void *norm_w, float eps, void *h_out, const void *amax_in, void *amax_zero, const void *B,
                         const void *ws, int N, int K, void *C, int ldc, int out_kind, int silu, void *amax_out,
                         int pdl, void *stream);

/* Clears n 32-bit words (stream-ordered memset): the absmax words of the first layer of a forward. */
int bm_zero_words(void *p, int n, void *stream);

/* bm_quant_rows for rows whose absmax is already known (amax_in uint32 [M]: float bits).  amax_zero
 * (optional, another array): M words cleared for the next producer.  K % 256 == 0. */
int bm_quant_rows_amax(const void *x, const void *amax_in, void *amax_zero, int M, int K, void *q,
                       void *q_prep, void *asum, void *s, int pdl, void *stream);

/* N-split of one wide layer over the GPUs of a node, GEMV and exchange in one kernel: this rank
 * computes the N_shard output rows of its shard (B, ws: the shard's codes and scales) and stores every
 * value at columns [col0, col0 + N_shard) of EVERY rank's bf16 [W, ldc] output buffer over NVLink
 * (peer_C0[i] / peer_C1[i]: the two buffers of rank i as mapped into this process, e.g. by torch
 * symmetric memory; calls use them in turn, so a rank that is one call ahead never writes into rows a
 * peer's consumers still read).  The last CTA to finish publishes the call number in slot [rank] of
 * every peer's flag array (peer_flags[i]: uint32 [world] of rank i) and waits, with a limit, until all
 * peers have published the same number in the local array: when the kernel ends the full [W, ldc]
 * block is in this GPU's buffer, bit-identical to the single-GPU product.  state: local uint32 [4],
 * zero before the first call ([0] CTA counter, [1] completed calls, [2] status, [3] unused;
 * device-resident, so a captured graph can be replayed).  The result of call k (k = 1, 2, ...) is in
 * buffer k & 1.  All ranks make the same sequence of calls.
 * A peer that does not publish within poll_limit polls of its flag (0 = the default, 2^22 polls of
 * >= 100 ns each) ends the wait: the kernel returns, state[2] = k names the call, and
 * bm_device_error() = 4.  The output of call k is then INVALID for that peer's columns (they still
 * hold the values of call k - 2); the local shard's columns are correct.  Read state[2] with the
 * step's own device-to-host copy to learn of it without synchronising the device.
 * The reference has no multi-GPU inference path; this is the exchange step of the wide-layer
 * configuration. */
int bm_t2_gemv_nsplit(const void *A, const void *B, const void *s, const void *ws, int W, int N_shard,
                      int K, int ldc, int col0, int world, int rank, void *const *peer_C0,
                      void *const *peer_C1, void *const *peer_flags, void *state, int poll_limit, int pdl,
                      void *stream);

/* bm_qknorm_rope_kvappend + bm_verify_attention in two launches instead of three: the attention's chunk
 * kernel reads the qkv projection output (xqkv bf16 [M, (H + 2 Hkv) * 128]) and does the q/k head norm, the
 * RoPE and the append of the replay's K and V rows at [sigma, sigma + M) of the planes itself.  Other
 * arguments and results as for those two calls; bit-identical to them. */
int bm_rope_verify_attention(const void *xqkv, const void *q_w, const void *k_w, float eps, const void *cos_t,
                             const void *sin_t, const void *positions, void *k_base, void *v_base, int M,
                             int H, int Hkv, int kv_rows, int sigma, const void *state, void *scratch,
                             void *att_out, void *q_out, void *q_prep, void *asum, void *s_out, int pdl,
                             void *stream);

/* bm_rope_verify_attention without the quantisation and with the merge spread over (row, 4 heads) CTAs:
 * writes the bf16 rows att_out [M, H*128] and folds each row's absmax into amax_out uint32 [M] by atomic
 * max (float bits; zero on entry).  bm_quant_rows_amax(att_out, amax_out, ...) then yields exactly the
 * codes and multipliers of bm_rope_verify_attention.  H % 4 == 0. */
int bm_rope_verify_attention_rows(const void *xqkv, const void *q_w, const void *k_w, float eps,
                                  const void *cos_t, const void *sin_t, const void *positions, void *k_base,
                                  void *v_base, int M, int H, int Hkv, int kv_rows, int sigma,
                                  const void *state, void *scratch, void *att_out, void *amax_out, int pdl,
                                  void *stream);

/* Row argmax (lowest index on ties): logits fp32 [rows, ld] -> idx int64 [rows],
 * optional max_out fp32 [rows].  Replaces `.argmax(dim=-1)` on the logit rows
 * (src/bonsai_sft/gpu/fast_generate.py:786, 809, 1079). */
int bm_argmax_rows(const void *logits, int rows, int vocab, int ld, void *idx, void *max_out,
                   void *stream);

/* Draft confidence chain: idx int64 [D] = row argmax, conf fp32 [D] =
 * exp(max - logsumexp), *n_out (device int32) = 1 + number of leading rows r >= 1
 * with conf[r] > tau.  max_buf: fp32 [D] work area.  Replaces _fused_draft_chain
 * (src/bonsai_sft/gpu/fast_generate.py:111-130). */
int bm_draft_chain(const void *logits, int D, int vocab, int ld, float tau, void *idx,
                   void *max_buf, void *conf, void *n_out, void *stream);

/* The two reductions above spread over 16 to 128 CTAs per logit row (more when there are few rows) (one CTA per row leaves most of the GPU idle on
 * rows of 151936 values); same results bit for bit.  `scratch`: bm_logit_scratch_bytes() bytes of device
 * memory, 16-byte aligned, zero before its first use (the kernels leave its counters zero), not shared by
 * calls that may run at the same time.  rows, D <= 32.  bm_draft_chain_split is ONE launch where the device holds a
 * 16-CTA thread-block cluster per row (each CTA reads its part of the row once, maxima and chunk sums travel
 * through distributed shared memory), else an argmax launch followed by a confidence launch. */
long long bm_logit_scratch_bytes(void);
int bm_argmax_rows_split(const void *logits, int rows, int vocab, int ld, void *idx, void *max_out, void *scratch,
                         void *stream);
int bm_draft_chain_split(const void *logits, int D, int vocab, int ld, float tau, void *idx, void *max_buf,
                         void *conf, void *n_out, void *scratch, void *stream);

/* Freeze + pack on the device: w bf16 [N, K] (latent or already frozen) -> packed uint8 [N, K/4] (four
 * natural-order codes per byte, value + 2), scale bf16 [N, K/128] and, when frozen != NULL, the bf16
 * weights on the {-s, 0, +s} grid.  The arithmetic of freeze_quantize_to_ternary_g128
 * (src/bonsai_sft/ternary_modules.py:86-93) followed by _pack_t2_g128
 * (src/bonsai_sft/gpu/convert_bonsai_mtp_to_gpu.py:127-144), which the reference's converter runs on the
 * CPU; same bytes.  K % 128 == 0; w and frozen 16-byte aligned. */
int bm_pack_t2_g128(const void *w, int N, int K, void *packed, void *scale, void *frozen, void *stream);

/* The packed product for MANY rows at once (a prompt): C bf16 [T, ldc] = the value bm_t2_gemv_prepared
 * gives every row alone, bit for bit, with each weight byte read once per 32 rows instead of once per
 * GEMV launch.  A_prep / a_sums / s: GEMV-ready INT8 rows, their group sums and multipliers for T rows;
 * N % 128 == 0, K % 128 == 0.  Tensor-core kernel (mma.sync int8, exact int32 group sums, the GEMV's
 * fp32 order).  Replaces the dense bf16 fallback of T2LinearKernel.forward behind forward_sdlm_prefill
 * (src/bonsai_sft/gpu/model.py:650-656, 1306-1340). */
int bm_t2_gemm_wide(const void *A_prep, const void *a_sums, const void *B, void *C, const void *s, const void *ws,
                    int T, int N, int K, int ldc, int pdl, void *stream);

/* Causal attention of a whole prompt in one launch.  The K / V rows of the T prompt rows already sit at
 * rows [hist0, hist0 + T) of the planes (bm_qknorm_rope_kvappend with sigma = hist0); q bf16 [T, H, 128]
 * are the rotated queries.  The rows are served as AR-causal slabs of slab_rows rows (slab s sees rows
 * [0, hist0 + s * slab_rows) as history and its own rows causally), which is exactly what
 * bm_verify_attention computes when called once per slab with sigma = cache_len = the slab's start, so
 * the results equal that slab-by-slab prefill bit for bit.  att_out bf16 [T, H*128]; amax_out uint32 [T]
 * (zero on entry) gathers the row absmax bits for bm_quant_rows_amax.  scratch:
 * bm_prompt_attention_scratch_bytes(...) bytes, zero before first use.  slab_rows <= 32,
 * hist0 + T <= 8064.  Replaces the SDPA call of the prompt forward (model.py:797-800). */
long long bm_prompt_attention_scratch_bytes(int T, int hist0, int slab_rows, int H, int Hkv);
int bm_prompt_attention(const void *q, const void *k_base, const void *v_base, int T, int hist0, int slab_rows,
                        int H, int Hkv, int kv_rows, void *scratch, void *att_out, void *amax_out, int pdl,
                        void *stream);

/* Dense tied head for the draft role: out fp32 [R, ldc] = bf16-rounded logits of the R bf16 rows
 * h [R, K] against the dense table W [N, K].
 *   fp8 == 0: W is bf16 (the tied embedding itself), out = bf16(h . W^T): the `bf16_raw` branch of
 *             Transformer._lm_head (src/bonsai_sft/gpu/model.py:1276-1282, F.linear);
 *   fp8 != 0: W is e4m3 (prepare_fp8_lm_head, model.py:1169-1194: W / w_scale with w_scale =
 *             bf16(amax|W| / 448) in *w_scale, a device fp32); the rows are scaled per tensor by
 *             h_scale = bf16(amax|h| / 448), cast to e4m3 and the product is multiplied by
 *             h_scale * w_scale: the `fp8` branch (model.py:1266-1275, torch._scaled_mm).
 *             h_scale_out (optional device fp32) receives h_scale.
 * fp32 accumulation on the tensor cores (mma.sync, fixed k order); R <= 24, N % 16 == 0,
 * K % 256 == 0.  Streams the whole table once: 2 (1) bytes per weight. */
int bm_dense_head(const void *h, const void *W, int fp8, const void *w_scale, int R, int N, int K, void *out,
                  int ldc, void *h_scale_out, int pdl, void *stream);

/* *n_out (device int32) = length of the longest common prefix of draft[0:D] and
 * verify[0:D] (int64).  Replaces _fused_verify_accept
 * (src/bonsai_sft/gpu/fast_generate.py:133-146). */
int bm_verify_accept(const void *draft, const void *verify, int D, void *n_out, void *stream);

#ifdef __cplusplus
}
#endif

#endif /* BITMTP_B200_H_ */
