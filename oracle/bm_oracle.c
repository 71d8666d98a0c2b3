// CPU oracle for the packed T2-g128 decode path.  TEST INFRASTRUCTURE ONLY:
// tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs link this
// file; nothing under bitmtp_b200/ may.
//
// What is restated, and from where (paths within the reference project):
//   bmo_t2_gemv              src/bonsai_sft/gpu/t2g128_kernels/t2g128_kernels.cu:21-27
//                            (2-bit decode, code-2), :62-81 (int8 x ternary dot,
//                            group scale applied per 128-wide K group), :83-91
//                            (cross-lane sum, division by the activation
//                            multiplier, bf16 store)
//   bmo_quant_rows           src/bonsai_sft/gpu/model.py:632-636
//   bmo_rmsnorm_quant        src/bonsai_sft/gpu/model.py:307-319
//   bmo_add_rmsnorm_quant    src/bonsai_sft/gpu/model.py:322-336
//   bmo_rmsnorm              src/bonsai_sft/gpu/model.py:290-295
//   bmo_silu_mul_quant       src/bonsai_sft/gpu/model.py:1059-1061
//   bmo_qknorm_rope_kvappend src/bonsai_sft/gpu/model.py:388-436
//   bmo_attention            src/bonsai_sft/gpu/model.py:993-1004 with the masks of
//                            src/bonsai_sft/gpu/fast_runtime.py:345-372,391-465
//   bmo_argmax_rows,
//   bmo_draft_chain          src/bonsai_sft/gpu/fast_generate.py:111-130
//   bmo_verify_accept        src/bonsai_sft/gpu/fast_generate.py:133-146
//
// Integer results (group sums, INT8 codes, argmax, accept lengths) are exact by
// definition.  For fp32 sums the reference leaves the order to the launch
// geometry of its CUDA kernel or to torch's reduction kernels; this file fixes
// one order per operation (documented at each function) and the CUDA kernels
// follow the same order, so the two agree bit for bit, while agreement with
// the reference's own fp32 results is to rounding (tests/golden pins both).
//
// Pinning: tests/golden/make_golden.py imports the reference's Python modules
// and records their outputs on seeded inputs; tests/test_oracle_golden.py
// checks this file against those records.

#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#include "../bitmtp_b200/csrc/bm_math.h"

#define BMO_API __attribute__((visibility("default")))

BMO_API int bmo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

BMO_API void bmo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// ---------------------------------------------------------------------------
// Canonical fp32 reductions
// ---------------------------------------------------------------------------

// Sum over 32 lanes in the order of a warp xor-butterfly with offsets
// 16, 8, 4, 2, 1.  After the butterfly every lane holds the same value.
static float bmo_butterfly32(float lane[32]) {
    float tmp[32];
    for (int off = 16; off > 0; off >>= 1) {
        for (int t = 0; t < 32; ++t) tmp[t] = lane[t] + lane[t ^ off];
        memcpy(lane, tmp, sizeof(tmp));
    }
    return lane[0];
}

// Sum of squares of L values: chunks of 32*E consecutive elements; inside a
// chunk lane t accumulates its E consecutive elements with fma in ascending
// order, the 32 lanes are combined by the butterfly, and chunk results are
// added in ascending order.  L must be a multiple of 32*E.
static float bmo_sumsq(const float *h, int L, int E) {
    float total = 0.0f;
    for (int c0 = 0; c0 < L; c0 += 32 * E) {
        float lane[32];
        for (int t = 0; t < 32; ++t) {
            float acc = 0.0f;
            for (int e = 0; e < E; ++e) {
                const float v = h[c0 + t * E + e];
                acc = fmaf(v, v, acc);
            }
            lane[t] = acc;
        }
        total += bmo_butterfly32(lane);
    }
    return total;
}

// Sum of the 16 slot partials in the order of an xor-butterfly with offsets
// 1, 2, 4, 8: ((s0+s1)+(s2+s3)) + ((s4+s5)+(s6+s7)) + ...
static float bmo_slot_tree(float slot[BM_SLOTS]) {
    for (int step = 1; step < BM_SLOTS; step <<= 1)
        for (int i = 0; i < BM_SLOTS; i += 2 * step) slot[i] = slot[i] + slot[i + step];
    return slot[0];
}

// ---------------------------------------------------------------------------
// T2-g128 GEMV / skinny GEMM
// ---------------------------------------------------------------------------
// A   int8  [W, K]      per-token INT8 activations
// B   uint8 [N, K/4]    element j of a row in bits 2*(j%4) of byte j/4; the
//                       stored code c means the ternary value c-2
// ws  bf16  [N, K/128]  group scales
// s   fp32  [W]         activation multipliers (127/absmax); the output is
//                       divided by s (as a multiplication by 1/s)
// G_out   int32 [W, N, K/128] or NULL   exact group sums
// out_f32 fp32  [W, N] or NULL
// out_bf16 bf16 [W, N] or NULL          out_f32 rounded once
//
// fp32 order: group g feeds slot g%16; a slot accumulates
// fma((float)G, scale, slot) over its groups in ascending g; the 16 slots are
// combined by bmo_slot_tree; the sum is multiplied by the IEEE reciprocal
// 1/s[m] (the reference divides under --use_fast_math, i.e. multiplies by an
// approximate reciprocal).
BMO_API void bmo_t2_gemv(const int8_t *A, const uint8_t *B, const uint16_t *ws, const float *s,
                         int W, int N, int K, float *out_f32, uint16_t *out_bf16,
                         int32_t *G_out) {
    const int ng = K / BM_GROUP;
    // byte -> its four ternary values, as one 32-bit store per packed byte
    uint32_t lut[256];
    for (int b = 0; b < 256; ++b) {
        uint32_t v = 0;
        for (int i = 0; i < 4; ++i) v |= ((uint32_t)(uint8_t)(int8_t)(((b >> (2 * i)) & 3) - 2)) << (8 * i);
        lut[b] = v;
    }
#pragma omp parallel
    {
        int8_t *t = (int8_t *)malloc((size_t)K);
#pragma omp for schedule(static)
        for (int n = 0; n < N; ++n) {
            const uint8_t *brow = B + (size_t)n * (K / 4);
            for (int j = 0; j < K / 4; ++j) memcpy(t + 4 * j, &lut[brow[j]], 4);
            for (int m = 0; m < W; ++m) {
                const int8_t *a = A + (size_t)m * K;
                float slot[BM_SLOTS];
                for (int i = 0; i < BM_SLOTS; ++i) slot[i] = 0.0f;
                for (int g = 0; g < ng; ++g) {
                    int32_t G = 0;
                    const int8_t *ag = a + g * BM_GROUP;
                    const int8_t *tg = t + g * BM_GROUP;
                    for (int i = 0; i < BM_GROUP; ++i) G += (int32_t)ag[i] * (int32_t)tg[i];
                    if (G_out) G_out[((size_t)m * N + n) * ng + g] = G;
                    const float sc = bm_bf16_to_f32(ws[(size_t)n * ng + g]);
                    slot[g % BM_SLOTS] = fmaf((float)G, sc, slot[g % BM_SLOTS]);
                }
                const float y = bmo_slot_tree(slot) * (1.0f / s[m]);
                if (out_f32) out_f32[(size_t)m * N + n] = y;
                if (out_bf16) out_bf16[(size_t)m * N + n] = bm_f32_to_bf16(y);
            }
        }
        free(t);
    }
}

// ---------------------------------------------------------------------------
// Activation quantisation and the fused norm helpers
// ---------------------------------------------------------------------------
static void bmo_quant_row_f32(const float *x, int K, int8_t *q, float *s_out) {
    float amax = 0.0f;
    for (int k = 0; k < K; ++k) {
        const float a = fabsf(x[k]);
        amax = a > amax ? a : amax;
    }
    const float s = bm_act_scale(amax);
    for (int k = 0; k < K; ++k) q[k] = (int8_t)bm_quant_i8(x[k], s);
    *s_out = s;
}

// x bf16 [M, K] -> q int8 [M, K], s fp32 [M]
BMO_API void bmo_quant_rows(const uint16_t *x, int M, int K, int8_t *q, float *s) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        float *xf = (float *)malloc(sizeof(float) * K);
        for (int k = 0; k < K; ++k) xf[k] = bm_bf16_to_f32(x[(size_t)m * K + k]);
        bmo_quant_row_f32(xf, K, q + (size_t)m * K, s + m);
        free(xf);
    }
}

// One RMSNorm row with the reference's two bf16 roundings:
// n = bf16(w) * bf16(h * rsqrt(mean(h^2) + eps)), product rounded to bf16.
// E = elements per lane of the sum-of-squares order (8 for hidden rows, 4 for
// a 128-wide head).
static void bmo_rmsnorm_row(const float *h, const uint16_t *w, float eps, int L, int E,
                            float *n_out) {
    const float var = bmo_sumsq(h, L, E) / (float)L;
    const float r = bm_rsqrtf(var + eps);
    for (int k = 0; k < L; ++k) {
        const float hn = bm_bf16_rn(h[k] * r);
        n_out[k] = bm_bf16_rn(bm_bf16_to_f32(w[k]) * hn);
    }
}

// x bf16 [M, dim], w bf16 [dim] -> out bf16 [M, dim]   (final norm)
BMO_API void bmo_rmsnorm(const uint16_t *x, const uint16_t *w, float eps, int M, int dim,
                         uint16_t *out) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        float *h = (float *)malloc(sizeof(float) * dim * 2);
        float *n = h + dim;
        for (int k = 0; k < dim; ++k) h[k] = bm_bf16_to_f32(x[(size_t)m * dim + k]);
        bmo_rmsnorm_row(h, w, eps, dim, 8, n);
        for (int k = 0; k < dim; ++k) out[(size_t)m * dim + k] = bm_f32_to_bf16(n[k]);
        free(h);
    }
}

// x bf16 [M, dim] -> q int8, s fp32
BMO_API void bmo_rmsnorm_quant(const uint16_t *x, const uint16_t *w, float eps, int M, int dim,
                               int8_t *q, float *s) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        float *h = (float *)malloc(sizeof(float) * dim * 2);
        float *n = h + dim;
        for (int k = 0; k < dim; ++k) h[k] = bm_bf16_to_f32(x[(size_t)m * dim + k]);
        bmo_rmsnorm_row(h, w, eps, dim, 8, n);
        bmo_quant_row_f32(n, dim, q + (size_t)m * dim, s + m);
        free(h);
    }
}

// h = bf16(x + residual); then as bmo_rmsnorm_quant.  h_out bf16 [M, dim].
BMO_API void bmo_add_rmsnorm_quant(const uint16_t *x, const uint16_t *res, const uint16_t *w,
                                   float eps, int M, int dim, uint16_t *h_out, int8_t *q,
                                   float *s) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        float *h = (float *)malloc(sizeof(float) * dim * 2);
        float *n = h + dim;
        for (int k = 0; k < dim; ++k) {
            const size_t i = (size_t)m * dim + k;
            const uint16_t hb = bm_f32_to_bf16(bm_bf16_to_f32(x[i]) + bm_bf16_to_f32(res[i]));
            h_out[i] = hb;
            h[k] = bm_bf16_to_f32(hb);
        }
        bmo_rmsnorm_row(h, w, eps, dim, 8, n);
        bmo_quant_row_f32(n, dim, q + (size_t)m * dim, s + m);
        free(h);
    }
}

// h = bf16(x + residual) only (the residual add ahead of the final norm,
// model.py:1401).
BMO_API void bmo_add_bf16(const uint16_t *x, const uint16_t *res, size_t n, uint16_t *out) {
    for (size_t i = 0; i < n; ++i)
        out[i] = bm_f32_to_bf16(bm_bf16_to_f32(x[i]) + bm_bf16_to_f32(res[i]));
}

// gu bf16 [M, 2F] (gate | up) -> inner = bf16(bf16(silu(g)) * u) -> q, s.
// inner_out (bf16 [M, F]) may be NULL.
BMO_API void bmo_silu_mul_quant(const uint16_t *gu, int M, int F, int8_t *q, float *s,
                                uint16_t *inner_out) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m) {
        float *v = (float *)malloc(sizeof(float) * F);
        const uint16_t *g = gu + (size_t)m * 2 * F;
        const uint16_t *u = g + F;
        for (int k = 0; k < F; ++k) {
            const float sg = bm_silu_bf16(bm_bf16_to_f32(g[k]));
            v[k] = bm_bf16_rn(sg * bm_bf16_to_f32(u[k]));
            if (inner_out) inner_out[(size_t)m * F + k] = bm_f32_to_bf16(v[k]);
        }
        bmo_quant_row_f32(v, F, q + (size_t)m * F, s + m);
        free(v);
    }
}

// ---------------------------------------------------------------------------
// q/k head norm + RoPE + KV append
// ---------------------------------------------------------------------------
// xqkv bf16 [M, (H + 2*Hkv) * 128]; q_w, k_w bf16 [128]; cos, sin bf16
// [max_pos, 128]; positions int64 [M].
// k_base / v_base: bf16 [Hkv, kv_rows, 128] of one layer; rows [sigma, sigma+M)
// are written.  q_out bf16 [M, H, 128].
// RoPE (halves convention) with every product and the sum rounded to bf16:
// out = bf16(bf16(x*cos) + bf16(rot(x)*sin)), rot(x)[i] = -x[i+64] (i<64),
// x[i-64] otherwise.
static void bmo_head_norm_rope(const uint16_t *x, const uint16_t *w, float eps,
                               const uint16_t *cosr, const uint16_t *sinr, uint16_t *out) {
    float h[128], n[128];
    for (int i = 0; i < 128; ++i) h[i] = bm_bf16_to_f32(x[i]);
    bmo_rmsnorm_row(h, w, eps, 128, 4, n);
    for (int i = 0; i < 128; ++i) {
        const float rot = i < 64 ? -n[i + 64] : n[i - 64];
        const float a = bm_bf16_rn(n[i] * bm_bf16_to_f32(cosr[i]));
        const float b = bm_bf16_rn(rot * bm_bf16_to_f32(sinr[i]));
        out[i] = bm_f32_to_bf16(a + b);
    }
}

BMO_API void bmo_qknorm_rope_kvappend(const uint16_t *xqkv, const uint16_t *q_w,
                                      const uint16_t *k_w, float eps, const uint16_t *cos_t,
                                      const uint16_t *sin_t, const int64_t *positions, int M,
                                      int H, int Hkv, uint16_t *k_base, uint16_t *v_base,
                                      int kv_rows, int sigma, uint16_t *q_out) {
    const int width = (H + 2 * Hkv) * 128;
    for (int m = 0; m < M; ++m) {
        const uint16_t *row = xqkv + (size_t)m * width;
        const uint16_t *cr = cos_t + (size_t)positions[m] * 128;
        const uint16_t *sr = sin_t + (size_t)positions[m] * 128;
        for (int h = 0; h < H; ++h)
            bmo_head_norm_rope(row + h * 128, q_w, eps, cr, sr, q_out + ((size_t)m * H + h) * 128);
        for (int h = 0; h < Hkv; ++h) {
            uint16_t *kd = k_base + ((size_t)h * kv_rows + sigma + m) * 128;
            uint16_t *vd = v_base + ((size_t)h * kv_rows + sigma + m) * 128;
            bmo_head_norm_rope(row + (H + h) * 128, k_w, eps, cr, sr, kd);
            memcpy(vd, row + (size_t)(H + Hkv + h) * 128, 256);
        }
    }
}

// ---------------------------------------------------------------------------
// Block-verify attention over the shared KV buffer
// ---------------------------------------------------------------------------
// q bf16 [M, H, 128]; k_base, v_base bf16 [Hkv, kv_rows, 128]; the M rows this
// replay appended sit at [sigma, sigma+M).  out bf16 [M, H*128].
//
// Keys are visited in super-chunks of BM_ATTN_SUPER (128) rows, each cut into sub-chunks of
// BM_ATTN_CHUNK (32): history super-chunks [128J, 128J+128) clipped to cache_len, then one
// super-chunk holding the M appended rows.  Three levels, every one in a fixed order:
//   level 0, per sub-chunk and query vector:
//     score   dot over the 128 dims with fma in ascending d, times 1/sqrt(128)
//     m_c     max of the visible scores (-inf when none is visible)
//     p       bm_expf(score - m_c), 0 for hidden keys
//     l_c     sum of p over the sub-chunk's 32 positions in butterfly order
//     o_c[d]  fma(bf16(p_k), v[k][d], o_c[d]) over visible k ascending
//   level 1, per super-chunk: M_J = max_c m_c; w_c = bm_expf(m_c - M_J) (0 when m_c = -inf);
//     L_J = fma(l_c, w_c, L_J) and O_J[d] = fma(o_c[d], w_c, O_J[d]) over its four sub-chunks
//     ascending (a sub-chunk without rows contributes l = 0, o = 0, w = 0)
//   level 2: m = max_J M_J; W_J = bm_expf(M_J - m) (0 when M_J = -inf); l = fma(L_J, W_J, l),
//     o[d] = fma(O_J[d], W_J, o[d]) over the super-chunks ascending, the appended rows last.
// out = bf16(o / l).
BMO_API void bmo_attention(const uint16_t *q, const uint16_t *k_base, const uint16_t *v_base,
                           int M, int H, int Hkv, int kv_rows, int sigma, int cache_len,
                           int n_pend, int P, int role, uint16_t *out) {
    const int G = H / Hkv;
    const float scale = 0.08838834764831845f;   // 1/sqrt(128)
    const int SUB = BM_ATTN_SUPER / BM_ATTN_CHUNK;
    const int n_hs = (cache_len + BM_ATTN_SUPER - 1) / BM_ATTN_SUPER;
    const int n_super = n_hs + 1;
#pragma omp parallel for collapse(2) schedule(static)
    for (int m = 0; m < M; ++m) {
        for (int h = 0; h < H; ++h) {
            const int hk = h / G;
            const uint16_t *kb = k_base + (size_t)hk * kv_rows * 128;
            const uint16_t *vb = v_base + (size_t)hk * kv_rows * 128;
            float qf[128];
            for (int d = 0; d < 128; ++d) qf[d] = bm_bf16_to_f32(q[((size_t)m * H + h) * 128 + d]);
            float *SM = (float *)malloc(sizeof(float) * n_super * 130);   // M_J, L_J, O_J[128]
            float *SL = SM + n_super;
            float *SO = SL + n_super;
            float gmax = -INFINITY;
            for (int J = 0; J < n_super; ++J) {
                const int key0 = J < n_hs ? J * BM_ATTN_SUPER : sigma;
                const int nkeys = J < n_hs ? (cache_len - key0 < BM_ATTN_SUPER ? cache_len - key0 : BM_ATTN_SUPER) : M;
                float cm[8], cl[8], co[8][128];
                for (int c = 0; c < SUB; ++c) {
                    const int c0 = key0 + c * BM_ATTN_CHUNK;
                    int cn = nkeys - c * BM_ATTN_CHUNK;
                    cn = cn > BM_ATTN_CHUNK ? BM_ATTN_CHUNK : cn;
                    float sc[BM_ATTN_CHUNK];
                    int vis[BM_ATTN_CHUNK];
                    float mc = -INFINITY;
                    for (int k = 0; k < cn; ++k) {
                        vis[k] = bm_visible(role, m, c0 + k, sigma, cache_len, n_pend, P);
                        if (!vis[k]) continue;
                        const uint16_t *kr = kb + (size_t)(c0 + k) * 128;
                        float acc = 0.0f;
                        for (int d = 0; d < 128; ++d) acc = fmaf(qf[d], bm_bf16_to_f32(kr[d]), acc);
                        sc[k] = acc * scale;
                        mc = sc[k] > mc ? sc[k] : mc;
                    }
                    cm[c] = mc;
                    for (int d = 0; d < 128; ++d) co[c][d] = 0.0f;
                    float lane[32];
                    for (int k = 0; k < 32; ++k) lane[k] = 0.0f;
                    for (int k = 0; k < cn; ++k) {
                        if (!vis[k]) continue;
                        const float p = bm_expf(sc[k] - mc);
                        lane[k] = p;
                        const float pb = bm_bf16_rn(p);
                        const uint16_t *vr = vb + (size_t)(c0 + k) * 128;
                        for (int d = 0; d < 128; ++d) co[c][d] = fmaf(pb, bm_bf16_to_f32(vr[d]), co[c][d]);
                    }
                    cl[c] = bmo_butterfly32(lane);
                }
                float MJ = -INFINITY;
                for (int c = 0; c < SUB; ++c) MJ = cm[c] > MJ ? cm[c] : MJ;
                float LJ = 0.0f;
                float *OJ = SO + (size_t)J * 128;
                for (int d = 0; d < 128; ++d) OJ[d] = 0.0f;
                for (int c = 0; c < SUB; ++c) {
                    const float w = cm[c] > -INFINITY ? bm_expf(cm[c] - MJ) : 0.0f;
                    LJ = fmaf(cl[c], w, LJ);
                    for (int d = 0; d < 128; ++d) OJ[d] = fmaf(co[c][d], w, OJ[d]);
                }
                SM[J] = MJ;
                SL[J] = LJ;
                gmax = MJ > gmax ? MJ : gmax;
            }
            float l = 0.0f, o[128];
            for (int d = 0; d < 128; ++d) o[d] = 0.0f;
            for (int J = 0; J < n_super; ++J) {
                const float w = SM[J] > -INFINITY ? bm_expf(SM[J] - gmax) : 0.0f;
                l = fmaf(SL[J], w, l);
                const float *OJ = SO + (size_t)J * 128;
                for (int d = 0; d < 128; ++d) o[d] = fmaf(OJ[d], w, o[d]);
            }
            for (int d = 0; d < 128; ++d)
                out[(size_t)m * H * 128 + h * 128 + d] = bm_f32_to_bf16(o[d] / l);
            free(SM);
        }
    }
}

// Visibility predicate exposed for the mask tests.
BMO_API int bmo_visible(int role, int r, int c, int sigma, int cache_len, int n_pend, int P) {
    return bm_visible(role, r, c, sigma, cache_len, n_pend, P);
}

// ---------------------------------------------------------------------------
// Logit reductions and acceptance
// ---------------------------------------------------------------------------
// logits fp32 [rows, vocab] -> idx int64 [rows]: first index of the row maximum.
BMO_API void bmo_argmax_rows(const float *logits, int rows, int vocab, int64_t *idx) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const float *x = logits + (size_t)r * vocab;
        float best = x[0];
        int64_t bi = 0;
        for (int v = 1; v < vocab; ++v)   // NaN counts as the maximum, lowest index wins (bm_argmax_better)
            if (bm_argmax_better(x[v], v, best, (int)bi)) { best = x[v]; bi = v; }
        idx[r] = bi;
    }
}

// Confidence chain of one draft block (fast_generate.py:111-130).
// conf[r] = exp(max - logsumexp), logsumexp = max + log(sum exp(x - max)).
// The sum runs over 256-element chunks: lane t of a chunk adds its 8
// consecutive terms in ascending order, lanes are combined by the butterfly,
// chunk sums are added in ascending order (a short tail chunk is padded with
// zeros).  iter_accept = 1 + number of leading rows r >= 1 with conf > tau.
BMO_API int bmo_draft_chain(const float *logits, int D, int vocab, float tau, int64_t *idx,
                            float *conf_out) {
    bmo_argmax_rows(logits, D, vocab, idx);
    int chain = 0, open = 1;
    for (int r = 0; r < D; ++r) {
        const float *x = logits + (size_t)r * vocab;
        const float mx = x[idx[r]];
        float total = 0.0f;
        for (int c0 = 0; c0 < vocab; c0 += 256) {
            float lane[32];
            for (int t = 0; t < 32; ++t) {
                float acc = 0.0f;
                for (int e = 0; e < 8; ++e) {
                    const int v = c0 + t * 8 + e;
                    if (v < vocab) acc += bm_expf(x[v] - mx);
                }
                lane[t] = acc;
            }
            total += bmo_butterfly32(lane);
        }
        const float lse = mx + bm_logf(total);
        const float conf = bm_expf(mx - lse);
        if (conf_out) conf_out[r] = conf;
        if (r >= 1) {
            if (open && conf > tau) chain += 1; else open = 0;
        }
    }
    return 1 + chain;
}

// Longest prefix of equal token ids (fast_generate.py:133-146).
BMO_API int bmo_verify_accept(const int64_t *draft, const int64_t *verify, int D) {
    int n = 0;
    while (n < D && draft[n] == verify[n]) ++n;
    return n;
}

// Embedding gather: table bf16 [vocab, dim], tokens int64 [M] -> out bf16 [M, dim]
BMO_API void bmo_embed(const uint16_t *table, const int64_t *tokens, int M, int dim,
                       uint16_t *out) {
    for (int m = 0; m < M; ++m)
        memcpy(out + (size_t)m * dim, table + (size_t)tokens[m] * dim, (size_t)dim * 2);
}

// Scalar helpers exposed so the tests can pin bm_math.h against libm.
BMO_API float bmo_expf(float x) { return bm_expf(x); }
BMO_API float bmo_logf(float x) { return bm_logf(x); }
BMO_API uint16_t bmo_f32_to_bf16(float x) { return bm_f32_to_bf16(x); }
