// Scalar arithmetic shared by the CUDA kernels and the CPU oracle.
//
// Every function here is plain IEEE-754 binary32 arithmetic built from
// add/mul/fma/div/sqrt and integer bit operations, so a CPU build (gcc with
// -ffp-contract=off) and a device build (nvcc with -fmad=false, no fast-math)
// produce bit-identical results.  Nothing in this header calls libm's
// transcendental functions: expf/logf differ between glibc and CUDA by an ulp
// or two, and a one-ulp difference before a bf16 rounding is enough to flip a
// greedy token several layers later.
//
// Rounding points follow the eager tensor expressions of the reference
// (src/bonsai_sft/gpu/model.py:307-336, 388-436, 632-636, 1059-1061): values
// are bf16 in memory, arithmetic is fp32, and each `.to(bfloat16)` in the
// reference is one bm_bf16_rn() here.
#ifndef BM_MATH_H_
#define BM_MATH_H_

#include <stdint.h>
#include <string.h>
#include <math.h>

#if defined(__CUDACC__)
#define BM_HD __host__ __device__ __forceinline__
#else
#define BM_HD static inline
#endif

#define BM_GROUP 128          /* K elements that share one weight scale      */
#define BM_SLOTS 16           /* partial sums per output before the tree     */
#define BM_ATTN_CHUNK 32      /* keys per attention sub-chunk (one warp pass) */
#define BM_ATTN_SUPER 128     /* keys per attention super-chunk (one partial) */
#define BM_MAX_W 32           /* widest token block accepted by any kernel   */

BM_HD uint32_t bm_f32_bits(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}

BM_HD float bm_bits_f32(uint32_t u) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f; memcpy(&f, &u, 4); return f;
#endif
}

// bf16 <-> fp32.  Widening is exact; narrowing is round-to-nearest-even, the
// rounding torch's `.to(torch.bfloat16)` performs.
BM_HD float bm_bf16_to_f32(uint16_t h) { return bm_bits_f32(((uint32_t)h) << 16); }

BM_HD uint16_t bm_f32_to_bf16(float f) {
    uint32_t u = bm_f32_bits(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);  // NaN stays NaN
#if defined(__CUDA_ARCH__)
    // the hardware conversion rounds to nearest even exactly as the integer form below does
    // (denormals and the overflow to infinity included); one instruction instead of five
    unsigned short r;
    asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
    return r;
#else
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
#endif
}

// fp32 value after one bf16 rounding.
BM_HD float bm_bf16_rn(float f) { return bm_bf16_to_f32(bm_f32_to_bf16(f)); }

// e^x.  Range reduction x = n*ln2 + r with a split ln2, degree-6 polynomial
// for e^r on |r| <= ln2/2, exponent inserted with integer arithmetic.
// Below -87 the result is 0, above 88 it is +inf (callers: softmax weights with
// x <= 0, SiLU with any x, confidence with x <= 0).
BM_HD float bm_expf(float x) {
    if (!(x >= -87.0f)) return (x != x) ? x : 0.0f;
    if (x > 88.0f) return bm_bits_f32(0x7f800000u);
    const float t = x * 1.44269504088896341f;
    const float n = rintf(t);
    float r = fmaf(n, -0.693145751953125f, x);
    r = fmaf(n, -1.42860682030941723e-6f, r);
    float p = 1.3888889225e-3f;                  // 1/720
    p = fmaf(p, r, 8.3333337680e-3f);            // 1/120
    p = fmaf(p, r, 4.1666667908e-2f);            // 1/24
    p = fmaf(p, r, 1.6666667163e-1f);            // 1/6
    p = fmaf(p, r, 0.5f);
    p = fmaf(p, r, 1.0f);
    p = fmaf(p, r, 1.0f);
    const int ni = (int)n;                       // in [-126, 127]
    // Two-step scaling keeps ni == 128 (x just under 88.0) finite-correct.
    const int half = ni >> 1;
    const float s1 = bm_bits_f32((uint32_t)(half + 127) << 23);
    const float s2 = bm_bits_f32((uint32_t)(ni - half + 127) << 23);
    return (p * s1) * s2;
}

// Natural logarithm for finite x > 0 (normal range).  Mantissa folded to
// [sqrt(1/2), sqrt(2)), degree-8 polynomial in f = m - 1, exponent added with
// a split ln2.  Used for logsumexp in the draft confidence chain.
BM_HD float bm_logf(float x) {
    uint32_t u = bm_f32_bits(x);
    int e = (int)(u >> 23) - 127;
    u = (u & 0x007fffffu) | 0x3f800000u;
    float m = bm_bits_f32(u);                    // [1, 2)
    if (m > 1.41421356237f) { m = m * 0.5f; e += 1; }
    const float f = m - 1.0f;
    const float z = f * f;
    float p = 7.0376836292e-2f;
    p = fmaf(p, f, -1.1514610310e-1f);
    p = fmaf(p, f, 1.1676998740e-1f);
    p = fmaf(p, f, -1.2420140846e-1f);
    p = fmaf(p, f, 1.4249322787e-1f);
    p = fmaf(p, f, -1.6668057665e-1f);
    p = fmaf(p, f, 2.0000714765e-1f);
    p = fmaf(p, f, -2.4999993993e-1f);
    p = fmaf(p, f, 3.3333331174e-1f);
    float y = (f * z) * p;
    const float fe = (float)e;
    y = fmaf(fe, -2.12194440e-4f, y);
    y = fmaf(-0.5f, z, y);
    float r = f + y;
    r = fmaf(fe, 0.693359375f, r);
    return r;
}

// 1/sqrt(v) as torch.rsqrt computes it on CPU tensors: a correctly rounded
// square root followed by a correctly rounded reciprocal.
BM_HD float bm_rsqrtf(float v) { return 1.0f / sqrtf(v); }

// Per-token symmetric INT8 quantisation of one value (model.py:632-636):
// round-half-to-even of x*s, clamped to [-128, 127].
BM_HD int bm_quant_i8(float x, float s) {
    float r = rintf(x * s);
    r = r < -128.0f ? -128.0f : r;
    r = r > 127.0f ? 127.0f : r;
    return (int)r;
}

// Activation multiplier s = 127 / max(absmax, 1e-5) (model.py:635).  torch evaluates
// `scalar / tensor` as reciprocal(tensor) * scalar, i.e. with two roundings; the fixture
// recorded from the reference pins that form (a single correctly rounded division differs
// in the last bit for some absmax values and moves INT8 codes that sit on a .5 boundary).
BM_HD float bm_act_scale(float absmax) {
    return (1.0f / (absmax < 1e-5f ? 1e-5f : absmax)) * 127.0f;
}

// SiLU on a bf16 value, result rounded to bf16, as F.silu does for a bf16
// tensor: x / (1 + e^-x) in fp32.
BM_HD float bm_silu_bf16(float x) {
    return bm_bf16_rn(x / (1.0f + bm_expf(-x)));
}

// Row argmax comparison: does candidate (f at index v) beat the current best (best at index bi)?
// A NaN counts as the largest value and the lowest index wins among equals, which is what
// torch.argmax returns (fast_generate.py:786, 809, 1079 call it on the logit rows).  With this rule
// a row always yields an index inside the row, whatever it holds, so an id that stays on the device
// and feeds the next replay's embedding gather can never point outside the table.
BM_HD int bm_argmax_better(float f, int v, float best, int bi) {
    const int fn = f != f, bn = best != best;
    if (fn != bn) return fn;
    return f > best || ((fn || f == best) && v < bi);
}

// Position of element k (0..15 within a 16-element run) after the 4x4 byte
// transpose the GEMV kernels apply to activations so that one dp4a / MMA
// register lines up with the codes `(word >> 2i) & 0x03030303` extracts:
// permuted[4*t + e] = natural[4*e + t].
BM_HD int bm_perm16(int k) { return ((k & 3) << 2) | (k >> 2); }


// Attention visibility for the three replay roles.  Restates the additive
// masks the reference rebuilds on the host before every replay
// (src/bonsai_sft/gpu/fast_runtime.py:345-372 draft template, :391-421 draft
// history patch, :423-465 verify / AR) as a predicate the kernels evaluate
// from (role, cache_len, n_pend) instead of reading a [M, sigma+M] tensor.
//   r        query row, 0..M-1
//   c        key row of the shared buffer: history rows are [0, sigma),
//            the rows written by this replay are [sigma, sigma+M)
//   P        M - D, the number of pending/PAD rows ahead of the draft block
//   n_pend   pending rows (clamped to [0, P] as prepare_step does)
#define BM_ROLE_DRAFT 0
#define BM_ROLE_VERIFY 1
#define BM_ROLE_AR 2
#ifndef BM_PDL_STABLE_STATE
#define BM_PDL_STABLE_STATE 2      /* pdl bit: step record and history rows predate the launch chain */
#endif

BM_HD int bm_visible(int role, int r, int c, int sigma, int cache_len, int n_pend, int P) {
    if (role == BM_ROLE_DRAFT) {
        if (n_pend < 0) n_pend = 0;
        if (n_pend > P) n_pend = P;
        const int is_pad = (r >= n_pend && r < P);
        if (c < sigma) {
            int vis = (c < cache_len) || (is_pad && c == 0);
            if (cache_len > 0 && n_pend == 0 && c == cache_len - 1) vis = 0;
            return vis;
        }
        const int w = c - sigma;
        if (r < n_pend) return w <= r;
        if (is_pad) return 0;
        return (w >= P && w <= r) || (w < n_pend - 1);
    }
    if (c < sigma) {
        if (c >= cache_len) return 0;
        if (role == BM_ROLE_VERIFY && c == cache_len - 1) return 0;
        return 1;
    }
    return (c - sigma) <= r;
}

#endif  // BM_MATH_H_
