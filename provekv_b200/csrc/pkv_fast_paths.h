/*
 * pkv_fast_paths.h -- certified shortcuts of the turbo-quant encoder.
 *
 * Each shortcut computes a *decision* of the reference (an angle bucket, the sign of a
 * QJL projection) by a cheaper route and reports whether that decision is certain, i.e.
 * provably equal to what the exact operation sequence gives.  Undecided cases take the
 * exact path, so the emitted bytes are unchanged.  The functions compile for host and
 * device from the same source; tests/test_fast_paths.py runs them on the CPU against
 * the exact definitions.
 */
#ifndef PKV_FAST_PATHS_H
#define PKV_FAST_PATHS_H

#include "../../include/pkv_portable_math.h"

#if defined(__CUDA_ARCH__)
#define PKV_FMUL(a, b) __fmul_rn((a), (b))
#define PKV_FSUB(a, b) __fsub_rn((a), (b))
#define PKV_FADD(a, b) __fadd_rn((a), (b))
#define PKV_FSQRT(a) __fsqrt_rn(a)
/* An upper bound of the square root for use inside error bounds: the one-instruction approximation
 * (relative error below 2^-22) scaled up by 1e-5; an argument small enough to be flushed to zero
 * contributes less than the constant term of every bound it is used in.  The host build uses the
 * exact root, which is smaller: the device certifies a subset of what the host-side checks cover. */
static __device__ __forceinline__ float pkv_sqrt_upper(float a) {
  float r;
  asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(a));
  return __fmul_rn(r, 1.00001f);
}
#define PKV_FSQRT_UP(a) pkv_sqrt_upper(a)
#else
#define PKV_FSQRT(a) __builtin_sqrtf(a)
#define PKV_FSQRT_UP(a) __builtin_sqrtf(a)
#define PKV_FMUL(a, b) ((a) * (b))
#define PKV_FSUB(a, b) ((a) - (b))
#define PKV_FADD(a, b) ((a) + (b))
#endif

/* Margin of the bucket shortcut, as a fraction of |a| + |b|.  A pair is decided only if
 * it lies more than this far (>= 1e-5 rad) from both rays bounding its sector.  The true
 * decision boundaries (where the binary32 angle crosses a bucket threshold of
 * turbo-quant/src/polar.rs:415-420) are checked at profile creation to lie within 2e-6 rad
 * of the ideal rays, and the rounding of the two cross products is below 2e-7 (|a|+|b|). */
#define PKV_BUCKET_EPS 1.0e-5f

/* Angle bucket of the pair (a, b) for 2^polar_bits levels, polar_bits >= 2, without
 * computing the angle.  The plane is folded into the first quadrant (psi = atan2(|b|,|a|)),
 * the sector j = floor(psi * L / 2pi) is found by bisection over the rays at angles
 * beta_t = 2 pi t / L (ray_cos/ray_sin hold cos/sin beta_t for t = 0..L/4), and the quadrant
 * maps j back to the bucket.  *certain = 0 when (a, b) is too close to a ray (this includes
 * zeros, NaNs, under- and overflow); the caller then evaluates the exact expression. */
PKV_HD uint32_t pkv_fast_bucket(float a, float b, int polar_bits, const float* ray_cos,
                                const float* ray_sin, int* certain) {
  const int Q = 1 << (polar_bits - 2);
  const uint32_t ab = pkv_f32_bits(a), bb = pkv_f32_bits(b);
  const float ax = pkv_f32_from_bits(ab & 0x7fffffffu), ay = pkv_f32_from_bits(bb & 0x7fffffffu);
  int j = 0;
  for (int step = Q >> 1; step >= 1; step >>= 1) {
    const int t = j + step;
    if (PKV_FSUB(PKV_FMUL(ay, ray_cos[t]), PKV_FMUL(ax, ray_sin[t])) >= 0.0f) j = t;
  }
  const float d_lo = PKV_FSUB(PKV_FMUL(ay, ray_cos[j]), PKV_FMUL(ax, ray_sin[j]));
  const float d_hi = PKV_FSUB(PKV_FMUL(ax, ray_sin[j + 1]), PKV_FMUL(ay, ray_cos[j + 1]));
  const float m = d_lo < d_hi ? d_lo : d_hi;
  *certain = m > PKV_FMUL(PKV_BUCKET_EPS, PKV_FADD(ax, ay));
  const int neg_a = (int)(ab >> 31), neg_b = (int)(bb >> 31);
  const int k = neg_b ? (neg_a ? j : 2 * Q - 1 - j) : (neg_a ? 4 * Q - 1 - j : 2 * Q + j);
  return (uint32_t)k;
}

/* The same shortcut for 8 levels (3 bits) with the rays folded into constants: inside the first
 * quadrant the only interior ray is the diagonal, so the sector is `|b| >= |a|`, the distance to
 * the axis rays is min(|a|, |b|) and the distance to the diagonal is ||b| - |a|| / sqrt 2. */
PKV_HD uint32_t pkv_fast_bucket3(float a, float b, int* certain) {
  const uint32_t ab = pkv_f32_bits(a), bb = pkv_f32_bits(b);
  const float ax = pkv_f32_from_bits(ab & 0x7fffffffu), ay = pkv_f32_from_bits(bb & 0x7fffffffu);
  const int j = ay >= ax;
  const float axis = j ? ax : ay;
  const float diff = PKV_FSUB(ay, ax);
  const float diag = PKV_FMUL(pkv_f32_from_bits(pkv_f32_bits(diff) & 0x7fffffffu), 0.70710678118654752f);
  const float m = axis < diag ? axis : diag;
  *certain = m > PKV_FMUL(PKV_BUCKET_EPS, PKV_FADD(ax, ay));
  const int neg_a = (int)(ab >> 31), neg_b = (int)(bb >> 31);
  return (uint32_t)(neg_b ? (neg_a ? j : 3 - j) : (neg_a ? 7 - j : 4 + j));
}

/* 16 levels (4 bits): fold to the first octant (lo = min, hi = max of |a|, |b|); the interior ray
 * is at 22.5 degrees, the octant's upper ray is the diagonal. */
PKV_HD uint32_t pkv_fast_bucket4(float a, float b, int* certain) {
  const uint32_t ab = pkv_f32_bits(a), bb = pkv_f32_bits(b);
  const float ax = pkv_f32_from_bits(ab & 0x7fffffffu), ay = pkv_f32_from_bits(bb & 0x7fffffffu);
  const int swap = ay > ax;
  const float lo = swap ? ax : ay, hi = swap ? ay : ax;
  const float t = PKV_FSUB(PKV_FMUL(lo, 0.92387953251128674f), PKV_FMUL(hi, 0.38268343236508977f));
  const int jp = t >= 0.0f;
  const float d_a = jp ? t : lo;
  const float d_b = jp ? PKV_FMUL(PKV_FSUB(hi, lo), 0.70710678118654752f) : -t;
  const float m = d_a < d_b ? d_a : d_b;
  *certain = m > PKV_FMUL(PKV_BUCKET_EPS, PKV_FADD(ax, ay));
  const int j = swap ? 3 - jp : jp;
  const int neg_a = (int)(ab >> 31), neg_b = (int)(bb >> 31);
  return (uint32_t)(neg_b ? (neg_a ? j : 7 - j) : (neg_a ? 15 - j : 8 + j));
}

/* Dispatch on the width: constant-folded when polar_bits is a compile-time constant. */
PKV_HD uint32_t pkv_fast_bucket_any(float a, float b, int polar_bits, const float* ray_cos,
                                    const float* ray_sin, int* certain) {
  if (polar_bits == 3) return pkv_fast_bucket3(a, b, certain);
  if (polar_bits == 4) return pkv_fast_bucket4(a, b, certain);
  return pkv_fast_bucket(a, b, polar_bits, ray_cos, ray_sin, certain);
}

/* Relative threshold of the QJL sign shortcut: a dot product of n = dim <= 128 terms
 * evaluated in binary32 in any order, fused or not, differs from the exact sum by at most
 * gamma_n * sum|g_j x_j| <= gamma_n |g| |x| (gamma_n = n u / (1 - n u), u = 2^-24).  If the
 * shortcut's |dot| exceeds twice that bound, the reference's sequential unfused sum
 * (turbo-quant/src/qjl.rs:214-217) has the same sign.  The factor below is 2 gamma_129 with
 * 2 % slack for the rounding of the norms themselves. */
#define PKV_QJL_REL_BOUND (2.0f * 129.0f * 5.9604645e-8f * 1.02f / (1.0f - 129.0f * 5.9604645e-8f))
/* First tier of the same test for dots taken on the tensor cores in TF32: each operand keeps 10
 * explicit mantissa bits (relative error below 2^-10, whether the unit truncates or rounds), the
 * products of the shortened operands are exact and are summed in binary32, so the result differs
 * from the exact sum by at most (2^-9 + 2^-20) sum|g_j x_j| plus the summation error (below
 * 2^-17 sum|g_j x_j| for 128 terms).  2.1e-3 leaves 7 % on top of 2^-9 = 1.953e-3.  A dot that fails
 * this test is retaken in binary32 (bound above) before the exact sequence is used. */
#define PKV_QJL_TF32_BOUND 2.1e-3f
/* Absolute floor covering products that underflow to subnormals. */
#define PKV_QJL_ABS_BOUND 1.0e-35f

/* BlockLogU8 radius code (turbo-quant/src/radius.rs:58-77) from an approximate logarithm.
 * The reference takes q = round(255 * clamp((ln r - mn) / span)) in binary32.  With l~ within
 * eps_l of the logarithm the reference uses and k ~ 255 / span, s~ = (l~ - mn) k differs from the
 * reference's 255 * nrm by at most eps_l * k plus the roundings of both chains (three binary32
 * roundings each, together below 1.2e-4 code units), so q is the nearest integer of s~ unless s~
 * lies that close to a half.  eps_l: the fast device logarithm is documented to stay within
 * 2^-21.41 absolute on [0.5, 2] and 3 ulp elsewhere; 5.4e-7 * max(1, |l~|) is 1.5 times that.
 * A span too small for the bound to mean anything (delta >= 1/4) is never certain. */
#define PKV_RADII_LOG_REL 5.4e-7f
#define PKV_RADII_CHAIN_ABS 3.0e-4f
PKV_HD uint32_t pkv_fast_radius_code(float l_approx, float mn, float k, int* certain) {
  float st = PKV_FMUL(PKV_FSUB(l_approx, mn), k);
  const float al = l_approx < 0.0f ? -l_approx : l_approx;
  const float delta = PKV_FADD(PKV_FMUL(PKV_FMUL(PKV_RADII_LOG_REL, al > 1.0f ? al : 1.0f), k), PKV_RADII_CHAIN_ABS);
  st = st < 0.0f ? 0.0f : (st > 255.0f ? 255.0f : st);
  const uint32_t fl = (uint32_t)st; /* st >= 0: truncation is the floor */
  const float fr = PKV_FSUB(st, (float)fl);
  const float d = fr > 0.5f ? PKV_FSUB(fr, 0.5f) : PKV_FSUB(0.5f, fr);
  *certain = d > delta && delta < 0.25f;
  return fl + (fr > 0.5f ? 1u : 0u);
}

/* ------------------------------------------------------------------------------------------
 * fib-quant encoder shortcuts (fib-quant/src/codec.rs:578-729).
 *
 * (1) Normalised element.  The reference takes n = (f32)((f64)x / norm).  With 1/norm held as a
 * pair of binary32 numbers, invh + invl = RN64(1/norm) to 2^-48, the quotient is
 *   x / norm = p + e + x invl (1 + 2^-48),   p = RN(x invh),  e = x invh - p  (one fused operation, exact),
 * so d = RN(x invl + e) puts p + d within 2^-47 |p| of the true quotient.  n is RN(p + d) unless
 * p + d lies that close to a binary32 rounding boundary, where |d| >= 2^-25.5 |p|; the test rounds
 * p + d (1 + 2^-19) and p + d (1 - 2^-19) and accepts when both give the same number (slack
 * 2^-44.5 |p| at a boundary, six times the error).  Exactness of e needs the product free of
 * underflow: the caller guarantees 2^-40 <= norm <= 2^40 and every nonzero |x| >= 2^-60
 * (pkv_fib_fast_norm_ok); everything else takes the division.
 */
#if defined(__CUDA_ARCH__)
#define PKV_FMAF(a, b, c) fmaf((a), (b), (c))
#else
#define PKV_FMAF(a, b, c) __builtin_fmaf((a), (b), (c))
#endif

/* 2 * bits(x) - 1 modulo 2^32: drops the sign, orders by magnitude, and sends both zeros to the top,
 * so an unsigned minimum over a vector is its smallest nonzero magnitude. */
PKV_HD uint32_t pkv_fib_mag_key(float x) { return 2u * pkv_f32_bits(x) - 1u; }

/* May the pair form be used for a vector with this norm and this minimum of pkv_fib_mag_key? */
PKV_HD int pkv_fib_fast_norm_ok(double norm, uint32_t min_mag_key) {
  return norm >= 0x1p-40 && norm <= 0x1p40 && min_mag_key >= 2u * 0x21800000u - 1u; /* 2^-60 */
}

/* Normalised element by the pair form; *unsure collects a nonzero word when the result is not
 * certain (the caller then divides). */
PKV_HD float pkv_fib_norm_quotient(float x, float invh, float invl, uint32_t* unsure) {
  const float p = PKV_FMUL(x, invh);
  const float e = PKV_FMAF(x, invh, -p);
  const float d = PKV_FMAF(x, invl, e);
  const float r1 = PKV_FMAF(d, 1.0f + 0x1p-19f, p);
  const float r2 = PKV_FMAF(d, 1.0f - 0x1p-19f, p);
  *unsure |= pkv_f32_bits(r1) ^ pkv_f32_bits(r2);
  return r1;
}

/* (2) Rotated value.  y~ = sum_j M32[r][j] n_j accumulated in binary32 with fused multiply-adds
 * (j ascending, D terms) differs from the reference's y = (f32) sum_j M[r][j] n_j (binary64) by at most
 *   |M32 - M| |n| + gamma_D |M32| |n| + u |y|  <=  (1 + (D + 1) + 1) u * |M_r|_2 |n|_2,  u = 2^-24,
 * and the rows of an orthogonal M and the normalised n have 2-norm 1 (to 1e-7):
 * 4.0e-6 for D = 64, 7.9e-6 for D = 128. */
#define PKV_FIB_ROT_ERR 4.0e-6f
#define PKV_FIB_ROT_ERR_D(D) ((float)((D) + 3) * 5.97e-8f)

/* (3) Nearest codeword of a 4-block.  Scores F_c = |c|^2/2 - s.c (so |s - c|^2 = 2 F_c + |s|^2) are
 * evaluated with fused multiply-adds; the codeword index rides in the 5 low significand bits of
 * the score, so best and second-best come from three min/max operations per codeword.  With
 * |s~ - s|_2 <= 2 PKV_FIB_ROT_ERR the reference's rounded distances satisfy
 *   | d_c - (2 F_c + |s~|^2) | <= 4 eta sqrt(D_c) + 4 eta^2 + 4 u D_c + e_F,   eta = PKV_FIB_ROT_ERR,
 * with D_c = |s~ - c|^2 and e_F <= 2^-17 |F_c| (the index bits) + 4 u A_c (the four fused roundings, each
 * at most u times a partial sum no larger than A_c = |c|^2 / 2 + |s~| |c|; when |c|^2 is close to 2 s.c the
 * score itself is small and a bound relative to |F_c| alone would not cover them).  The encoders pass
 * score_abs = 4 u (max |c|^2 / 2 + 1.001 max |c|) for blocks of normalised vectors (pkv_fib_score_abs);
 * the stand-alone lookup forms it from the block's own norm.  If the gap between best and second best
 * exceeds the two bounds, the reference's strict-less-than scan (gpu-backend/src/simd_nearest.rs:72-79)
 * selects the same codeword in either summation order. */
/* Score of codeword c (c0..c3, half squared norm hn) for the block s, index in the low bits. */
PKV_HD float pkv_fib_key(float s0, float s1, float s2, float s3, float c0, float c1, float c2,
                         float c3, float hn, uint32_t c) {
  float f = PKV_FMAF(-s0, c0, hn);
  f = PKV_FMAF(-s1, c1, f);
  f = PKV_FMAF(-s2, c2, f);
  f = PKV_FMAF(-s3, c3, f);
  return pkv_f32_from_bits((pkv_f32_bits(f) & ~31u) | c);
}

/* Keep the two smallest keys seen so far. */
PKV_HD void pkv_fib_top2(float* best, float* second, float key) {
#if defined(__CUDA_ARCH__)
  const float hi = fmaxf(*best, key);  // three min/max instructions, no predicates
  *best = fminf(*best, key);
  *second = fminf(*second, hi);
#else
  const float lo = key < *best ? key : *best, hi = key < *best ? *best : key;
  *second = hi < *second ? hi : *second;
  *best = lo;
#endif
}

/* The same for two new keys at once: the second smallest of {best, second, a, b} is the smaller of
 * max(best, min(a, b)) and min(second, max(a, b)).  With the three-operand minimum of sm_100 that is
 * five instructions for two keys. */
PKV_HD void pkv_fib_top2_pair(float* best, float* second, float a, float b) {
#if defined(__CUDA_ARCH__)
  const float lo = fminf(a, b), hi = fmaxf(a, b);
  const float t = fmaxf(*best, lo);
  float s;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(s) : "f"(*second), "f"(hi), "f"(t));
  *second = s;
  *best = fminf(*best, lo);
#else
  pkv_fib_top2(best, second, a);
  pkv_fib_top2(best, second, b);
#endif
}

/* (2b) The same rotated value from the tensor cores.  n and M32 are each split into a part with
 * 11 significant bits (what a TF32 operand keeps) and the exact remainder, and the unit sums
 * n_hi M_hi + n_hi M_lo + n_lo M_hi with the remainders shortened to 11 bits in turn.  Left out or
 * cut off: n_lo M_lo and the two shortenings, each below 2^-20 sum|n_j M_rj|, together 2.9e-6.
 * The vendor does not specify the rounding inside the accumulation of the 24 partial products;
 * 7e-6 sum|n_j M_rj| is assumed for it (a correctly rounded binary32 accumulation of 24 partial
 * sums stays below 1.4e-6, one that truncates below 2.9e-6).  With |M_r| = |n| = 1:   1.0e-5.
 * (Measured: with the bound set to 2e-6 the encoder still reproduced every byte of 25 M blocks; the largest
 * error of the unit's output against the exact rotation over 60,000 captured vectors was 8.3e-7 at D = 64 and
 * 7.2e-7 at D = 128, pkv_test_capture_rotated.) */
#ifndef PKV_FIB_ROT_ERR_TC
#define PKV_FIB_ROT_ERR_TC 1.0e-5f
#endif
/* D = 128: the same three cut-offs (2.9e-6) and 48 partial products, assumed 1.4e-5 (rounded 2.9e-6,
 * truncating 5.7e-6). */
#ifndef PKV_FIB_ROT_ERR_TC128
#define PKV_FIB_ROT_ERR_TC128 1.7e-5f
#endif
#define PKV_FIB_ROT_ERR_TC_D(D) ((D) == 64 ? PKV_FIB_ROT_ERR_TC : PKV_FIB_ROT_ERR_TC128)

/* Is the best key's codeword provably the reference's choice when the rotated block is known to
 * eta per coordinate?  (bound in the comment above with eta for PKV_FIB_ROT_ERR) */
PKV_HD int pkv_fib_certify_eta(float best, float second, float s0, float s1, float s2, float s3, float eta,
                               float score_abs) {
  const float ss = PKV_FADD(PKV_FADD(PKV_FMUL(s0, s0), PKV_FMUL(s1, s1)),
                            PKV_FADD(PKV_FMUL(s2, s2), PKV_FMUL(s3, s3)));
  const float d1 = PKV_FADD(PKV_FMUL(2.0f, best), ss), d2 = PKV_FADD(PKV_FMUL(2.0f, second), ss);
  const float d2p = d2 > 0.0f ? d2 : 0.0f, d1p = d1 > 0.0f ? d1 : 0.0f;
  const float fb = pkv_f32_from_bits(pkv_f32_bits(best) & 0x7fffffffu);
  const float fs = pkv_f32_from_bits(pkv_f32_bits(second) & 0x7fffffffu);
  const float roots = PKV_FADD(PKV_FSQRT_UP(d1p), PKV_FSQRT_UP(d2p));
  /* two scores, each doubled in its distance: 4 score_abs */
  const float bound = PKV_FADD(
      PKV_FADD(PKV_FADD(PKV_FMUL(4.0f * eta, roots), 8.0f * eta * eta), PKV_FMUL(4.0f, score_abs)),
      PKV_FADD(PKV_FMUL(2.5e-7f, PKV_FADD(d1p, d2p)), PKV_FMUL(1.0e-5f, PKV_FADD(fb, fs))));
  return PKV_FSUB(d2, d1) > PKV_FMUL(1.05f, bound);
}

/* The same test for scores kept with an absolute error of at most e_f each (the biased scores of
 * pkv_fib_search.cuh): the terms for the index bits and the fused roundings give way to 2 e_f per
 * distance. */
PKV_HD int pkv_fib_certify_abs(float f1, float f2, float s0, float s1, float s2, float s3, float eta, float e_f) {
  const float ss = PKV_FADD(PKV_FADD(PKV_FMUL(s0, s0), PKV_FMUL(s1, s1)),
                            PKV_FADD(PKV_FMUL(s2, s2), PKV_FMUL(s3, s3)));
  const float d1 = PKV_FADD(PKV_FMUL(2.0f, f1), ss), d2 = PKV_FADD(PKV_FMUL(2.0f, f2), ss);
  const float d2p = d2 > 0.0f ? d2 : 0.0f, d1p = d1 > 0.0f ? d1 : 0.0f;
  const float roots = PKV_FADD(PKV_FSQRT_UP(d1p), PKV_FSQRT_UP(d2p));
  const float bound = PKV_FADD(PKV_FADD(PKV_FMUL(4.0f * eta, roots), 8.0f * eta * eta),
                               PKV_FADD(PKV_FMUL(2.5e-7f, PKV_FADD(d1p, d2p)), PKV_FMUL(4.2f, e_f)));
  return PKV_FSUB(d2, d1) > PKV_FMUL(1.05f, bound);
}

/* score_abs of the encoders: blocks of a normalised vector have |s| <= 1.001 (rounding of the normalisation,
 * bounded error of an approximate rotation). */
static inline float pkv_fib_score_abs(const float* codebook, int n_codewords) {
  double hmax = 0.0, cmax = 0.0;
  for (int c = 0; c < n_codewords; c++) {
    double s = 0.0;
    for (int j = 0; j < 4; j++) s += (double)codebook[4 * c + j] * (double)codebook[4 * c + j];
    if (0.5 * s > hmax) hmax = 0.5 * s;
    if (__builtin_sqrt(s) > cmax) cmax = __builtin_sqrt(s);
  }
  return (float)(4.0 * 5.9604645e-8 * 1.01 * (hmax + 1.001 * cmax));
}

/* (3b) The same search on biased scores (csrc/pkv_fib_search.cuh gives the layout of the keys).
 * off = 1.5 * 2^k with k the smallest exponent whose binade [2^k, 2^(k+1)) holds off + F for every
 * score F = |c|^2 / 2 - s . c of a block with |s| <= 1.001; e_f = 2.5 ulps of that binade bounds the
 * error of a kept score (the start value and four fused operations, half an ulp each); quick_gap is a
 * gap of the two best scores, in ulps of the binade, above which pkv_fib_certify_abs with this eta holds
 * for every block: it asks for 2 (F2 - F1) > 1.05 (4 eta (sqrt d1 + sqrt d2) + 8 eta^2 + 2.5e-7 (d1 + d2)
 * + 4.2 e_f), squared distances stay below dmax = (1.001 + max |c|)^2, and 0.63 = 0.525 * 1.2 leaves room
 * for the roundings of that test itself.
 * Returns 0 when no binade below 2^99 holds the scores (or the codebook is not finite). */
static inline int pkv_fib_search_bias(const float* codebook, int n_codewords, double eta, float* off, float* e_f,
                                      uint32_t* quick_gap) {
  double hmax = 0.0, cmax = 0.0;
  for (int c = 0; c < n_codewords; c++) {
    double s = 0.0;
    for (int j = 0; j < 4; j++) s += (double)codebook[4 * c + j] * (double)codebook[4 * c + j];
    if (0.5 * s > hmax) hmax = 0.5 * s;
    if (__builtin_sqrt(s) > cmax) cmax = __builtin_sqrt(s);
  }
  const double fmax = 1.001 * (hmax + 1.001 * cmax) + 1.0e-30;
  if (!(fmax < __builtin_ldexp(1.0, 98))) return 0;
  int k = -100;
  while (__builtin_ldexp(1.0, k - 1) < fmax) k++;
  const double ulp_b = __builtin_ldexp(1.0, k - 23), dmax = (1.001 + cmax) * (1.001 + cmax);
  *off = (float)__builtin_ldexp(1.5, k);
  *e_f = (float)(2.5 * ulp_b);
  const double gap = 0.63 * (8.0 * eta * __builtin_sqrt(dmax) + 8.0 * eta * eta + 5.05e-7 * dmax + 10.5 * ulp_b) / ulp_b;
  *quick_gap = gap < 4.0e9 ? (uint32_t)__builtin_ceil(gap) + 1u : 0xffffffffu;
  return 1;
}

/* Key of codeword c (negated coordinates nc0..nc3, start value hn_off = RN(|c|^2 / 2 + off)). */
PKV_HD uint32_t pkv_fib_biased_key(float s0, float s1, float s2, float s3, float nc0, float nc1, float nc2,
                                   float nc3, float hn_off, uint32_t c) {
  float f = PKV_FMAF(s0, nc0, hn_off);
  f = PKV_FMAF(s1, nc1, f);
  f = PKV_FMAF(s2, nc2, f);
  f = PKV_FMAF(s3, nc3, f);
  return pkv_f32_bits(f) * 32u + c;
}

/* The score a key was made from (exact: the biased score and off lie in the same binade). */
PKV_HD float pkv_fib_key_score(uint32_t key, float off) {
  return PKV_FSUB(pkv_f32_from_bits((pkv_f32_bits(off) & 0xf8000000u) | (key >> 5)), off);
}

#endif /* PKV_FAST_PATHS_H */
