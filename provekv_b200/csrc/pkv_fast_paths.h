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
#else
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
/* Absolute floor covering products that underflow to subnormals. */
#define PKV_QJL_ABS_BOUND 1.0e-35f

#endif /* PKV_FAST_PATHS_H */
