/*
 * pkv_portable_math.h -- the three transcendental functions of the turbo-quant
 * path, written out as a fixed sequence of IEEE-754 binary64 operations so the
 * same source gives the same bits on the host (gcc, -ffp-contract=off) and on
 * the device (nvcc, explicit round-to-nearest intrinsics, never contracted).
 *
 * Why this exists.  The reference reaches atan2f / logf / expf through Rust's
 * std, i.e. through whatever libm the platform ships
 * (turbo-quant/src/polar.rs:413-421 `b.atan2(a)`, turbo-quant/src/radius.rs:61
 * `.ln()`, turbo-quant/src/radius.rs:143 `.exp()`).  Those results are not
 * correctly rounded and differ between libm versions, so "the reference's
 * bits" are only defined per platform.  A GPU cannot call the host libm.  The
 * functions below evaluate each quantity in binary64 with an error of a few
 * 1e-16 and round once to binary32, which is the correctly rounded binary32
 * result except when the exact value lies within ~1e-9 ulp of a rounding
 * boundary.  They are the *normative* definition for this library: the CUDA
 * kernels and the oracle's "portable" mode both evaluate exactly this code.
 * The oracle's "platform" mode calls the host libm instead, and the test-suite
 * measures how often the two disagree.
 *
 * The algorithms are textbook ones (table + Taylor series for atan, atanh
 * series for log, Taylor series for exp); the constants were produced with
 * mpmath at 200 bits and are written as hexadecimal literals.
 */
#ifndef PKV_PORTABLE_MATH_H
#define PKV_PORTABLE_MATH_H

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define PKV_HD __host__ __device__ __forceinline__
#else
#define PKV_HD static inline
#endif

#if defined(__CUDA_ARCH__)
#define PKV_DADD(a, b) __dadd_rn((a), (b))
#define PKV_DSUB(a, b) __dsub_rn((a), (b))
#define PKV_DMUL(a, b) __dmul_rn((a), (b))
#define PKV_DDIV(a, b) __ddiv_rn((a), (b))
#define PKV_D2F(a) __double2float_rn(a)
#else
/* Host builds must use -ffp-contract=off (the oracle Makefile does). */
#define PKV_DADD(a, b) ((a) + (b))
#define PKV_DSUB(a, b) ((a) - (b))
#define PKV_DMUL(a, b) ((a) * (b))
#define PKV_DDIV(a, b) ((a) / (b))
#define PKV_D2F(a) ((float)(a))
#endif

PKV_HD uint32_t pkv_f32_bits(float x) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(x);
#else
  uint32_t u;
  memcpy(&u, &x, 4);
  return u;
#endif
}
PKV_HD float pkv_f32_from_bits(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float x;
  memcpy(&x, &u, 4);
  return x;
#endif
}
PKV_HD double pkv_f64_from_bits(uint64_t u) {
#if defined(__CUDA_ARCH__)
  return __longlong_as_double((long long)u);
#else
  double x;
  memcpy(&x, &u, 8);
  return x;
#endif
}

/* atan(i/16), i = 0..16, rounded to binary64. */
#define PKV_ATAN_TABLE_INIT                                                   \
  {0x0.0p+0,               0x1.ff55bb72cfdeap-5,  0x1.fd5ba9aac2f6ep-4,       \
   0x1.7b97b4bce5b02p-3,   0x1.f5b75f92c80ddp-3,  0x1.362773707ebccp-2,       \
   0x1.6f61941e4def1p-2,   0x1.a64eec3cc23fdp-2,  0x1.dac670561bb4fp-2,       \
   0x1.0657e94db30d0p-1,   0x1.1e00babdefeb4p-1,  0x1.345f01cce37bbp-1,       \
   0x1.4978fa3269ee1p-1,   0x1.5d58987169b18p-1,  0x1.700a7c5784634p-1,       \
   0x1.819d0b7158a4dp-1,   0x1.921fb54442d18p-1}

#if defined(__CUDACC__)
__device__ __constant__ static const double pkv_atan_tab_dev[17] = PKV_ATAN_TABLE_INIT;
#endif
static const double pkv_atan_tab_host[17] = PKV_ATAN_TABLE_INIT;

#define PKV_PI_HI 0x1.921fb54442d18p+1
#define PKV_PI_LO 0x1.1a62633145c07p-53
#define PKV_PIO2_HI 0x1.921fb54442d18p+0
#define PKV_PIO2_LO 0x1.1a62633145c07p-54
#define PKV_LN2_HI 0x1.62e42fee00000p-1 /* low 21 bits zero: k*LN2_HI exact */
#define PKV_LN2_LO 0x1.a39ef35793c76p-33
#define PKV_INV_LN2 0x1.71547652b82fep+0
#define PKV_SQRT2 0x1.6a09e667f3bcdp+0

/* atan(t) for t in [0, 1]:  t = c + (t - c), c = i/16,
 * atan(t) = atan(c) + atan(u), u = (t - c) / (1 + t c), |u| <= 1/32,
 * atan(u) by its Taylor series through u^13 (next term < 2^-78). */
PKV_HD double pkv_atan_unit(double t) {
  int i = (int)PKV_DADD(PKV_DMUL(t, 16.0), 0.5);
  double c = PKV_DMUL((double)i, 0.0625);
  double u = PKV_DDIV(PKV_DSUB(t, c), PKV_DADD(1.0, PKV_DMUL(t, c)));
  double w = PKV_DMUL(u, u);
  double p = 0x1.3b13b13b13b14p-4; /* 1/13 */
  p = PKV_DSUB(0x1.745d1745d1746p-4, PKV_DMUL(w, p)); /* 1/11 */
  p = PKV_DSUB(0x1.c71c71c71c71cp-4, PKV_DMUL(w, p)); /* 1/9 */
  p = PKV_DSUB(0x1.2492492492492p-3, PKV_DMUL(w, p)); /* 1/7 */
  p = PKV_DSUB(0x1.999999999999ap-3, PKV_DMUL(w, p)); /* 1/5 */
  p = PKV_DSUB(0x1.5555555555555p-2, PKV_DMUL(w, p)); /* 1/3 */
  p = PKV_DSUB(1.0, PKV_DMUL(w, p));
#if defined(__CUDA_ARCH__)
  double a = pkv_atan_tab_dev[i];
#else
  double a = pkv_atan_tab_host[i];
#endif
  return PKV_DADD(a, PKV_DMUL(u, p));
}

/* atan2(y, x) in binary64 for finite binary32 arguments, with the signed-zero
 * cases of C Annex F (atan2(+-0, +0) = +-0, atan2(+-0, -0) = +-pi, ...). */
PKV_HD double pkv_atan2_f(float yf, float xf) {
  uint32_t yb = pkv_f32_bits(yf), xb = pkv_f32_bits(xf);
  double ay = (double)pkv_f32_from_bits(yb & 0x7fffffffu);
  double ax = (double)pkv_f32_from_bits(xb & 0x7fffffffu);
  double a;
  if (ax == 0.0 && ay == 0.0) {
    a = 0.0;
  } else if (ay <= ax) {
    a = pkv_atan_unit(PKV_DDIV(ay, ax));
  } else {
    a = PKV_DADD(PKV_DSUB(PKV_PIO2_HI, pkv_atan_unit(PKV_DDIV(ax, ay))), PKV_PIO2_LO);
  }
  if (xb >> 31) a = PKV_DADD(PKV_DSUB(PKV_PI_HI, a), PKV_PI_LO);
  if (yb >> 31) a = -a;
  return a;
}

/* binary32 atan2: one rounding of the binary64 value above. */
PKV_HD float pkv_atan2f_portable(float y, float x) { return PKV_D2F(pkv_atan2_f(y, x)); }

/* log(x) in binary64 for a positive *normal* binary32 x.
 * x = 2^e m, m in [sqrt(1/2), sqrt(2));  log m = 2 atanh(s), s = (m-1)/(m+1),
 * |s| <= 0.1716, series through s^23 (next term < 2^-66 relative). */
PKV_HD double pkv_log_f(float xf) {
  uint32_t b = pkv_f32_bits(xf);
  int e = (int)(b >> 23) - 127;
  double m = PKV_DADD(1.0, PKV_DMUL((double)(b & 0x7fffffu), 0x1.0p-23));
  if (m > PKV_SQRT2) {
    m = PKV_DMUL(m, 0.5);
    e += 1;
  }
  double s = PKV_DDIV(PKV_DSUB(m, 1.0), PKV_DADD(m, 1.0));
  double w = PKV_DMUL(s, s);
  double q = 0x1.642c8590b2164p-5;                       /* 1/23 */
  q = PKV_DADD(0x1.8618618618618p-5, PKV_DMUL(w, q));    /* 1/21 */
  q = PKV_DADD(0x1.af286bca1af28p-5, PKV_DMUL(w, q));    /* 1/19 */
  q = PKV_DADD(0x1.e1e1e1e1e1e1ep-5, PKV_DMUL(w, q));    /* 1/17 */
  q = PKV_DADD(0x1.1111111111111p-4, PKV_DMUL(w, q));    /* 1/15 */
  q = PKV_DADD(0x1.3b13b13b13b14p-4, PKV_DMUL(w, q));    /* 1/13 */
  q = PKV_DADD(0x1.745d1745d1746p-4, PKV_DMUL(w, q));    /* 1/11 */
  q = PKV_DADD(0x1.c71c71c71c71cp-4, PKV_DMUL(w, q));    /* 1/9 */
  q = PKV_DADD(0x1.2492492492492p-3, PKV_DMUL(w, q));    /* 1/7 */
  q = PKV_DADD(0x1.999999999999ap-3, PKV_DMUL(w, q));    /* 1/5 */
  q = PKV_DADD(0x1.5555555555555p-2, PKV_DMUL(w, q));    /* 1/3 */
  q = PKV_DADD(1.0, PKV_DMUL(w, q));
  double logm = PKV_DMUL(PKV_DMUL(2.0, s), q);
  double ed = (double)e;
  return PKV_DADD(PKV_DADD(PKV_DMUL(ed, PKV_LN2_HI), logm), PKV_DMUL(ed, PKV_LN2_LO));
}

PKV_HD float pkv_logf_portable(float x) { return PKV_D2F(pkv_log_f(x)); }

/* expf for a finite binary32 argument: x = k (ln2/32) + r with |r| <= ln2/64, k = 32 e + j,
 * exp(x) = 2^e * 2^(j/32) * exp(r); 2^(j/32) from a 32-entry table, exp(r) by its Taylor series
 * through r^7 (next term < 2^-67) evaluated with fused multiply-adds, one rounding to binary32
 * (which also produces subnormals, 0 and +inf correctly). */
#define PKV_EXP_INV_C 0x1.71547652b82fep+5 /* 32 / ln2 */
#define PKV_EXP_C_HI 0x1.62e42fefa0000p-6  /* ln2 / 32, 38 significant bits: k * C_HI is exact */
#define PKV_EXP_C_LO 0x1.cf79abc9e3b3ap-45
#define PKV_EXP2_TABLE_INIT                                                                          \
  {0x1.0000000000000p+0, 0x1.059b0d3158574p+0, 0x1.0b5586cf9890fp+0, 0x1.11301d0125b51p+0,           \
   0x1.172b83c7d517bp+0, 0x1.1d4873168b9aap+0, 0x1.2387a6e756238p+0, 0x1.29e9df51fdee1p+0,           \
   0x1.306fe0a31b715p+0, 0x1.371a7373aa9cbp+0, 0x1.3dea64c123422p+0, 0x1.44e086061892dp+0,           \
   0x1.4bfdad5362a27p+0, 0x1.5342b569d4f82p+0, 0x1.5ab07dd485429p+0, 0x1.6247eb03a5585p+0,           \
   0x1.6a09e667f3bcdp+0, 0x1.71f75e8ec5f74p+0, 0x1.7a11473eb0187p+0, 0x1.82589994cce13p+0,           \
   0x1.8ace5422aa0dbp+0, 0x1.93737b0cdc5e5p+0, 0x1.9c49182a3f090p+0, 0x1.a5503b23e255dp+0,           \
   0x1.ae89f995ad3adp+0, 0x1.b7f76f2fb5e47p+0, 0x1.c199bdd85529cp+0, 0x1.cb720dcef9069p+0,           \
   0x1.d5818dcfba487p+0, 0x1.dfc97337b9b5fp+0, 0x1.ea4afa2a490dap+0, 0x1.f50765b6e4540p+0}
#if defined(__CUDACC__)
/* in global memory (cached loads): the index differs from thread to thread */
__device__ static const double pkv_exp2_tab_dev[32] = PKV_EXP2_TABLE_INIT;
#endif
static const double pkv_exp2_tab_host[32] = PKV_EXP2_TABLE_INIT;
#if defined(__CUDA_ARCH__)
#define PKV_DFMA(a, b, c) fma((a), (b), (c))
#else
#define PKV_DFMA(a, b, c) __builtin_fma((a), (b), (c))
#endif

PKV_HD float pkv_expf_portable(float xf) {
  double x = (double)xf;
  if (x > 89.0) return pkv_f32_from_bits(0x7f800000u);
  if (x < -150.0) return 0.0f;
#if defined(__CUDA_ARCH__)
  double kd = rint(PKV_DMUL(x, PKV_EXP_INV_C));
#else
  double kd = __builtin_rint(PKV_DMUL(x, PKV_EXP_INV_C));
#endif
  double r = PKV_DFMA(-kd, PKV_EXP_C_LO, PKV_DFMA(-kd, PKV_EXP_C_HI, x));
  double p = 0x1.a01a01a01a01ap-13;               /* 1/7! */
  p = PKV_DFMA(r, p, 0x1.6c16c16c16c17p-10);      /* 1/6! */
  p = PKV_DFMA(r, p, 0x1.1111111111111p-7);       /* 1/5! */
  p = PKV_DFMA(r, p, 0x1.5555555555555p-5);       /* 1/4! */
  p = PKV_DFMA(r, p, 0x1.5555555555555p-3);       /* 1/3! */
  p = PKV_DFMA(r, p, 0x1.0000000000000p-1);       /* 1/2! */
  p = PKV_DFMA(r, p, 1.0);
  p = PKV_DFMA(r, p, 1.0);
  int k = (int)kd;
  int j = k & 31, e = k >> 5; /* k = 32 e + j, 0 <= j < 32 (arithmetic shift) */
#if defined(__CUDA_ARCH__)
  double t = pkv_exp2_tab_dev[j];
#else
  double t = pkv_exp2_tab_host[j];
#endif
  double two_e = pkv_f64_from_bits((uint64_t)(e + 1023) << 52);
  return PKV_D2F(PKV_DMUL(PKV_DMUL(p, t), two_e));
}

#endif /* PKV_PORTABLE_MATH_H */
