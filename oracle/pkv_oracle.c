/*
 * pkv_oracle.c -- CPU restatement of proveKV's KV-cache codec hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA kernels are
 * compared against (tests/, the smoke check and the bench's cpu_baseline leg).
 * Nothing in the shipped library calls, links or loads it.
 *
 * PARITY UNPINNED: the reference is Rust and cannot be built where this was
 * written, and its own tests hold no known-answer vectors for codes, wire
 * bytes or tables.  The restatement is pinned only by the facts the
 * reference's tests do state (byte sizes, header offsets, bit order, tie rule,
 * impulse response, batch == single decode); tests/test_oracle_pins.py checks
 * each of them.
 *
 * Every function cites the reference lines it follows.  Arithmetic contracts:
 * every f32/f64 operation is a separately rounded IEEE operation (build with
 * -ffp-contract=off, no -ffast-math); sums run in the reference's order.
 *
 * libm_mode selects how atan2f / logf / expf are evaluated:
 *   PKVO_LIBM_PLATFORM (0): the host libm, which is what Rust's std calls.
 *   PKVO_LIBM_PORTABLE (1): include/pkv_portable_math.h, the definition the
 *                           GPU kernels implement bit for bit.
 */
#include <float.h>
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "../include/pkv_portable_math.h"
#include "../include/provekv_b200.h"

#define PKVO_LIBM_PLATFORM 0
#define PKVO_LIBM_PORTABLE 1

#define PKVO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------ */
/* small helpers                                                             */
/* ------------------------------------------------------------------------ */

static int is_finite_f32(float x) { return (pkv_f32_bits(x) & 0x7f800000u) != 0x7f800000u; }

/* f32 -> f16 bits, round to nearest even, IEEE (what half::f16::from_f32 does;
 * fib-quant/src/codec.rs:1002). */
static uint16_t f32_to_f16_bits(float f) {
  uint32_t x = pkv_f32_bits(f);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t exp = (x >> 23) & 0xffu;
  uint32_t man = x & 0x7fffffu;
  if (exp == 0xffu) return (uint16_t)(sign | 0x7c00u | (man ? 0x200u | (man >> 13) : 0));
  int32_t e = (int32_t)exp - 127 + 15;
  if (e >= 0x1f) return (uint16_t)(sign | 0x7c00u); /* overflow -> inf */
  if (e <= 0) {
    if (e < -10) return (uint16_t)sign; /* underflow -> 0 */
    man |= 0x800000u;
    uint32_t shift = (uint32_t)(14 - e);
    uint32_t half_man = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_man & 1u))) half_man++;
    return (uint16_t)(sign | half_man);
  }
  uint32_t half = sign | ((uint32_t)e << 10) | (man >> 13);
  uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1u))) half++; /* may carry into exponent / inf */
  return (uint16_t)half;
}

static float f16_bits_to_f32(uint16_t h) {
  uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t out;
  if (exp == 0) {
    if (man == 0) {
      out = sign;
    } else {
      int e = -1;
      do {
        man <<= 1;
        e++;
      } while (!(man & 0x400u));
      man &= 0x3ffu;
      out = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 0x1f) {
    out = sign | 0x7f800000u | (man << 13);
  } else {
    out = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  return pkv_f32_from_bits(out);
}

PKVO_API uint16_t pkvo_f32_to_f16_bits(float f) { return f32_to_f16_bits(f); }
PKVO_API float pkvo_f16_bits_to_f32(uint16_t h) { return f16_bits_to_f32(h); }

/* LSB-first fixed-width packing: value i occupies stream bits [w*i, w*i+w).
 * fib-quant/src/bitpack.rs:4-44, turbo-quant/src/bitpack.rs:21-34,135-143. */
static void pack_bits(const uint32_t* values, int count, int width, uint8_t* out, int out_len) {
  memset(out, 0, (size_t)out_len);
  for (int i = 0; i < count; i++)
    for (int b = 0; b < width; b++)
      if ((values[i] >> b) & 1u) {
        int pos = i * width + b;
        out[pos / 8] |= (uint8_t)(1u << (pos % 8));
      }
}

/* fib-quant/src/bitpack.rs:47-90, turbo-quant/src/bitpack.rs:37-45,88-110.
 * Returns 0 when the padding bits after count*width are not all zero. */
static int unpack_bits(const uint8_t* bytes, int count, int width, uint32_t* values) {
  int total = count * width, nbytes = (total + 7) / 8;
  for (int pos = total; pos < nbytes * 8; pos++)
    if ((bytes[pos / 8] >> (pos % 8)) & 1u) return 0;
  for (int i = 0; i < count; i++) {
    uint32_t v = 0;
    for (int b = 0; b < width; b++) {
      int pos = i * width + b;
      if ((bytes[pos / 8] >> (pos % 8)) & 1u) v |= 1u << b;
    }
    values[i] = v;
  }
  return 1;
}

PKVO_API void pkvo_pack_bits(const uint32_t* values, int count, int width, uint8_t* out) {
  pack_bits(values, count, width, out, (count * width + 7) / 8);
}
PKVO_API int pkvo_unpack_bits(const uint8_t* bytes, int count, int width, uint32_t* values) {
  return unpack_bits(bytes, count, width, values);
}

/* ------------------------------------------------------------------------ */
/* nearest codeword: gpu-backend/src/simd_nearest.rs                         */
/* ------------------------------------------------------------------------ */

/* :24-39, the scalar order ((d0+d1)+d2)+d3 starting from 0.0. */
static int nearest_sequential(const float* s, const float* cb, int n_codewords, int k) {
  int best = 0;
  float best_dist = INFINITY;
  for (int c = 0; c < n_codewords; c++) {
    float dist = 0.0f;
    for (int j = 0; j < k; j++) {
      float delta = s[j] - cb[c * k + j];
      dist += delta * delta;
    }
    if (dist < best_dist) {
      best_dist = dist;
      best = c;
    }
  }
  return best;
}

/* :44-94, the AVX2 k=4 order: delta = codeword - sample, squares, then two
 * hadd steps = (q0+q1)+(q2+q3); codewords visited in ascending order with a
 * strict '<'.  The odd tail codeword (:82-92) uses the scalar order. */
static int nearest_pairwise_k4(const float* s, const float* cb, int n_codewords) {
  int best = 0;
  float best_dist = INFINITY;
  int c = 0;
  for (; c + 2 <= n_codewords; c += 2) {
    for (int h = 0; h < 2; h++) {
      const float* w = cb + (c + h) * 4;
      float d0 = w[0] - s[0], d1 = w[1] - s[1], d2 = w[2] - s[2], d3 = w[3] - s[3];
      float q0 = d0 * d0, q1 = d1 * d1, q2 = d2 * d2, q3 = d3 * d3;
      float dist = (q0 + q1) + (q2 + q3);
      if (dist < best_dist) {
        best_dist = dist;
        best = c + h;
      }
    }
  }
  if (c < n_codewords) {
    float dist = 0.0f;
    for (int j = 0; j < 4; j++) {
      float delta = s[j] - cb[c * 4 + j];
      dist += delta * delta;
    }
    if (dist < best_dist) best = c;
  }
  return best;
}

PKVO_API int pkvo_nearest_codeword(const float* sample, const float* codebook, int n_codewords,
                                   int k, int order) {
  if (k == 4 && order == PKV_ARGMIN_PAIRWISE) return nearest_pairwise_k4(sample, codebook, n_codewords);
  return nearest_sequential(sample, codebook, n_codewords, k);
}

/* ------------------------------------------------------------------------ */
/* fib-quant                                                                  */
/* ------------------------------------------------------------------------ */

static int fib_index_bits(int n_codewords) { /* profile.rs wire_index_bits: ceil(log2 N), >= 1 */
  int b = 1;
  while ((1 << b) < n_codewords) b++;
  return b;
}

PKVO_API int pkvo_fib_record_bytes(int dim, int k, int n_codewords, int norm_format) {
  int blocks = dim / k;
  return (norm_format == PKV_NORM_FP16 ? 2 : 4) + (blocks * fib_index_bits(n_codewords) + 7) / 8;
}

/* gpu-backend/src/fallback.rs:76-88: one LCG step per coordinate, bit 32 of the state picks the sign. */
PKVO_API void pkvo_hadamard_signs(int padded_dim, uint64_t seed, float* signs) {
  uint64_t state = seed;
  for (int i = 0; i < padded_dim; i++) {
    state = state * 6364136223846793005ull + 1442695040888963407ull;
    signs[i] = ((state >> 32) & 1) == 0 ? -1.0f : 1.0f;
  }
}

static int next_pow2(int n) {
  int p = 1;
  while (p < n) p <<= 1;
  return p;
}

/* One vector of hadamard_batch_cpu (gpu-backend/src/fallback.rs:26-59): zero-padded to a power of two,
 * butterflies for step = 1, 2, 4, .., then x sign, then x 1 / sqrt(padded) (f32), truncated back. */
static void pkvo_hadamard_one(float* v, int dim, const float* signs) {
  const int pd = next_pow2(dim);
  float padded[1024];
  for (int i = 0; i < pd; i++) padded[i] = i < dim ? v[i] : 0.0f;
  for (int step = 1; step < pd; step *= 2)
    for (int i = 0; i < pd; i += 2 * step)
      for (int j = 0; j < step; j++) {
        float a = padded[i + j], b = padded[i + j + step];
        padded[i + j] = a + b;
        padded[i + j + step] = a - b;
      }
  for (int i = 0; i < pd; i++) padded[i] *= signs[i];
  const float scale = 1.0f / sqrtf((float)pd);
  for (int i = 0; i < pd; i++) padded[i] *= scale;
  for (int i = 0; i < dim; i++) v[i] = padded[i];
}

/* hadamard_batch_cpu over n vectors in place; dim <= 1024. */
PKVO_API int pkvo_hadamard_batch(float* data, int64_t n, int dim, uint64_t seed) {
  if (dim <= 0 || dim > 1024) return PKV_ERR_INVALID_ARGUMENT;
  float signs[1024];
  pkvo_hadamard_signs(next_pow2(dim), seed, signs);
  for (int64_t v = 0; v < n; v++) pkvo_hadamard_one(data + v * dim, dim, signs);
  return 0;
}

/* codebook_lookup_cpu (gpu-backend/src/fallback.rs:254-305): per k-block the squared distances summed in
 * coordinate order from 0.0, strict less-than scan from index 0 against +inf. */
PKVO_API int pkvo_codebook_lookup(const float* input, const float* codebook, int64_t n, int dim, int k,
                                  int n_codewords, uint32_t* out) {
  if (dim <= 0 || k <= 0 || dim % k || n_codewords < 1) return PKV_ERR_INVALID_ARGUMENT;
  const int blocks = dim / k;
  for (int64_t v = 0; v < n; v++)
    for (int b = 0; b < blocks; b++) {
      const float* s = input + v * dim + (int64_t)b * k;
      uint32_t best_idx = 0;
      float best_dist = INFINITY;
      for (int c = 0; c < n_codewords; c++) {
        float dist = 0.0f;
        for (int j = 0; j < k; j++) {
          const float delta = s[j] - codebook[c * k + j];
          dist += delta * delta;
        }
        if (dist < best_dist) {
          best_dist = dist;
          best_idx = (uint32_t)c;
        }
      }
      out[v * blocks + b] = best_idx;
    }
  return 0;
}

typedef struct {
  const float* x;
  int64_t n;
  int dim, k, n_codewords, norm_format, argmin_order, numerics;
  const double* rot;
  const float* codebook;
  uint8_t* payload;
  const float* wht_signs; /* non-null: the Hadamard rotation of the reference's `gpu` build, +-1 per padded coordinate */
  /* results */
  int pass0_code;
  int64_t pass0_index;
  int pass1_code;
  int64_t pass1_index;
} fib_enc_job;

/* One vector of FibQuantizer::encode_batch (fib-quant/src/codec.rs:578-729).
 * Returns 0, a pass-0 code (non-finite, zero norm) or PKV_VEC_NORM_RANGE. */
static int fib_encode_one(const fib_enc_job* J, int64_t v, int batch_numerics, uint8_t* rec) {
  const int d = J->dim, k = J->k, blocks = d / k;
  const float* x = J->x + v * d;
  /* check_finite, :1059-1064 */
  for (int i = 0; i < d; i++)
    if (!is_finite_f32(x[i])) return PKV_VEC_NONFINITE_INPUT;
  /* l2_norm, :1049-1057: sequential f64 sum of squares, sqrt */
  double acc = 0.0;
  for (int i = 0; i < d; i++) {
    double t = (double)x[i];
    acc += t * t;
  }
  double norm = sqrt(acc);
  if (norm == 0.0) return PKV_VEC_ZERO_NORM; /* :603 */
  double nrm[512];
  float rotated[512];
  if (J->wht_signs) {
    /* codec.rs:607-609 then gpu_backend::hadamard_batch (:619) on the f32 values */
    for (int i = 0; i < d; i++) rotated[i] = (float)((double)x[i] / norm);
    pkvo_hadamard_one(rotated, d, J->wht_signs);
  } else {
  for (int i = 0; i < d; i++) {
    double q = (double)x[i] / norm;
    /* batch path rounds to f32 (:607-609) and widens again (:662); single keeps f64 (:481) */
    nrm[i] = batch_numerics ? (double)(float)q : q;
  }
  /* StoredRotation::apply, fib-quant/src/rotation.rs:104-115: per row a sequential f64 dot */
  for (int r = 0; r < d; r++) {
    const double* row = J->rot + (size_t)r * d;
    double sum = 0.0;
    for (int j = 0; j < d; j++) sum += row[j] * nrm[j];
    rotated[r] = (float)sum; /* :483, :664 */
  }
  }
  uint32_t idx[128];
  for (int b = 0; b < blocks; b++)
    idx[b] = (uint32_t)pkvo_nearest_codeword(rotated + b * k, J->codebook, J->n_codewords, k,
                                             J->argmin_order);
  /* encode_norm, :994-1020 */
  int norm_len;
  if (J->norm_format == PKV_NORM_FP16) {
    uint16_t h = f32_to_f16_bits((float)norm);
    if ((h & 0x7fffu) >= 0x7c00u || (h & 0x7fffu) == 0 || (h & 0x8000u)) return PKV_VEC_NORM_RANGE;
    rec[0] = (uint8_t)(h & 0xff);
    rec[1] = (uint8_t)(h >> 8);
    norm_len = 2;
  } else {
    float nf = (float)norm;
    if (!is_finite_f32(nf) || nf <= 0.0f) return PKV_VEC_NORM_RANGE;
    uint32_t u = pkv_f32_bits(nf);
    rec[0] = (uint8_t)u;
    rec[1] = (uint8_t)(u >> 8);
    rec[2] = (uint8_t)(u >> 16);
    rec[3] = (uint8_t)(u >> 24);
    norm_len = 4;
  }
  int bits = fib_index_bits(J->n_codewords);
  pack_bits(idx, blocks, bits, rec + norm_len, (blocks * bits + 7) / 8);
  return 0;
}

typedef struct {
  void (*fn)(void*, int64_t, int64_t);
  void* arg;
  int64_t lo, hi;
} par_chunk;

static void* par_trampoline(void* p) {
  par_chunk* c = (par_chunk*)p;
  c->fn(c->arg, c->lo, c->hi);
  return NULL;
}

/* Static split of [0, n) over nthreads (the reference uses Rayon over vectors,
 * fib-quant/src/codec.rs:715-722, and over layers, proveKV/src/pool.rs:299-309). */
static void parallel_for(int64_t n, int nthreads, void (*fn)(void*, int64_t, int64_t), void* arg) {
  if (nthreads <= 1 || n < 2 * (int64_t)nthreads) {
    fn(arg, 0, n);
    return;
  }
  pthread_t* th = (pthread_t*)malloc(sizeof(pthread_t) * (size_t)nthreads);
  par_chunk* ch = (par_chunk*)malloc(sizeof(par_chunk) * (size_t)nthreads);
  for (int t = 0; t < nthreads; t++) {
    ch[t].fn = fn;
    ch[t].arg = arg;
    ch[t].lo = n * t / nthreads;
    ch[t].hi = n * (t + 1) / nthreads;
    pthread_create(&th[t], NULL, par_trampoline, &ch[t]);
  }
  for (int t = 0; t < nthreads; t++) pthread_join(th[t], NULL);
  free(th);
  free(ch);
}

typedef struct {
  fib_enc_job* J;
  int rec_bytes, batch_numerics;
  pthread_mutex_t mu;
} fib_enc_ctx;

static void fib_enc_range(void* p, int64_t lo, int64_t hi) {
  fib_enc_ctx* C = (fib_enc_ctx*)p;
  fib_enc_job* J = C->J;
  for (int64_t v = lo; v < hi; v++) {
    int code = fib_encode_one(J, v, C->batch_numerics, J->payload + v * C->rec_bytes);
    if (code) {
      pthread_mutex_lock(&C->mu);
      if (code == PKV_VEC_NORM_RANGE) {
        if (J->pass1_code == 0 || v < J->pass1_index) {
          J->pass1_code = code;
          J->pass1_index = v;
        }
      } else if (J->pass0_code == 0 || v < J->pass0_index) {
        J->pass0_code = code;
        J->pass0_index = v;
      }
      pthread_mutex_unlock(&C->mu);
    }
  }
}

/* FibQuantizer::encode_batch over n contiguous vectors -> n records (no header).
 * The first loop of the reference (:594-610) rejects non-finite / zero-norm
 * vectors before any norm is narrowed (:705), so those errors win over
 * PKV_VEC_NORM_RANGE whatever their index. */
PKVO_API int pkvo_fib_encode_batch(const float* x, int64_t n, int dim, int k, int n_codewords,
                                   int norm_format, int argmin_order, int numerics,
                                   const double* rot, const float* codebook, uint8_t* payload,
                                   int nthreads, int32_t* vec_code, int64_t* vec_index) {
  if (dim <= 0 || dim > 512 || k <= 0 || dim % k || n_codewords < 1 || dim / k > 128)
    return PKV_ERR_INVALID_ARGUMENT;
  if (vec_code) *vec_code = 0;
  if (vec_index) *vec_index = -1;
  if (n == 0) return PKV_ERR_EMPTY_BATCH; /* FibCodeV1::encode_batch, :226 */
  fib_enc_job J = {x, n, dim, k, n_codewords, norm_format, argmin_order, numerics, rot, codebook,
                   payload, NULL, 0, -1, 0, -1};
  fib_enc_ctx C;
  C.J = &J;
  C.rec_bytes = pkvo_fib_record_bytes(dim, k, n_codewords, norm_format);
  C.batch_numerics = numerics == PKV_FIB_NUMERICS_BATCH ||
                     (numerics == PKV_FIB_NUMERICS_AUTO && n >= 4); /* :587 */
  pthread_mutex_init(&C.mu, NULL);
  parallel_for(n, nthreads, fib_enc_range, &C);
  pthread_mutex_destroy(&C.mu);
  int code = J.pass0_code ? J.pass0_code : J.pass1_code;
  int64_t index = J.pass0_code ? J.pass0_index : J.pass1_index;
  if (code) {
    if (vec_code) *vec_code = code;
    if (vec_index) *vec_index = index;
  }
  return code;
}

/* The same batch when the reference is built with its `gpu` feature and the batch is large enough
 * (n >= 16, dim >= 64: fib-quant/src/codec.rs:612-656): the normalised f32 vectors go through
 * gpu_backend::hadamard_batch instead of the stored rotation; the rest is finish_batch_encode as above. */
PKVO_API int pkvo_fib_encode_batch_hadamard(const float* x, int64_t n, int dim, int k, int n_codewords,
                                            int norm_format, int argmin_order, uint64_t rotation_seed,
                                            const float* codebook, uint8_t* payload, int nthreads,
                                            int32_t* vec_code, int64_t* vec_index) {
  if (dim <= 0 || dim > 512 || k <= 0 || dim % k || n_codewords < 1 || dim / k > 128)
    return PKV_ERR_INVALID_ARGUMENT;
  if (vec_code) *vec_code = 0;
  if (vec_index) *vec_index = -1;
  if (n == 0) return PKV_ERR_EMPTY_BATCH;
  float signs[1024];
  pkvo_hadamard_signs(next_pow2(dim), rotation_seed, signs);
  fib_enc_job J = {x, n, dim, k, n_codewords, norm_format, argmin_order, PKV_FIB_NUMERICS_BATCH, NULL, codebook,
                   payload, signs, 0, -1, 0, -1};
  fib_enc_ctx C;
  C.J = &J;
  C.rec_bytes = pkvo_fib_record_bytes(dim, k, n_codewords, norm_format);
  C.batch_numerics = 1;
  pthread_mutex_init(&C.mu, NULL);
  parallel_for(n, nthreads, fib_enc_range, &C);
  pthread_mutex_destroy(&C.mu);
  int code = J.pass0_code ? J.pass0_code : J.pass1_code;
  int64_t index = J.pass0_code ? J.pass0_index : J.pass1_index;
  if (code) {
    if (vec_code) *vec_code = code;
    if (vec_index) *vec_index = index;
  }
  return code;
}

typedef struct {
  const uint8_t* payload;
  int64_t n;
  int dim, k, n_codewords, norm_format, rec_bytes;
  const float* rot32; /* (f32) of the f64 matrix, fib-quant/src/rotation.rs:139 */
  const float* codebook;
  float* out;
  int64_t out_stride;
  int code;
  int64_t index;
  pthread_mutex_t mu;
} fib_dec_job;

/* One code of FibQuantizer::decode_batch_fast (fib-quant/src/codec.rs:797-844). */
static int fib_decode_one(const fib_dec_job* J, const uint8_t* rec, float* out) {
  const int d = J->dim, k = J->k, blocks = d / k;
  const int norm_len = J->norm_format == PKV_NORM_FP16 ? 2 : 4;
  uint32_t idx[128];
  float rotated[512];
  if (!unpack_bits(rec + norm_len, blocks, fib_index_bits(J->n_codewords), idx))
    return PKV_VEC_PADDING_BITS; /* bitpack.rs:66-72 */
  for (int b = 0; b < blocks; b++) {
    if (idx[b] >= (uint32_t)J->n_codewords) return PKV_VEC_INDEX_RANGE; /* :819-824 */
    memcpy(rotated + b * k, J->codebook + idx[b] * k, sizeof(float) * (size_t)k); /* :827 */
  }
  double norm; /* decode_norm, :1022-1046 */
  if (J->norm_format == PKV_NORM_FP16) {
    float nf = f16_bits_to_f32((uint16_t)(rec[0] | (rec[1] << 8)));
    norm = (double)nf;
  } else {
    uint32_t u = (uint32_t)rec[0] | ((uint32_t)rec[1] << 8) | ((uint32_t)rec[2] << 16) |
                 ((uint32_t)rec[3] << 24);
    norm = (double)pkv_f32_from_bits(u);
  }
  if (!(isfinite(norm) && norm > 0.0)) return PKV_VEC_BAD_NORM;
  float nf = (float)norm; /* `norm as f32`, :838 */
  /* apply_inverse_f32, fib-quant/src/rotation.rs:136-149: per column, rows ascending,
   * f32 multiply then f32 add, starting from 0.0 */
  int bad = 0;
  for (int c = 0; c < d; c++) {
    float sum = 0.0f;
    for (int r = 0; r < d; r++) sum += J->rot32[(size_t)r * d + c] * rotated[r];
    float o = sum * nf;
    if (!is_finite_f32(o)) bad = 1; /* check_finite, :840 */
    out[c] = o;
  }
  return bad ? PKV_VEC_NONFINITE_OUTPUT : 0;
}

static void fib_dec_range(void* p, int64_t lo, int64_t hi) {
  fib_dec_job* J = (fib_dec_job*)p;
  for (int64_t v = lo; v < hi; v++) {
    int code = fib_decode_one(J, J->payload + v * J->rec_bytes, J->out + v * J->out_stride);
    if (code) {
      pthread_mutex_lock(&J->mu);
      if (J->code == 0 || v < J->index) {
        J->code = code;
        J->index = v;
      }
      pthread_mutex_unlock(&J->mu);
    }
  }
}

/* decode_batch_fast over n records -> n vectors at out + v*out_stride. */
/* FibQuantizer::decode (fib-quant/src/codec.rs:506-537): the single-vector decoder keeps binary64 --
 * codewords widened (codebook.rs:118-130), StoredRotation::apply_inverse (rotation.rs:118-130: per
 * column, rows ascending, `sum += m * v` in binary64 from 0.0), `(value * norm) as f32`.  Serial: it is
 * what KVecCodec::decode calls per payload (proveKV/src/codec.rs:612-638). */
PKVO_API int pkvo_fib_decode_exact_batch(const uint8_t* payload, int64_t n, int dim, int k, int n_codewords,
                                         int norm_format, const double* rot, const float* codebook,
                                         float* out, int32_t* vec_code, int64_t* vec_index) {
  if (dim <= 0 || dim > 512 || k <= 0 || dim % k || dim / k > 128) return PKV_ERR_INVALID_ARGUMENT;
  const int blocks = dim / k, norm_len = norm_format == PKV_NORM_FP16 ? 2 : 4;
  const int rec_bytes = pkvo_fib_record_bytes(dim, k, n_codewords, norm_format);
  if (vec_code) *vec_code = 0;
  if (vec_index) *vec_index = -1;
  for (int64_t v = 0; v < n; v++) {
    const uint8_t* rec = payload + v * rec_bytes;
    uint32_t idx[128];
    double rotated[512];
    int code = 0;
    if (!unpack_bits(rec + norm_len, blocks, fib_index_bits(n_codewords), idx)) code = PKV_VEC_PADDING_BITS;
    for (int b = 0; b < blocks && !code; b++) {
      if (idx[b] >= (uint32_t)n_codewords) code = PKV_VEC_INDEX_RANGE;
      else
        for (int j = 0; j < k; j++) rotated[b * k + j] = (double)codebook[idx[b] * k + j];
    }
    double norm = 0.0;
    if (!code) {
      if (norm_format == PKV_NORM_FP16) norm = (double)f16_bits_to_f32((uint16_t)(rec[0] | (rec[1] << 8)));
      else
        norm = (double)pkv_f32_from_bits((uint32_t)rec[0] | ((uint32_t)rec[1] << 8) | ((uint32_t)rec[2] << 16) |
                                         ((uint32_t)rec[3] << 24));
      if (!(isfinite(norm) && norm > 0.0)) code = PKV_VEC_BAD_NORM;
    }
    if (!code) {
      for (int c = 0; c < dim; c++) {
        double sum = 0.0;
        for (int r = 0; r < dim; r++) sum += rot[(size_t)r * dim + c] * rotated[r];
        const float o = (float)(sum * norm);
        if (!is_finite_f32(o)) code = PKV_VEC_NONFINITE_OUTPUT;
        out[v * dim + c] = o;
      }
    }
    if (code) {
      if (vec_code) *vec_code = code;
      if (vec_index) *vec_index = v;
      return code;
    }
  }
  return 0;
}

PKVO_API int pkvo_fib_decode_batch(const uint8_t* payload, int64_t n, int dim, int k,
                                   int n_codewords, int norm_format, const double* rot,
                                   const float* codebook, float* out, int64_t out_stride,
                                   int nthreads, int32_t* vec_code, int64_t* vec_index) {
  if (dim <= 0 || dim > 512 || k <= 0 || dim % k || dim / k > 128) return PKV_ERR_INVALID_ARGUMENT;
  if (vec_code) *vec_code = 0;
  if (vec_index) *vec_index = -1;
  float* rot32 = (float*)malloc(sizeof(float) * (size_t)dim * dim);
  for (int i = 0; i < dim * dim; i++) rot32[i] = (float)rot[i];
  fib_dec_job J;
  J.payload = payload;
  J.n = n;
  J.dim = dim;
  J.k = k;
  J.n_codewords = n_codewords;
  J.norm_format = norm_format;
  J.rec_bytes = pkvo_fib_record_bytes(dim, k, n_codewords, norm_format);
  J.rot32 = rot32;
  J.codebook = codebook;
  J.out = out;
  J.out_stride = out_stride;
  J.code = 0;
  J.index = -1;
  pthread_mutex_init(&J.mu, NULL);
  parallel_for(n, nthreads, fib_dec_range, &J);
  pthread_mutex_destroy(&J.mu);
  free(rot32);
  if (J.code) {
    if (vec_code) *vec_code = J.code;
    if (vec_index) *vec_index = J.index;
  }
  return J.code;
}

/* FB2 header, fib-quant/src/codec.rs:195-220,287-296. */
PKVO_API void pkvo_fb2_header_write(int dim, int k, int n_codewords, int norm_format,
                                    uint32_t n_vectors, uint8_t* out) {
  uint32_t blocks = (uint32_t)(dim / k);
  int bits = fib_index_bits(n_codewords);
  uint16_t norm_len = norm_format == PKV_NORM_FP16 ? 2 : 4;
  uint16_t idx_len = (uint16_t)((blocks * (uint32_t)bits + 7) / 8);
  out[0] = 'F';
  out[1] = 'B';
  out[2] = '2';
  out[3] = 1;
  out[4] = (uint8_t)bits;
  out[5] = 0;
  memcpy(out + 6, &blocks, 4);
  memcpy(out + 10, &n_vectors, 4);
  out[14] = (uint8_t)norm_format;
  memcpy(out + 15, &norm_len, 2);
  memcpy(out + 17, &idx_len, 2);
}

/* FibCodeV1::decode_batch header checks, fib-quant/src/codec.rs:323-398.
 * Returns 0 and n_vectors, or PKV_ERR_CORRUPT_HEADER. */
PKVO_API int pkvo_fb2_header_parse(int dim, int k, int n_codewords, int norm_format,
                                   const uint8_t* bytes, int64_t len, uint32_t* n_vectors) {
  if (len < 19) return PKV_ERR_CORRUPT_HEADER;
  if (bytes[0] != 'F' || bytes[1] != 'B' || bytes[2] != '2' || bytes[3] != 1)
    return PKV_ERR_CORRUPT_HEADER;
  uint32_t blocks, n;
  uint16_t norm_len, idx_len;
  memcpy(&blocks, bytes + 6, 4);
  memcpy(&n, bytes + 10, 4);
  memcpy(&norm_len, bytes + 15, 2);
  memcpy(&idx_len, bytes + 17, 2);
  int bits = fib_index_bits(n_codewords);
  if (bytes[4] != bits) return PKV_ERR_CORRUPT_HEADER;
  if (blocks != (uint32_t)(dim / k)) return PKV_ERR_CORRUPT_HEADER;
  if (bytes[14] > 1 || bytes[14] != norm_format) return PKV_ERR_CORRUPT_HEADER;
  if ((int64_t)len < 19 + (int64_t)n * (norm_len + idx_len)) return PKV_ERR_CORRUPT_HEADER;
  if (idx_len != (blocks * (uint32_t)bits + 7) / 8) return PKV_ERR_CORRUPT_HEADER;
  /* the per-code norm length is checked by decode_norm's try_into, :1025-1027 */
  if (norm_len != (norm_format == PKV_NORM_FP16 ? 2 : 4)) return PKV_ERR_CORRUPT_HEADER;
  *n_vectors = n;
  return 0;
}

/* ------------------------------------------------------------------------ */
/* turbo-quant                                                                */
/* ------------------------------------------------------------------------ */

#define PKVO_PI_F 3.14159274101257324f /* std::f32::consts::PI */

/* fwht_normalized, turbo-quant/src/rotation.rs:379-398 */
static void fwht_normalized(float* v, int n) {
  for (int step = 1; step < n; step *= 2)
    for (int start = 0; start < n; start += 2 * step)
      for (int o = 0; o < step; o++) {
        float a = v[start + o], b = v[start + o + step];
        v[start + o] = a + b;
        v[start + o + step] = a - b;
      }
  float scale = 1.0f / sqrtf((float)n); /* (n as f32).sqrt().recip() */
  for (int i = 0; i < n; i++) v[i] *= scale;
}

PKVO_API void pkvo_fwht_normalized(float* v, int n) { fwht_normalized(v, n); }

static float atan2f_mode(float y, float x, int libm_mode) {
  return libm_mode == PKVO_LIBM_PORTABLE ? pkv_atan2f_portable(y, x) : atan2f(y, x);
}
static float logf_mode(float x, int libm_mode) {
  return libm_mode == PKVO_LIBM_PORTABLE ? pkv_logf_portable(x) : logf(x);
}
static float expf_mode(float x, int libm_mode) {
  return libm_mode == PKVO_LIBM_PORTABLE ? pkv_expf_portable(x) : expf(x);
}

PKVO_API float pkvo_atan2f(float y, float x, int libm_mode) { return atan2f_mode(y, x, libm_mode); }
PKVO_API float pkvo_logf(float x, int libm_mode) { return logf_mode(x, libm_mode); }
PKVO_API float pkvo_expf(float x, int libm_mode) { return expf_mode(x, libm_mode); }

/* encode_pair's angle bucket, turbo-quant/src/polar.rs:415-420 */
static uint32_t angle_bucket(float theta, uint32_t levels) {
  float normalized = (theta + PKVO_PI_F) / (2.0f * PKVO_PI_F);
  float scaled = floorf(normalized * (float)levels);
  uint32_t u = scaled >= 4294967296.0f ? 0xffffffffu : (scaled > 0.0f ? (uint32_t)scaled : 0u);
  return u % levels;
}
PKVO_API uint32_t pkvo_angle_bucket(float theta, uint32_t levels) { return angle_bucket(theta, levels); }

/* PolarCode::dequantize_angle, turbo-quant/src/polar.rs:91-95 */
static float dequantize_angle(uint32_t idx, uint32_t levels) {
  return ((float)idx / (float)levels) * (2.0f * PKVO_PI_F) - PKVO_PI_F;
}

/* cos / sin of every dequantised angle with the host libm (polar.rs:312-313). */
PKVO_API void pkvo_polar_lut(int polar_bits, float* cos_lut, float* sin_lut) {
  uint32_t levels = 1u << polar_bits;
  for (uint32_t i = 0; i < levels; i++) {
    float t = dequantize_angle(i, levels);
    cos_lut[i] = cosf(t);
    sin_lut[i] = sinf(t);
  }
}

PKVO_API int pkvo_turbo_polar_bits(int bits, int mode) {
  return mode == PKV_TURBO_POLAR_WITH_QJL ? bits - 1 : bits; /* turbo.rs:169-172 */
}

/* wire.rs:311-327 */
PKVO_API int pkvo_turbo_record_bytes(int dim, int bits, int mode, int projections, int radii_codec) {
  int pairs = dim / 2, pb = pkvo_turbo_polar_bits(bits, mode);
  int radii = radii_codec == PKV_RADII_F32 ? pairs * 4 : pairs + 8;
  int angles = (pairs * pb + 7) / 8;
  int signs = mode == PKV_TURBO_POLAR_WITH_QJL ? (projections + 7) / 8 : 0;
  return radii + angles + signs;
}

typedef struct {
  const float* x;
  const uint8_t* payload_in;
  uint8_t* payload;
  float* out;
  int64_t out_stride;
  int64_t n;
  int dim, bits, mode, projections, radii_codec, libm_mode, rec_bytes;
  const float* signs;
  const float* qjl;
  const float* cos_lut;
  const float* sin_lut;
  int code;
  int64_t index;
  pthread_mutex_t mu;
} turbo_job;

/* TurboQuantizer::encode (turbo.rs:256-288) + the per-vector body of
 * TurboCodeWireV1::encode_batch_with_radii (wire.rs:350-396). */
static int turbo_encode_one(const turbo_job* J, const float* x, uint8_t* rec) {
  const int d = J->dim, pairs = d / 2;
  const int pb = pkvo_turbo_polar_bits(J->bits, J->mode);
  const uint32_t levels = 1u << pb;
  float rot[512], radii[256];
  uint32_t aidx[256];
  for (int i = 0; i < d; i++)
    if (!is_finite_f32(x[i])) return PKV_VEC_NONFINITE_INPUT; /* turbo.rs:263, polar.rs:248 */
  /* FastHadamardRotation::apply, rotation.rs:202-210 */
  for (int i = 0; i < d; i++) rot[i] = x[i] * J->signs[i];
  fwht_normalized(rot, d);
  /* encode_pair, polar.rs:413-421 */
  for (int i = 0; i < pairs; i++) {
    float a = rot[2 * i], b = rot[2 * i + 1];
    radii[i] = sqrtf(a * a + b * b);
    aidx[i] = angle_bucket(atan2f_mode(b, a, J->libm_mode), levels);
  }
  /* PolarCode::from_parts -> validate_for, polar.rs:127-133 */
  for (int i = 0; i < pairs; i++)
    if (!is_finite_f32(radii[i]) || radii[i] < 0.0f) return PKV_VEC_BAD_RADIUS;
  uint32_t signs_bits[64];
  if (J->mode == PKV_TURBO_POLAR_WITH_QJL) {
    /* polar.decode, polar.rs:272-278,306-316 then rotation.rs:212-221 */
    float rec_v[512];
    for (int i = 0; i < pairs; i++) {
      rec_v[2 * i] = radii[i] * J->cos_lut[aidx[i]];
      rec_v[2 * i + 1] = radii[i] * J->sin_lut[aidx[i]];
    }
    fwht_normalized(rec_v, d);
    for (int i = 0; i < d; i++) rec_v[i] *= J->signs[i];
    float res[512];
    for (int i = 0; i < d; i++) {
      res[i] = x[i] - rec_v[i]; /* turbo.rs:269-273 */
      if (!is_finite_f32(res[i])) return PKV_VEC_NONFINITE_RESIDUAL; /* qjl.rs:210 */
    }
    /* QjlQuantizer::sketch, qjl.rs:214-217: per row a sequential f32 dot, sign = dot >= 0 */
    for (int p = 0; p < J->projections; p++) {
      const float* g = J->qjl + (size_t)p * d;
      float dot = 0.0f;
      for (int j = 0; j < d; j++) dot += g[j] * res[j];
      signs_bits[p] = dot >= 0.0f ? 1u : 0u;
    }
  }
  uint8_t* w = rec;
  if (J->radii_codec == PKV_RADII_F32) { /* radius.rs:27-39 */
    memcpy(w, radii, (size_t)pairs * 4);
    w += pairs * 4;
  } else { /* BlockLogU8, radius.rs:58-77 */
    float logged[256];
    float mn = INFINITY, mx = -INFINITY;
    for (int i = 0; i < pairs; i++) {
      float r = radii[i] > 1.17549435e-38f ? radii[i] : 1.17549435e-38f; /* max(f32::MIN_POSITIVE) */
      logged[i] = logf_mode(r, J->libm_mode);
      mn = logged[i] < mn ? logged[i] : mn;
      mx = logged[i] > mx ? logged[i] : mx;
    }
    float span = mx - mn;
    if (!(span > 1.1920929e-07f)) span = 1.1920929e-07f; /* .max(f32::EPSILON) */
    for (int i = 0; i < pairs; i++) {
      float nrm = (logged[i] - mn) / span;
      nrm = nrm < 0.0f ? 0.0f : (nrm > 1.0f ? 1.0f : nrm); /* clamp(0,1) */
      w[i] = (uint8_t)roundf(nrm * 255.0f);
    }
    w += pairs;
    memcpy(w, &mn, 4);     /* wire.rs:368-371 */
    memcpy(w + 4, &mx, 4);
    w += 8;
  }
  int alen = (pairs * pb + 7) / 8;
  pack_bits(aidx, pairs, pb, w, alen);
  w += alen;
  if (J->mode == PKV_TURBO_POLAR_WITH_QJL)
    pack_bits(signs_bits, J->projections, 1, w, (J->projections + 7) / 8); /* bitpack.rs:48-62 */
  return 0;
}

static void turbo_report(turbo_job* J, int64_t v, int code) {
  pthread_mutex_lock(&J->mu);
  if (J->code == 0 || v < J->index) {
    J->code = code;
    J->index = v;
  }
  pthread_mutex_unlock(&J->mu);
}

static void turbo_enc_range(void* p, int64_t lo, int64_t hi) {
  turbo_job* J = (turbo_job*)p;
  for (int64_t v = lo; v < hi; v++) {
    int code = turbo_encode_one(J, J->x + v * J->dim, J->payload + v * J->rec_bytes);
    if (code) turbo_report(J, v, code);
  }
}

/* The per-vector body of TurboCodeWireV1::decode_batch (wire.rs:497-565) and
 * PolarQuantizer::decode_batch (polar.rs:286-316, rotation.rs:170-194). */
static int turbo_decode_one(const turbo_job* J, const uint8_t* rec, float* out) {
  const int d = J->dim, pairs = d / 2;
  const int pb = pkvo_turbo_polar_bits(J->bits, J->mode);
  float radii[256];
  uint32_t aidx[256];
  const uint8_t* r = rec;
  if (J->radii_codec == PKV_RADII_F32) { /* radius.rs:84-107 */
    memcpy(radii, r, (size_t)pairs * 4);
    r += pairs * 4;
    for (int i = 0; i < pairs; i++)
      if (!is_finite_f32(radii[i]) || radii[i] < 0.0f) return PKV_VEC_BAD_RADIUS;
  } else { /* radius.rs:128-145 */
    float mn, mx;
    memcpy(&mn, r + pairs, 4);
    memcpy(&mx, r + pairs + 4, 4);
    if (!is_finite_f32(mn) || !is_finite_f32(mx) || mn > mx) return PKV_VEC_BAD_RADIUS_RANGE;
    float span = mx - mn;
    for (int i = 0; i < pairs; i++)
      radii[i] = expf_mode(mn + span * ((float)r[i] / 255.0f), J->libm_mode);
    r += pairs + 8;
  }
  int alen = (pairs * pb + 7) / 8;
  if (!unpack_bits(r, pairs, pb, aidx)) return PKV_VEC_PADDING_BITS;
  r += alen;
  if (J->mode == PKV_TURBO_POLAR_WITH_QJL) {
    uint32_t sg[64];
    if (!unpack_bits(r, J->projections, 1, sg)) return PKV_VEC_PADDING_BITS;
  }
  /* TurboCode::validate_for -> PolarCode::validate_for, polar.rs:127-133 */
  for (int i = 0; i < pairs; i++)
    if (!is_finite_f32(radii[i]) || radii[i] < 0.0f) return PKV_VEC_BAD_RADIUS;
  for (int i = 0; i < pairs; i++) {
    out[2 * i] = radii[i] * J->cos_lut[aidx[i]];
    out[2 * i + 1] = radii[i] * J->sin_lut[aidx[i]];
  }
  fwht_normalized(out, d);
  for (int i = 0; i < d; i++) out[i] *= J->signs[i];
  return 0;
}

static void turbo_dec_range(void* p, int64_t lo, int64_t hi) {
  turbo_job* J = (turbo_job*)p;
  for (int64_t v = lo; v < hi; v++) {
    int code = turbo_decode_one(J, J->payload_in + v * J->rec_bytes, J->out + v * J->out_stride);
    if (code) turbo_report(J, v, code);
  }
}

/* TurboQuantizer::prepare_query (turbo.rs:322-337): the query after FastHadamardRotation::apply
 * (polar.rs:336-343, rotation.rs:202-210) and after the QJL matrix (qjl.rs:266-281: per row the
 * products g * q summed in order).  projected may be NULL for polar-only. */
PKVO_API int pkvo_turbo_prepare_query(const float* query, int dim, int projections, const float* signs,
                                      const float* qjl, float* rotated, float* projected) {
  if (dim <= 0 || dim > 512 || (dim & (dim - 1))) return PKV_ERR_INVALID_ARGUMENT;
  for (int i = 0; i < dim; i++)
    if (!is_finite_f32(query[i])) return PKV_VEC_NONFINITE_INPUT;
  for (int i = 0; i < dim; i++) rotated[i] = query[i] * signs[i];
  fwht_normalized(rotated, dim);
  for (int i = 0; i < dim; i++)
    if (!is_finite_f32(rotated[i])) return PKV_VEC_NONFINITE_INPUT;
  if (projected && qjl) {
    for (int j = 0; j < projections; j++) {
      volatile float sum = 0.0f;
      for (int k = 0; k < dim; k++) {
        volatile float prod = qjl[(size_t)j * dim + k] * query[k];
        sum = sum + prod;
      }
      projected[j] = sum;
      if (!is_finite_f32(projected[j])) return PKV_VEC_NONFINITE_INPUT;
    }
  }
  return 0;
}

/* TurboQuantizer::inner_product_estimate_prepared for one wire record (turbo.rs:340-369): record
 * parsed and validated as in turbo_decode_one, polar estimate polar.rs:346-370, QJL correction
 * qjl.rs:294-330 with source_norm 1. */
static int turbo_score_one(const turbo_job* J, const uint8_t* rec, const float* rotated,
                           const float* projected, float* score) {
  const int d = J->dim, pairs = d / 2;
  const int pb = pkvo_turbo_polar_bits(J->bits, J->mode);
  float radii[256];
  uint32_t aidx[256], sg[64];
  const uint8_t* r = rec;
  *score = 0.0f;
  if (J->radii_codec == PKV_RADII_F32) {
    memcpy(radii, r, (size_t)pairs * 4);
    r += pairs * 4;
    for (int i = 0; i < pairs; i++)
      if (!is_finite_f32(radii[i]) || radii[i] < 0.0f) return PKV_VEC_BAD_RADIUS;
  } else {
    float mn, mx;
    memcpy(&mn, r + pairs, 4);
    memcpy(&mx, r + pairs + 4, 4);
    if (!is_finite_f32(mn) || !is_finite_f32(mx) || mn > mx) return PKV_VEC_BAD_RADIUS_RANGE;
    float span = mx - mn;
    for (int i = 0; i < pairs; i++)
      radii[i] = expf_mode(mn + span * ((float)r[i] / 255.0f), J->libm_mode);
    r += pairs + 8;
  }
  if (!unpack_bits(r, pairs, pb, aidx)) return PKV_VEC_PADDING_BITS;
  r += (pairs * pb + 7) / 8;
  if (J->mode == PKV_TURBO_POLAR_WITH_QJL && !unpack_bits(r, J->projections, 1, sg)) return PKV_VEC_PADDING_BITS;
  for (int i = 0; i < pairs; i++)
    if (!is_finite_f32(radii[i]) || radii[i] < 0.0f) return PKV_VEC_BAD_RADIUS;
  volatile float estimate = 0.0f;
  for (int i = 0; i < pairs; i++) {
    volatile float qa = rotated[2 * i] * J->cos_lut[aidx[i]];
    volatile float qb = rotated[2 * i + 1] * J->sin_lut[aidx[i]];
    volatile float inner = qa + qb;
    volatile float term = radii[i] * inner;
    estimate = estimate + term;
  }
  if (!is_finite_f32(estimate)) return PKV_VEC_NONFINITE_OUTPUT;
  float total = estimate;
  if (J->mode == PKV_TURBO_POLAR_WITH_QJL) {
    const float pi = 3.14159274101257324f;
    volatile float root = sqrtf(pi / 2.0f);
    volatile float scale = (root * 1.0f) / (float)J->projections;
    volatile float sum = 0.0f;
    for (int j = 0; j < J->projections; j++) {
      volatile float term = (sg[j] ? 1.0f : -1.0f) * projected[j];
      sum = sum + term;
    }
    volatile float corr = scale * sum;
    if (!is_finite_f32(corr)) return PKV_VEC_NONFINITE_OUTPUT;
    total = estimate + corr;
    if (!is_finite_f32(total)) return PKV_VEC_NONFINITE_OUTPUT;
  }
  *score = total;
  return 0;
}

/* TurboQuantizer::score_batch_prepared (turbo.rs:372-381): the first failing record ends the batch. */
PKVO_API int pkvo_turbo_score_batch(const uint8_t* payload, int64_t n, int dim, int bits, int mode,
                                    int projections, int radii_codec, int libm_mode, const float* cos_lut,
                                    const float* sin_lut, const float* rotated, const float* projected,
                                    float* scores, int32_t* vec_code, int64_t* vec_index);

static int turbo_job_init(turbo_job* J, int64_t n, int dim, int bits, int mode, int projections,
                          int radii_codec, int libm_mode, const float* signs, const float* qjl,
                          const float* cos_lut, const float* sin_lut) {
  if (dim <= 0 || dim > 512 || (dim & (dim - 1)) || projections > 64) return PKV_ERR_INVALID_ARGUMENT;
  int pb = pkvo_turbo_polar_bits(bits, mode);
  if (pb < 1 || pb > 16) return PKV_ERR_INVALID_ARGUMENT;
  memset(J, 0, sizeof(*J));
  J->n = n;
  J->dim = dim;
  J->bits = bits;
  J->mode = mode;
  J->projections = projections;
  J->radii_codec = radii_codec;
  J->libm_mode = libm_mode;
  J->rec_bytes = pkvo_turbo_record_bytes(dim, bits, mode, projections, radii_codec);
  J->signs = signs;
  J->qjl = qjl;
  J->cos_lut = cos_lut;
  J->sin_lut = sin_lut;
  J->code = 0;
  J->index = -1;
  pthread_mutex_init(&J->mu, NULL);
  return 0;
}

PKVO_API int pkvo_turbo_score_batch(const uint8_t* payload, int64_t n, int dim, int bits, int mode,
                                    int projections, int radii_codec, int libm_mode, const float* cos_lut,
                                    const float* sin_lut, const float* rotated, const float* projected,
                                    float* scores, int32_t* vec_code, int64_t* vec_index) {
  turbo_job J;
  int st = turbo_job_init(&J, n, dim, bits, mode, projections, radii_codec, libm_mode, NULL, NULL, cos_lut,
                          sin_lut);
  if (st) return st;
  if (vec_code) *vec_code = 0;
  if (vec_index) *vec_index = -1;
  for (int64_t v = 0; v < n; v++) {
    int code = turbo_score_one(&J, payload + v * J.rec_bytes, rotated, projected, scores + v);
    if (code) {
      if (vec_code) *vec_code = code;
      if (vec_index) *vec_index = v;
      pthread_mutex_destroy(&J.mu);
      return code;
    }
  }
  pthread_mutex_destroy(&J.mu);
  return 0;
}

PKVO_API int pkvo_turbo_encode_batch(const float* x, int64_t n, int dim, int bits, int mode,
                                     int projections, int radii_codec, int libm_mode,
                                     const float* signs, const float* qjl, const float* cos_lut,
                                     const float* sin_lut, uint8_t* payload, int nthreads,
                                     int32_t* vec_code, int64_t* vec_index) {
  turbo_job J;
  int st = turbo_job_init(&J, n, dim, bits, mode, projections, radii_codec, libm_mode, signs, qjl,
                          cos_lut, sin_lut);
  if (st) return st;
  if (vec_code) *vec_code = 0;
  if (vec_index) *vec_index = -1;
  if (n == 0) return PKV_ERR_EMPTY_BATCH; /* wire.rs:302-306 */
  J.x = x;
  J.payload = payload;
  parallel_for(n, nthreads, turbo_enc_range, &J);
  pthread_mutex_destroy(&J.mu);
  if (J.code) {
    if (vec_code) *vec_code = J.code;
    if (vec_index) *vec_index = J.index;
  }
  return J.code;
}

PKVO_API int pkvo_turbo_decode_batch(const uint8_t* payload, int64_t n, int dim, int bits, int mode,
                                     int projections, int radii_codec, int libm_mode,
                                     const float* signs, const float* cos_lut, const float* sin_lut,
                                     float* out, int64_t out_stride, int nthreads,
                                     int32_t* vec_code, int64_t* vec_index) {
  turbo_job J;
  int st = turbo_job_init(&J, n, dim, bits, mode, projections, radii_codec, libm_mode, signs, NULL,
                          cos_lut, sin_lut);
  if (st) return st;
  if (vec_code) *vec_code = 0;
  if (vec_index) *vec_index = -1;
  J.payload_in = payload;
  J.out = out;
  J.out_stride = out_stride;
  parallel_for(n, nthreads, turbo_dec_range, &J);
  pthread_mutex_destroy(&J.mu);
  if (J.code) {
    if (vec_code) *vec_code = J.code;
    if (vec_index) *vec_index = J.index;
  }
  return J.code;
}

/* TQB1 header, turbo-quant/src/wire.rs:276-290,330-349. rotation flag 1 =
 * FastHadamard (wire.rs:583-589; Auto resolves to it for power-of-two dims). */
PKVO_API void pkvo_tqb1_header_write(int dim, int bits, int mode, int projections, int radii_codec,
                                     uint64_t seed, uint32_t n_vectors, uint8_t* out) {
  uint16_t ver = 1, rot = 1;
  uint32_t d = (uint32_t)dim, m = (uint32_t)projections;
  uint32_t rec = (uint32_t)pkvo_turbo_record_bytes(dim, bits, mode, projections, radii_codec);
  memcpy(out, "TQB1", 4);
  memcpy(out + 4, &ver, 2);
  memcpy(out + 6, &rot, 2);
  out[8] = 2;
  out[9] = 0;
  memcpy(out + 10, &d, 4);
  out[14] = (uint8_t)pkvo_turbo_polar_bits(bits, mode);
  out[15] = (uint8_t)(radii_codec == PKV_RADII_F32 ? 0 : 1);
  out[16] = 0;
  out[17] = 0;
  memcpy(out + 18, &m, 4);
  memcpy(out + 22, &seed, 8);
  memcpy(out + 30, &n_vectors, 4);
  memcpy(out + 34, &rec, 4);
}

/* TurboCodeWireV1::decode_batch header checks, wire.rs:401-495, and the
 * exact-length rule of WireCursor::finish (wire.rs:566). radii_codec is read
 * from byte 15 and returned. */
PKVO_API int pkvo_tqb1_header_parse(int dim, int bits, int mode, int projections, uint64_t seed,
                                    const uint8_t* bytes, int64_t len, uint32_t* n_vectors,
                                    int32_t* radii_codec) {
  if (len < 38) return PKV_ERR_CORRUPT_HEADER;
  uint16_t ver, rot;
  uint32_t d, m, n, rec;
  uint64_t s;
  if (memcmp(bytes, "TQB1", 4)) return PKV_ERR_CORRUPT_HEADER;
  memcpy(&ver, bytes + 4, 2);
  memcpy(&rot, bytes + 6, 2);
  memcpy(&d, bytes + 10, 4);
  memcpy(&m, bytes + 18, 4);
  memcpy(&s, bytes + 22, 8);
  memcpy(&n, bytes + 30, 4);
  memcpy(&rec, bytes + 34, 4);
  if (ver != 1 || rot != 1 || bytes[8] != 2) return PKV_ERR_CORRUPT_HEADER;
  if (bytes[15] > 1) return PKV_ERR_CORRUPT_HEADER;
  if (d != (uint32_t)dim || m != (uint32_t)projections || s != seed) return PKV_ERR_CORRUPT_HEADER;
  if (bytes[14] != pkvo_turbo_polar_bits(bits, mode)) return PKV_ERR_CORRUPT_HEADER;
  int codec = bytes[15] ? PKV_RADII_BLOCK_LOG_U8 : PKV_RADII_F32;
  if (rec != (uint32_t)pkvo_turbo_record_bytes(dim, bits, mode, projections, codec))
    return PKV_ERR_CORRUPT_HEADER;
  if (len != 38 + (int64_t)n * rec) return PKV_ERR_CORRUPT_HEADER;
  *n_vectors = n;
  *radii_codec = codec;
  return 0;
}

/* ------------------------------------------------------------------------ */
/* CPU check of the kernels' certified shortcuts (provekv_b200/csrc/pkv_fast_paths.h) */
/* ------------------------------------------------------------------------ */
#include "../provekv_b200/csrc/pkv_fast_paths.h"

static uint64_t xs64(uint64_t* s) {
  uint64_t x = *s;
  x ^= x << 13;
  x ^= x >> 7;
  x ^= x << 17;
  return *s = x;
}
static double unif(uint64_t* s) { return (double)(xs64(s) >> 11) * (1.0 / 9007199254740992.0); }

/* Runs the bucket shortcut on n pairs: a mix of Gaussian-like pairs, pairs placed within
 * +-spread radians of a sector boundary at many magnitudes, and degenerate pairs.  Every decided
 * pair must equal the exact bucket (portable atan2f + polar.rs:415-420).  counts[0] = decided and
 * wrong, counts[1] = undecided, counts[2] = decided. */
PKVO_API void pkvo_fast_bucket_check(int polar_bits, int64_t n, uint64_t seed, double spread,
                                     int64_t* counts) {
  const int levels = 1 << polar_bits, rays = levels / 4 + 1;
  float rc[80], rs[80];
  for (int t = 0; t < rays; t++) {
    double beta = 2.0 * 3.14159265358979323846 * t / levels;
    rc[t] = (float)cos(beta);
    rs[t] = (float)sin(beta);
  }
  uint64_t s = seed * 2654435761u + 88172645463325252ull;
  counts[0] = counts[1] = counts[2] = 0;
  for (int64_t i = 0; i < n; i++) {
    float a, b;
    int kind = (int)(xs64(&s) % 8);
    if (kind < 3) {
      a = (float)((unif(&s) + unif(&s) + unif(&s) - 1.5) * 4.0);
      b = (float)((unif(&s) + unif(&s) + unif(&s) - 1.5) * 4.0);
    } else if (kind < 7) {
      int k = (int)(xs64(&s) % (uint64_t)levels);
      double ang = -3.14159265358979323846 + 2.0 * 3.14159265358979323846 * k / levels +
                   (unif(&s) - 0.5) * 2.0 * spread;
      double r = exp((unif(&s) - 0.5) * (kind == 6 ? 160.0 : 12.0));
      a = (float)(r * cos(ang));
      b = (float)(r * sin(ang));
    } else {
      static const float sp[] = {0.0f, -0.0f, 1.0f, -1.0f, 1e-45f, -1e-45f, 3e38f, -3e38f, 1e-38f};
      a = sp[xs64(&s) % 9];
      b = sp[xs64(&s) % 9];
    }
    int certain = 0;
    uint32_t fast = pkv_fast_bucket_any(a, b, polar_bits, rc, rs, &certain);
    if (!certain) {
      counts[1]++;
      continue;
    }
    counts[2]++;
    if (fast != angle_bucket(pkv_atan2f_portable(b, a), (uint32_t)levels)) counts[0]++;
  }
}

/* Sign shortcut of the QJL rows: fused four-chain dot vs the reference's sequential dot.
 * counts[0] = decided with the wrong sign, counts[1] = undecided, counts[2] = decided. */
PKVO_API void pkvo_fast_qjl_check(int dim, int64_t n, uint64_t seed, double res_scale, int64_t* counts) {
  uint64_t s = seed * 11400714819323198485ull + 1;
  counts[0] = counts[1] = counts[2] = 0;
  float g[128], x[128];
  for (int64_t i = 0; i < n; i++) {
    double g2 = 0.0, x2 = 0.0;
    for (int j = 0; j < dim; j++) {
      g[j] = (float)((unif(&s) + unif(&s) + unif(&s) + unif(&s) - 2.0) * 1.7);
      x[j] = (float)((unif(&s) + unif(&s) + unif(&s) + unif(&s) - 2.0) * res_scale);
      g2 += (double)g[j] * g[j];
    }
    /* every other case: make the exact dot tiny by projecting x off g */
    if (i & 1) {
      double dot = 0.0;
      for (int j = 0; j < dim; j++) dot += (double)g[j] * x[j];
      double f = dot / g2 * (1.0 - unif(&s) * 1e-6);
      for (int j = 0; j < dim; j++) x[j] = (float)((double)x[j] - f * g[j]);
    }
    for (int j = 0; j < dim; j++) x2 += (double)x[j] * x[j];
    float thr = (float)(sqrt(g2) * 1.0001) * PKV_QJL_REL_BOUND;
    float s2 = 0.0f;
    for (int j = 0; j < dim; j++) s2 = fmaf(x[j], x[j], s2);
    float rnorm = sqrtf(s2) * 1.0001f;
    float d0 = 0, d1 = 0, d2 = 0, d3 = 0;
    for (int j = 0; j < dim; j += 4) {
      d0 = fmaf(g[j], x[j], d0);
      d1 = fmaf(g[j + 1], x[j + 1], d1);
      d2 = fmaf(g[j + 2], x[j + 2], d2);
      d3 = fmaf(g[j + 3], x[j + 3], d3);
    }
    float fast = (d0 + d1) + (d2 + d3);
    float tau = fmaf(thr, rnorm, PKV_QJL_ABS_BOUND);
    if (!(fabsf(fast) > tau)) {
      counts[1]++;
      continue;
    }
    counts[2]++;
    float ref = 0.0f;
    for (int j = 0; j < dim; j++) ref += g[j] * x[j];
    if ((ref >= 0.0f) != (fast >= 0.0f)) counts[0]++;
  }
}

/* Tensor-core (TF32) tier of the QJL sign shortcut: operands cut to 10 mantissa bits by truncation
 * (variant 0) or round-to-nearest (variant 1), products summed in binary32 in blocks of 8 terms.
 * counts as in pkvo_fast_qjl_check. */
static float tf32_cut(float v, int variant) {
  uint32_t u;
  memcpy(&u, &v, 4);
  if (variant) u += 0x00001000u;
  u &= 0xffffe000u;
  memcpy(&v, &u, 4);
  return v;
}

PKVO_API void pkvo_fast_qjl_tf32_check(int dim, int64_t n, uint64_t seed, double res_scale, int variant,
                                       int64_t* counts) {
  uint64_t s = seed * 11400714819323198485ull + 1;
  counts[0] = counts[1] = counts[2] = 0;
  float g[128], x[128];
  for (int64_t i = 0; i < n; i++) {
    double g2 = 0.0;
    for (int j = 0; j < dim; j++) {
      g[j] = (float)((unif(&s) + unif(&s) + unif(&s) + unif(&s) - 2.0) * 1.7);
      x[j] = (float)((unif(&s) + unif(&s) + unif(&s) + unif(&s) - 2.0) * res_scale);
      g2 += (double)g[j] * g[j];
    }
    if (i & 1) { /* every other case: a dot near the threshold of this tier */
      double dot = 0.0;
      for (int j = 0; j < dim; j++) dot += (double)g[j] * x[j];
      double f = dot / g2 * (1.0 - (unif(&s) - 0.5) * 0.1);
      for (int j = 0; j < dim; j++) x[j] = (float)((double)x[j] - f * g[j]);
    }
    float thr = (float)(sqrt(g2) * 1.0001) * PKV_QJL_TF32_BOUND;
    float s2 = 0.0f;
    for (int j = 0; j < dim; j++) s2 = fmaf(x[j], x[j], s2);
    float rnorm = sqrtf(s2) * 1.0001f;
    float fast = 0.0f;
    for (int j0 = 0; j0 < dim; j0 += 8) {
      float blk = 0.0f;
      for (int j = j0; j < j0 + 8; j++) blk += tf32_cut(g[j], variant) * tf32_cut(x[j], variant);
      fast += blk;
    }
    float tau = fmaf(thr, rnorm, PKV_QJL_ABS_BOUND);
    if (!(fabsf(fast) > tau)) {
      counts[1]++;
      continue;
    }
    counts[2]++;
    float ref = 0.0f;
    for (int j = 0; j < dim; j++) ref += g[j] * x[j];
    if ((ref >= 0.0f) != (fast >= 0.0f)) counts[0]++;
  }
}

/* BlockLogU8 code shortcut: the fast logarithm is modelled as the exact one displaced by up to
 * the documented error (max(2^-21.41, 3 ulp)) in either direction; counts as in the other checks. */
PKVO_API void pkvo_fast_radius_code_check(int64_t n, uint64_t seed, double spread, int64_t* counts) {
  uint64_t s = seed * 11400714819323198485ull + 7;
  counts[0] = counts[1] = counts[2] = 0;
  for (int64_t i = 0; i < n; i++) {
    float r[32], mn = INFINITY, mx = -INFINITY;
    const double centre = (unif(&s) - 0.5) * 40.0;
    for (int j = 0; j < 32; j++) {
      r[j] = (float)exp(centre + (unif(&s) - 0.5) * spread);
      if (!(r[j] > FLT_MIN)) r[j] = FLT_MIN;
      const float l = pkv_logf_portable(r[j]);
      mn = l < mn ? l : mn;
      mx = l > mx ? l : mx;
    }
    float span = mx - mn;
    if (!(span > FLT_EPSILON)) span = FLT_EPSILON;
    const float k = 255.0f / span;
    for (int j = 0; j < 32; j++) {
      const float l = pkv_logf_portable(r[j]);
      float nrm = (l - mn) / span;
      nrm = nrm < 0.0f ? 0.0f : (nrm > 1.0f ? 1.0f : nrm);
      const uint32_t want = (uint32_t)roundf(nrm * 255.0f) & 0xffu;
      const double exact = log((double)r[j]);
      const double ulp = ldexp(1.0, ilogb(fabs(exact) > 1e-300 ? fabs(exact) : 1e-300) - 23);
      double e = 3.0 * ulp;
      if (e < 3.6e-7) e = 3.6e-7;
      for (int side = -1; side <= 1; side++) {
        int certain;
        const uint32_t got = pkv_fast_radius_code((float)(exact + side * e), mn, k, &certain);
        if (!certain) counts[1]++;
        else {
          counts[2]++;
          if (got != want) counts[0]++;
        }
      }
    }
  }
}

/* The fib encoder's shortcuts on n vectors (batch numerics): certified normalisation, binary32
 * fused rotation, certified block argmin -- against the exact sequence of fib_encode_one.
 * counts[0] = decided blocks with the wrong index, [1] = flagged blocks, [2] = decided blocks,
 * [3] = elements whose normalised value was declared certain but differs, [4] = uncertain elements,
 * [5] = largest |y~ - y| seen, in units of 1e-9. */
PKVO_API void pkvo_fib_fast_check(const float* x, int64_t n, int dim, const double* rot,
                                  const float* codebook, int n_codewords, int order, int64_t* counts) {
  const int blocks = dim / 4;
  float* m32 = (float*)malloc(sizeof(float) * (size_t)dim * dim);
  float hn[32];
  for (int i = 0; i < dim * dim; i++) m32[i] = (float)rot[i];
  for (int c = 0; c < n_codewords; c++) {
    double s = 0.0;
    for (int j = 0; j < 4; j++) s += (double)codebook[4 * c + j] * codebook[4 * c + j];
    hn[c] = (float)(0.5 * s);
  }
  for (int k = 0; k < 6; k++) counts[k] = 0;
  double worst = 0.0;
  for (int64_t v = 0; v < n; v++) {
    const float* xv = x + v * dim;
    double acc = 0.0;
    for (int i = 0; i < dim; i++) acc += (double)xv[i] * (double)xv[i];
    const double norm = sqrt(acc);
    if (!(norm > 0.0)) continue;
    const double inv = 1.0 / norm;
    const float invh = (float)inv, invl = (float)(inv - (double)invh);
    uint32_t min_key = 0xffffffffu;
    for (int i = 0; i < dim; i++) {
      const uint32_t k = pkv_fib_mag_key(xv[i]);
      if (k < min_key) min_key = k;
    }
    const int pair_ok = pkv_fib_fast_norm_ok(norm, min_key);
    float nf[512], ne[512];
    for (int i = 0; i < dim; i++) {
      uint32_t unsure = pair_ok ? 0u : 1u;
      nf[i] = pkv_fib_norm_quotient(xv[i], invh, invl, &unsure);
      ne[i] = (float)((double)xv[i] / norm);
      if (unsure) counts[4]++;
      else if (pkv_f32_bits(nf[i]) != pkv_f32_bits(ne[i])) counts[3]++;
    }
    for (int b = 0; b < blocks; b++) {
      float yf[4], ye[4];
      for (int rr = 0; rr < 4; rr++) {
        const int r = 4 * b + rr;
        float a = 0.0f;
        double s = 0.0;
        for (int j = 0; j < dim; j++) {
          a = __builtin_fmaf(m32[(size_t)r * dim + j], ne[j], a);
          s += rot[(size_t)r * dim + j] * (double)ne[j];
        }
        yf[rr] = a;
        ye[rr] = (float)s;
        const double e = fabs((double)a - (double)ye[rr]);
        if (e > worst) worst = e;
      }
      int certain = 0;
      float best = INFINITY, second = INFINITY;
      for (int c = 0; c < n_codewords; c++)
        pkv_fib_top2(&best, &second,
                     pkv_fib_key(yf[0], yf[1], yf[2], yf[3], codebook[4 * c], codebook[4 * c + 1],
                                 codebook[4 * c + 2], codebook[4 * c + 3], hn[c], (uint32_t)c));
      certain = pkv_fib_certify_eta(best, second, yf[0], yf[1], yf[2], yf[3], PKV_FIB_ROT_ERR_D(dim),
                                    pkv_fib_score_abs(codebook, n_codewords));
      const uint32_t fast = pkv_f32_bits(best) & 31u;
      if (!certain) {
        counts[1]++;
        continue;
      }
      counts[2]++;
      if ((int)fast != pkvo_nearest_codeword(ye, codebook, n_codewords, 4, order)) counts[0]++;
    }
  }
  counts[5] = (int64_t)(worst * 1e9);
  free(m32);
}

/* Stress of the pair-form normalised element (pkv_fast_paths.h (1)) against the division it stands
 * for.  mode 0: random x and norm with |x| <= norm.  mode m > 0: quotients placed next to binary32
 * rounding boundaries -- a random binary32 t in [2^-12, 1), the midpoint above it moved by k 2^-52
 * relative for a random |k| <= 2^m, and norm = |x| / midpoint, so that x / norm lands within 2^(m-52)
 * of the boundary.  counts[0] = declared certain but different from (f32)((f64)x / norm),
 * counts[1] = unsure, counts[2] = cases where the pair form was admissible. */
static uint64_t pkvo_mix64(uint64_t* st) {
  uint64_t z = (*st += 0x9e3779b97f4a7c15ull);
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

PKVO_API void pkvo_fib_quotient_check(uint64_t seed, int64_t n, int mode, int64_t* counts) {
  uint64_t st = seed;
  counts[0] = counts[1] = counts[2] = 0;
  for (int64_t it = 0; it < n; it++) {
    const uint64_t a = pkvo_mix64(&st), b = pkvo_mix64(&st);
    /* x: random sign, exponent in [-20, 20], random significand */
    const uint32_t xb = (uint32_t)(((a >> 63) << 31) | ((uint64_t)(107 + (a >> 32) % 41) << 23) | (a & 0x7fffffu));
    const float x = pkv_f32_from_bits(xb);
    double norm;
    if (mode == 0) {
      const double scale = 1.0 + (double)(b >> 11) * 0x1p-53 * 4095.0; /* |x| / norm in (2^-12, 1] */
      norm = fabs((double)x) * scale;
    } else {
      const uint32_t tb = (uint32_t)(((uint64_t)(115 + (b >> 40) % 12) << 23) | (b & 0x7fffffu));
      const float t = pkv_f32_from_bits(tb), tn = pkv_f32_from_bits(tb + 1u);
      const double mid = 0.5 * ((double)t + (double)tn);
      const int64_t span = 1ll << mode, k = (int64_t)((b >> 24) % (uint64_t)(2 * span + 1)) - span;
      norm = fabs((double)x) / (mid * (1.0 + (double)k * 0x1p-52));
    }
    const uint32_t key = pkv_fib_mag_key(x);
    if (!pkv_fib_fast_norm_ok(norm, key)) continue;
    counts[2]++;
    const double inv = 1.0 / norm;
    const float invh = (float)inv, invl = (float)(inv - (double)invh);
    uint32_t unsure = 0;
    const float q = pkv_fib_norm_quotient(x, invh, invl, &unsure);
    const float ref = (float)((double)x / norm);
    if (unsure) counts[1]++;
    else if (pkv_f32_bits(q) != pkv_f32_bits(ref)) counts[0]++;
  }
}

/* The score search on biased integer keys (pkv_fast_paths.h (3b)) for exactly known rotated blocks
 * (eta = 0, the Hadamard encoder): y holds n blocks of 4 values with |block| <= 1.  counts[0] = blocks
 * declared certain (by the key gap or by pkv_fib_certify_abs) whose index differs from the reference's
 * scan, counts[1] = undecided, counts[2] = certain, counts[3] = certain by the key gap alone,
 * counts[4] = scores that left the binade (must be 0). */
PKVO_API int pkvo_fib_biased_search_check(const float* y, int64_t n, const float* codebook, int n_codewords,
                                          int order, int64_t* counts) {
  float off, e_f, hn_off[32], nc[32][4];
  uint32_t quick_gap;
  for (int k = 0; k < 5; k++) counts[k] = 0;
  if (n_codewords > 32 || !pkv_fib_search_bias(codebook, n_codewords, 0.0, &off, &e_f, &quick_gap)) return 1;
  const uint32_t binade = pkv_f32_bits(off) & 0xff800000u;
  for (int c = 0; c < n_codewords; c++) {
    double s = 0.0;
    for (int j = 0; j < 4; j++) {
      s += (double)codebook[4 * c + j] * codebook[4 * c + j];
      nc[c][j] = -codebook[4 * c + j];
    }
    hn_off[c] = (float)(0.5 * s) + off; /* what the kernel forms: RN(RN(|c|^2 / 2) + off) */
  }
  for (int64_t v = 0; v < n; v++) {
    const float* s = y + 4 * v;
    uint32_t best = 0xffffffffu, second = 0xffffffffu;
    for (int c = 0; c < n_codewords; c++) {
      const uint32_t key = pkv_fib_biased_key(s[0], s[1], s[2], s[3], nc[c][0], nc[c][1], nc[c][2], nc[c][3],
                                              hn_off[c], (uint32_t)c);
      float f = __builtin_fmaf(s[0], nc[c][0], hn_off[c]);
      f = __builtin_fmaf(s[1], nc[c][1], f);
      f = __builtin_fmaf(s[2], nc[c][2], f);
      f = __builtin_fmaf(s[3], nc[c][3], f);
      if ((pkv_f32_bits(f) & 0xff800000u) != binade) counts[4]++;
      if (key < best) {
        second = best;
        best = key;
      } else if (key < second) {
        second = key;
      }
    }
    int certain = (second >> 5) - (best >> 5) > quick_gap;
    if (certain) counts[3]++;
    else
      certain = pkv_fib_certify_abs(pkv_fib_key_score(best, off), pkv_fib_key_score(second, off), s[0], s[1], s[2],
                                    s[3], 0.0f, e_f);
    if (!certain) {
      counts[1]++;
      continue;
    }
    counts[2]++;
    if ((int)(best & 31u) != pkvo_nearest_codeword(s, codebook, n_codewords, 4, order)) counts[0]++;
  }
  return 0;
}

/* The same check for the tensor-core rotation of the d = 64 encoder (PKV_FIB_ROT_ERR_TC). */
PKVO_API void pkvo_fib_tc_check(const float* x, int64_t n, int dim, const double* rot,
                                  const float* codebook, int n_codewords, int order, int64_t* counts) {
  const int blocks = dim / 4;
  float* m32 = (float*)malloc(sizeof(float) * (size_t)dim * dim);
  float hn[32];
  for (int i = 0; i < dim * dim; i++) m32[i] = (float)rot[i];
  for (int c = 0; c < n_codewords; c++) {
    double s = 0.0;
    for (int j = 0; j < 4; j++) s += (double)codebook[4 * c + j] * codebook[4 * c + j];
    hn[c] = (float)(0.5 * s);
  }
  for (int k = 0; k < 6; k++) counts[k] = 0;
  double worst = 0.0;
  for (int64_t v = 0; v < n; v++) {
    const float* xv = x + v * dim;
    double acc = 0.0;
    for (int i = 0; i < dim; i++) acc += (double)xv[i] * (double)xv[i];
    const double norm = sqrt(acc);
    if (!(norm > 0.0)) continue;
    const double inv = 1.0 / norm;
    const float invh = (float)inv, invl = (float)(inv - (double)invh);
    uint32_t min_key = 0xffffffffu;
    for (int i = 0; i < dim; i++) {
      const uint32_t k = pkv_fib_mag_key(xv[i]);
      if (k < min_key) min_key = k;
    }
    const int pair_ok = pkv_fib_fast_norm_ok(norm, min_key);
    float nf[512], ne[512];
    for (int i = 0; i < dim; i++) {
      uint32_t unsure = pair_ok ? 0u : 1u;
      nf[i] = pkv_fib_norm_quotient(xv[i], invh, invl, &unsure);
      ne[i] = (float)((double)xv[i] / norm);
      if (unsure) counts[4]++;
      else if (pkv_f32_bits(nf[i]) != pkv_f32_bits(ne[i])) counts[3]++;
    }
    for (int b = 0; b < blocks; b++) {
      float yf[4], ye[4];
      for (int rr = 0; rr < 4; rr++) {
        const int r = 4 * b + rr;
        /* n_lo M_hi, n_hi M_hi, n_hi M_lo with every operand cut to 11 significant bits, products
         * exact, partial sums of 8 terms added to a binary32 accumulator one after another */
        float a = 0.0f;
        double s = 0.0;
        for (int pass = 0; pass < 3; pass++)
          for (int j0 = 0; j0 < dim; j0 += 8) {
            double blk8 = 0.0;
            for (int j = j0; j < j0 + 8; j++) {
              const float m = m32[(size_t)r * dim + j], mh = tf32_cut(m, 0), ml = tf32_cut(m - mh, 0);
              const float nh = tf32_cut(ne[j], 0), nl = tf32_cut(ne[j] - nh, 0);
              blk8 += pass == 0 ? (double)nl * mh : pass == 1 ? (double)nh * mh : (double)nh * ml;
            }
            a = (float)((double)a + blk8);
          }
        for (int j = 0; j < dim; j++) s += rot[(size_t)r * dim + j] * (double)ne[j];
        yf[rr] = a;
        ye[rr] = (float)s;
        const double e = fabs((double)a - (double)ye[rr]);
        if (e > worst) worst = e;
      }
      int certain = 0;
      float best = INFINITY, second = INFINITY;
      for (int c = 0; c < n_codewords; c++)
        pkv_fib_top2(&best, &second,
                     pkv_fib_key(yf[0], yf[1], yf[2], yf[3], codebook[4 * c], codebook[4 * c + 1],
                                 codebook[4 * c + 2], codebook[4 * c + 3], hn[c], (uint32_t)c));
      certain = pkv_fib_certify_eta(best, second, yf[0], yf[1], yf[2], yf[3], PKV_FIB_ROT_ERR_TC_D(dim),
                                    pkv_fib_score_abs(codebook, n_codewords));
      const uint32_t fast = pkv_f32_bits(best) & 31u;
      if (!certain) {
        counts[1]++;
        continue;
      }
      counts[2]++;
      if ((int)fast != pkvo_nearest_codeword(ye, codebook, n_codewords, 4, order)) counts[0]++;
    }
  }
  counts[5] = (int64_t)(worst * 1e9);
  free(m32);
}
