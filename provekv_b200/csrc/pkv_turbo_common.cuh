// Pieces shared by the turbo-quant encode and decode kernels (pkv_turbo.cu).
//
// Work unit: one warp owns a tile of 32 vectors (one thread per vector) with its own slice of
// shared memory, so warps never wait for each other; a CTA's warps only share the read-only
// tables (QJL matrix, cos/sin and ray tables) loaded once at the start.
#pragma once

#include "pkv_common.cuh"
#include "pkv_fast_paths.h"

namespace pkv_turbo {

#define PKV_PI_F 3.14159274101257324f
#define PKV_TWO_PI_F 6.28318548202514648f
#define PKV_FLT_MIN 1.17549435e-38f
#define PKV_FLT_EPS 1.1920929e-07f

template <int D>
struct Turbo {
  static constexpr int NWARPS = D == 64 ? 4 : 2;  // warps (tiles in flight) per CTA
  static constexpr int THREADS = NWARPS * 32;
  static constexpr int TV = 32;      // vectors per warp tile
  static constexpr int XS = D + 4;   // f32 tile row stride (keeps float4 alignment)
  static constexpr int WS = TV + 1;  // word-transposed record tile row stride (odd: no bank conflicts)
  static constexpr int P = D / 2;
  static constexpr int LPV = D / 4;  // lanes per vector in the coalesced copies
};

struct TurboParams {
  int polar_bits, mode, projections, lossy;
  int radii_words, angle_words, sign_words, rec_words;
  float scale;
  uint32_t sign_mask[4];
  float sgn[128];        // the Rademacher signs as +-1.0f and as +-scale: constant-bank operands, so a
  float sgn_scale[128];  // sign flip costs one multiply (or none, merged with the 1/sqrt(d) scaling)
  float qjl_thr_tf32[64];  // per QJL row: |g| * PKV_QJL_TF32_BOUND (tensor-core tier)
  int fast_bucket;     // ray table present and validated against the exact thresholds
  int ray_count;       // 2^polar_bits / 4 + 1 rays, 0 without the shortcut
  int skip_issue;      // test hook: the tensor-core product is not issued, so its bounded wait runs out
  const float* qjl;    // [m][dim] then m sign-shortcut thresholds
  const float* qjl_rot;  // [m][dim]: rows of G S H~ scaled to unit length (the rotated-domain sketch)
  const float* lut;    // cos[L], sin[L], ray_cos[ray_count], ray_sin[ray_count]
  PkvUlpTable logf_table;  // BlockLogU8 radii with the host libm's logf / expf; keys null = portable functions
  PkvUlpTable expf_table;
};

// fwht_normalized, turbo-quant/src/rotation.rs:379-398: butterflies for
// step = 1, 2, 4, ... on pairs (i, i + step): (a, b) -> (a + b, a - b); then * scale.
template <int D>
__device__ __forceinline__ void fwht_regs(float (&v)[D], float scale) {
#pragma unroll
  for (int step = 1; step < D; step <<= 1) {
#pragma unroll
    for (int start = 0; start < D; start += 2 * step) {
#pragma unroll
      for (int o = 0; o < step; o++) {
        const float a = v[start + o], b = v[start + o + step];
        v[start + o] = __fadd_rn(a, b);
        v[start + o + step] = __fsub_rn(a, b);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < D; i++) v[i] = __fmul_rn(v[i], scale);
}

// Packed two-lane f32 add / subtract / multiply (sm_100): each lane is the IEEE operation of its
// own pair of inputs, so a butterfly on two adjacent coordinates costs one issue slot per output
// pair.  The pair (v[i], v[i + 1]) must sit in an aligned register pair; the arrays below are only
// ever touched in such pairs once past the first stage.  A packed multiply must not feed a packed
// add or subtract directly: the assembler contracts that pair into a fused multiply-add.
__device__ __forceinline__ void add_sub2(float& a0, float& a1, float& b0, float& b1) {
  unsigned long long pa, pb, ps, pd;
  asm("mov.b64 %0, {%1, %2};" : "=l"(pa) : "f"(a0), "f"(a1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(pb) : "f"(b0), "f"(b1));
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(ps) : "l"(pa), "l"(pb));
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(pd) : "l"(pa), "l"(pb));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(ps));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(b0), "=f"(b1) : "l"(pd));
}
__device__ __forceinline__ void mul2(float& a0, float& a1, float m0, float m1) {
  unsigned long long pa, pm, pr;
  asm("mov.b64 %0, {%1, %2};" : "=l"(pa) : "f"(a0), "f"(a1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(pm) : "f"(m0), "f"(m1));
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(pr) : "l"(pa), "l"(pm));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(pr));
}

// Forward rotation, FastHadamardRotation::apply (rotation.rs:202-210): signs, butterflies, scale.
// The sign multiplications are folded into the first butterfly stage: with a' = a * sa (exact),
// fma(b, sb, a') = RN(a' + sb b) and fma(b, -sb, a') = RN(a' - sb b) are the reference's rounded
// sum and difference of the two signed values.
template <int D>
__device__ __forceinline__ void fwht_forward_signed(float (&v)[D], const float (&sgn)[128], float scale) {
#pragma unroll
  for (int i = 0; i < D; i += 2) {
    const float a = __fmul_rn(v[i], sgn[i]), b = v[i + 1];
    v[i] = __fmaf_rn(b, sgn[i + 1], a);
    v[i + 1] = __fmaf_rn(b, -sgn[i + 1], a);
  }
#pragma unroll
  for (int step = 2; step < D; step <<= 1) {
#pragma unroll
    for (int start = 0; start < D; start += 2 * step) {
#pragma unroll
      for (int o = 0; o < step; o += 2) add_sub2(v[start + o], v[start + o + 1], v[start + o + step], v[start + o + step + 1]);
    }
  }
#pragma unroll
  for (int i = 0; i < D; i += 2) mul2(v[i], v[i + 1], scale, scale);
}

// Inverse rotation, FastHadamardRotation::apply_inverse (rotation.rs:212-221): butterflies, scale,
// signs.  RN(v * scale) * (+-1) = RN(v * (+-scale)): one multiply by the signed scale.
template <int D>
__device__ __forceinline__ void fwht_inverse_signed(float (&v)[D], const float (&sgn_scale)[128]) {
#pragma unroll
  for (int i = 0; i < D; i += 2) {
    const float a = v[i], b = v[i + 1];
    v[i] = __fadd_rn(a, b);
    v[i + 1] = __fsub_rn(a, b);
  }
#pragma unroll
  for (int step = 2; step < D; step <<= 1) {
#pragma unroll
    for (int start = 0; start < D; start += 2 * step) {
#pragma unroll
      for (int o = 0; o < step; o += 2) add_sub2(v[start + o], v[start + o + 1], v[start + o + step], v[start + o + step + 1]);
    }
  }
#pragma unroll
  for (int i = 0; i < D; i += 2) mul2(v[i], v[i + 1], sgn_scale[i], sgn_scale[i + 1]);
}

// value * sign with sign = +-1.0 is a sign-bit flip (also for zeros and NaNs).
template <int D>
__device__ __forceinline__ void apply_signs(float (&v)[D], const uint32_t (&mask)[4]) {
#pragma unroll
  for (int i = 0; i < D; i++)
    v[i] = __uint_as_float(__float_as_uint(v[i]) ^ ((mask[i >> 5] << (31 - (i & 31))) & 0x80000000u));
}

// encode_pair's bucket, turbo-quant/src/polar.rs:415-420
__device__ __forceinline__ uint32_t angle_bucket(float theta, uint32_t levels) {
  const float normalized = __fdiv_rn(__fadd_rn(theta, PKV_PI_F), PKV_TWO_PI_F);
  const float scaled = floorf(__fmul_rn(normalized, (float)levels));
  return ((uint32_t)scaled) & (levels - 1u);  // f32 -> u32 saturates like Rust's `as`
}

// The exact (slow) forms, kept out of line: taken only by undecided pairs / projections.
static __device__ __noinline__ uint32_t exact_bucket(float b, float a, uint32_t levels) {
  return angle_bucket(pkv_atan2f_portable(b, a), levels);
}

// QjlQuantizer::sketch's dot (qjl.rs:214-217): sequential, separately rounded * and +.
// `res` is the thread's residual vector in shared memory (its row of the f32 tile).
static __device__ __noinline__ float exact_dot(const float* g, const float* res, int dim) {
  float dot = 0.0f;
  for (int j = 0; j < dim; j++) dot = __fadd_rn(dot, __fmul_rn(g[j], res[j]));
  return dot;
}

// Packed two-lane f32 fused multiply-add (one issue slot for two FMAs on sm_100).
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  unsigned long long ra, rb, rc, rd;
  ra = *reinterpret_cast<unsigned long long*>(&a);
  rb = *reinterpret_cast<unsigned long long*>(&b);
  rc = *reinterpret_cast<unsigned long long*>(&c);
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
  return *reinterpret_cast<float2*>(&rd);
}

// A warp's records between global memory (vector-major words) and its shared tile
// ([word][vector]).  Word i of the tile belongs to vector i / rec_words; (v, k) is advanced
// incrementally so the loop has no division.  Loads are asynchronous (caller waits).
template <int D, bool IN>
__device__ __forceinline__ void stage_records(uint32_t* s_w, uint32_t* g, int nv, int rec_words,
                                              int lane) {
  using K = Turbo<D>;
  const int total = nv * rec_words;
  int i = lane;
  int v = i / rec_words, k = i - v * rec_words;
  const int dv = 32 / rec_words, dk = 32 - dv * rec_words;
  for (; i < total; i += 32) {
    if (IN) pkv_cp_async4(s_w + k * K::WS + v, g + i);
    else g[i] = s_w[k * K::WS + v];
    v += dv;
    k += dk;
    if (k >= rec_words) {
      k -= rec_words;
      v++;
    }
  }
}

}  // namespace pkv_turbo
