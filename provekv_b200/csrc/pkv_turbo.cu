// turbo-quant hot-shell kernels for sm_100a: randomised Hadamard transform
// (Rademacher signs, FWHT held in registers), polar decomposition with b-bit
// angle buckets, f32 or BlockLogU8 radii, optional QJL residual sign sketch,
// and the inverse fused with the write into the KV cache.
//
// One thread owns one vector; a CTA stages TV vectors (f32 tile, padded rows)
// and TV records (word-transposed, so record word k of vector v sits at
// [k][v]) through shared memory so that every global access is coalesced.
//
// Arithmetic follows the reference operation by operation:
//  encode  turbo-quant/src/turbo.rs:256-288, polar.rs:246-266,413-421,
//          rotation.rs:202-221,379-398, qjl.rs:203-220, radius.rs:58-77,
//          bitpack.rs:21-62, wire.rs:350-396
//  decode  turbo-quant/src/wire.rs:497-565, radius.rs:81-147, polar.rs:286-316,
//          rotation.rs:170-194
// atan2f / logf / expf are the portable definitions of pkv_portable_math.h.
#include "pkv_common.cuh"

namespace {

#define PKV_PI_F 3.14159274101257324f
#define PKV_TWO_PI_F 6.28318548202514648f
#define PKV_FLT_MIN 1.17549435e-38f
#define PKV_FLT_EPS 1.1920929e-07f

template <int D>
struct Turbo {
  static constexpr int TV = D == 64 ? 128 : 64;
  static constexpr int XS = D + 4;   // f32 tile row stride (keeps float4 alignment)
  static constexpr int WS = TV + 1;  // word-transposed record tile row stride
  static constexpr int P = D / 2;
};

struct TurboParams {
  int polar_bits, mode, projections, lossy;
  int radii_words, angle_words, sign_words, rec_words;
  float scale;
  uint32_t sign_mask[4];
  const float* qjl;
  const float* lut;
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

// value * sign with sign = +-1.0 is a sign-bit flip (also for zeros and NaNs).
template <int D>
__device__ __forceinline__ void apply_signs(float (&v)[D], const uint32_t (&mask)[4]) {
#pragma unroll
  for (int i = 0; i < D; i++)
    v[i] = __uint_as_float(__float_as_uint(v[i]) ^ (((mask[i >> 5] >> (i & 31)) & 1u) << 31));
}

// encode_pair's bucket, turbo-quant/src/polar.rs:415-420
__device__ __forceinline__ uint32_t angle_bucket(float theta, uint32_t levels) {
  const float normalized = __fdiv_rn(__fadd_rn(theta, PKV_PI_F), PKV_TWO_PI_F);
  const float scaled = floorf(__fmul_rn(normalized, (float)levels));
  return ((uint32_t)scaled) & (levels - 1u);  // f32 -> u32 saturates like Rust's `as`
}

template <int D>
__device__ __forceinline__ void stage_records_in(uint32_t* s_w, const uint8_t* src, int nv,
                                                 int rec_words) {
  using K = Turbo<D>;
  const uint32_t* g = reinterpret_cast<const uint32_t*>(src);
  const int total = nv * rec_words;
  for (int i = threadIdx.x; i < total; i += K::TV) {
    const int v = i / rec_words, k = i - v * rec_words;
    s_w[k * K::WS + v] = __ldg(g + i);
  }
}

template <int D>
__device__ __forceinline__ void stage_records_out(uint8_t* dst, const uint32_t* s_w, int nv,
                                                  int rec_words) {
  using K = Turbo<D>;
  uint32_t* g = reinterpret_cast<uint32_t*>(dst);
  const int total = nv * rec_words;
  for (int i = threadIdx.x; i < total; i += K::TV) {
    const int v = i / rec_words, k = i - v * rec_words;
    g[i] = s_w[k * K::WS + v];
  }
}

// ---------------------------------------------------------------------------
// decode + patch
// ---------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(Turbo<D>::TV)
turbo_decode_patch_kernel(PkvGeom g, TurboParams tp, const uint8_t* __restrict__ payload,
                          float* __restrict__ cache, uint64_t* err) {
  using K = Turbo<D>;
  extern __shared__ __align__(16) uint8_t smem[];
  float* s_x = reinterpret_cast<float*>(smem);                       // [TV][XS]
  int64_t* s_off = reinterpret_cast<int64_t*>(s_x + K::TV * K::XS);  // [TV]
  float* s_q255 = reinterpret_cast<float*>(s_off + K::TV);           // [256]
  float* s_lut = s_q255 + 256;                                       // [2][levels]
  const int levels = 1 << tp.polar_bits;
  uint32_t* s_w = reinterpret_cast<uint32_t*>(s_lut + 2 * levels);   // [rec_words][WS]

  const int tile = blockIdx.x % g.tiles_per_batch;
  const int batch = blockIdx.x / g.tiles_per_batch;
  const int v0 = tile * K::TV;
  const int nv = min(K::TV, g.vpb - v0);
  const int v = threadIdx.x;

  stage_records_in<D>(s_w, payload + (int64_t)batch * g.payload_batch_stride +
                               (int64_t)v0 * g.rec_bytes, nv, tp.rec_words);
  for (int i = threadIdx.x; i < 2 * levels; i += K::TV) s_lut[i] = __ldg(tp.lut + i);
  if (tp.lossy)  // `*value as f32 / u8::MAX as f32`, radius.rs:143
    for (int i = threadIdx.x; i < 256; i += K::TV) s_q255[i] = __fdiv_rn((float)i, 255.0f);
  __syncthreads();

  if (v < nv) {
    const int64_t gvec = (int64_t)batch * g.vpb + v0 + v;
    s_off[v] = pkv_vec_offset(g.L, batch, v0 + v);
    const uint32_t* w = s_w + v;
    int code = 0;
    float y[D];
    // radii -> y[2i] (temporarily)
    if (!tp.lossy) {
#pragma unroll
      for (int i = 0; i < K::P; i++) {
        const float r = __uint_as_float(w[i * K::WS]);
        if (!code && (!pkv_finite(r) || r < 0.0f)) code = PKV_VEC_BAD_RADIUS;  // radius.rs:98-103
        y[2 * i] = r;
      }
    } else {
      const float mn = __uint_as_float(w[(K::P / 4) * K::WS]);
      const float mx = __uint_as_float(w[(K::P / 4 + 1) * K::WS]);
      if (!pkv_finite(mn) || !pkv_finite(mx) || mn > mx) code = PKV_VEC_BAD_RADIUS_RANGE;
      const float span = __fsub_rn(mx, mn);
#pragma unroll
      for (int k = 0; k < K::P / 4; k++) {
        const uint32_t q4 = w[k * K::WS];
#pragma unroll
        for (int b = 0; b < 4; b++) {
          const float t = __fadd_rn(mn, __fmul_rn(span, s_q255[(q4 >> (8 * b)) & 0xffu]));
          const float r = code ? 0.0f : pkv_expf_portable(t);
          if (!code && !pkv_finite(r)) code = PKV_VEC_BAD_RADIUS;  // polar.rs:127-133
          y[2 * (4 * k + b)] = r;
        }
      }
    }
    // angles (LSB-first stream of polar_bits-wide values) and the polar -> cartesian step
    {
      const uint32_t* aw = w + tp.radii_words * K::WS;
      uint64_t bitbuf = 0;
      int nbits = 0, wk = 0;
      const uint32_t mask = (uint32_t)levels - 1u;
#pragma unroll
      for (int i = 0; i < K::P; i++) {
        if (nbits < tp.polar_bits) {
          bitbuf |= (uint64_t)aw[wk * K::WS] << nbits;
          wk++;
          nbits += 32;
        }
        const uint32_t idx = (uint32_t)bitbuf & mask;
        bitbuf >>= tp.polar_bits;
        nbits -= tp.polar_bits;
        const float r = y[2 * i];
        y[2 * i] = __fmul_rn(r, s_lut[idx]);               // r * theta.cos(), polar.rs:312
        y[2 * i + 1] = __fmul_rn(r, s_lut[levels + idx]);  // r * theta.sin(), polar.rs:313
      }
    }
    if (code) pkv_report(err, 0, gvec, code);
    // FastHadamardRotation::apply_inverse, rotation.rs:212-221
    fwht_regs<D>(y, tp.scale);
    apply_signs<D>(y, tp.sign_mask);
    float* row = s_x + v * K::XS;
#pragma unroll
    for (int i = 0; i < D; i += 4)
      *reinterpret_cast<float4*>(row + i) = make_float4(y[i], y[i + 1], y[i + 2], y[i + 3]);
  }
  __syncthreads();

  // coalesced write-out: D/4 lanes per vector, one float4 each, every replica
  constexpr int LPV = D / 4;
  for (int i = threadIdx.x; i < nv * LPV; i += K::TV) {
    const int vv = i / LPV, q = i % LPV;
    const float4 val = *reinterpret_cast<const float4*>(s_x + vv * K::XS + 4 * q);
    float* dst = cache + s_off[vv] + 4 * q;
    for (int r = 0; r < g.L.n_replicas; r++) {
      *reinterpret_cast<float4*>(dst) = val;
      dst += g.L.replica_stride;
    }
  }
}

template <int D>
size_t turbo_decode_smem(const TurboParams& tp) {
  using K = Turbo<D>;
  return sizeof(float) * K::TV * K::XS + sizeof(int64_t) * K::TV + sizeof(float) * 256 +
         sizeof(float) * 2 * (1 << tp.polar_bits) + sizeof(uint32_t) * tp.rec_words * K::WS;
}


// ---------------------------------------------------------------------------
// encode
// ---------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(Turbo<D>::TV)
turbo_encode_kernel(PkvGeom g, TurboParams tp, const float* __restrict__ x,
                    uint8_t* __restrict__ payload, uint64_t* err) {
  using K = Turbo<D>;
  extern __shared__ __align__(16) uint8_t smem[];
  float* s_x = reinterpret_cast<float*>(smem);                 // [TV][XS]
  float* s_g = s_x + K::TV * K::XS;                            // [m][D]
  const int levels = 1 << tp.polar_bits;
  float* s_lut = s_g + tp.projections * D;                     // [2][levels]
  uint32_t* s_w = reinterpret_cast<uint32_t*>(s_lut + 2 * levels);  // [rec_words][WS]
  float* s_rad = reinterpret_cast<float*>(s_w + tp.rec_words * K::WS);  // [P][WS], lossy only

  const int tile = blockIdx.x % g.tiles_per_batch;
  const int batch = blockIdx.x / g.tiles_per_batch;
  const int v0 = tile * K::TV;
  const int nv = min(K::TV, g.vpb - v0);
  const int v = threadIdx.x;

  constexpr int LPV = D / 4;
  for (int i = threadIdx.x; i < nv * LPV; i += K::TV) {
    const int vv = i / LPV, q = i % LPV;
    *reinterpret_cast<float4*>(s_x + vv * K::XS + 4 * q) =
        __ldg(reinterpret_cast<const float4*>(x + pkv_vec_offset(g.L, batch, v0 + vv)) + q);
  }
  for (int i = threadIdx.x; i < tp.projections * D / 4; i += K::TV)
    reinterpret_cast<float4*>(s_g)[i] = __ldg(reinterpret_cast<const float4*>(tp.qjl) + i);
  for (int i = threadIdx.x; i < 2 * levels; i += K::TV) s_lut[i] = __ldg(tp.lut + i);
  __syncthreads();

  if (v < nv) {
    const int64_t gvec = (int64_t)batch * g.vpb + v0 + v;
    const float* row = s_x + v * K::XS;
    uint32_t* w = s_w + v;
    int code = 0;
    float y[D];
    bool finite = true;
#pragma unroll
    for (int i = 0; i < D; i += 4) {
      const float4 t = *reinterpret_cast<const float4*>(row + i);
      y[i] = t.x; y[i + 1] = t.y; y[i + 2] = t.z; y[i + 3] = t.w;
      finite = finite && pkv_finite(t.x) && pkv_finite(t.y) && pkv_finite(t.z) && pkv_finite(t.w);
    }
    if (!finite) code = PKV_VEC_NONFINITE_INPUT;  // turbo.rs:263
    // FastHadamardRotation::apply, rotation.rs:202-210
    apply_signs<D>(y, tp.sign_mask);
    fwht_regs<D>(y, tp.scale);
    // encode_pair per pair (polar.rs:413-421); radii to the record (f32) or to s_rad (lossy);
    // y is overwritten with the de-quantised pair for the residual step.
    float* radp = tp.lossy ? (s_rad + v) : reinterpret_cast<float*>(w);
    {
      uint32_t* aw = w + tp.radii_words * K::WS;
      uint64_t bitbuf = 0;
      int nbits = 0, wk = 0;
      bool rad_ok = true;
#pragma unroll
      for (int i = 0; i < K::P; i++) {
        const float a = y[2 * i], b = y[2 * i + 1];
        const float r = __fsqrt_rn(__fadd_rn(__fmul_rn(a, a), __fmul_rn(b, b)));
        const uint32_t idx = angle_bucket(pkv_atan2f_portable(b, a), (uint32_t)levels);
        rad_ok = rad_ok && pkv_finite(r);
        radp[i * K::WS] = r;
        bitbuf |= (uint64_t)idx << nbits;
        nbits += tp.polar_bits;
        if (nbits >= 32) {
          aw[wk * K::WS] = (uint32_t)bitbuf;
          wk++;
          bitbuf >>= 32;
          nbits -= 32;
        }
        y[2 * i] = __fmul_rn(r, s_lut[idx]);
        y[2 * i + 1] = __fmul_rn(r, s_lut[levels + idx]);
      }
      if (nbits > 0) aw[wk * K::WS] = (uint32_t)bitbuf;
      if (!code && !rad_ok) code = PKV_VEC_BAD_RADIUS;  // PolarCode::from_parts, polar.rs:127-133
    }
    if (tp.mode == PKV_TURBO_POLAR_WITH_QJL) {
      // polar.decode (polar.rs:272-278) then residual = vector - reconstruction (turbo.rs:268-273)
      fwht_regs<D>(y, tp.scale);
      apply_signs<D>(y, tp.sign_mask);
      bool res_ok = true;
#pragma unroll
      for (int i = 0; i < D; i += 4) {
        const float4 t = *reinterpret_cast<const float4*>(row + i);
        y[i] = __fsub_rn(t.x, y[i]);
        y[i + 1] = __fsub_rn(t.y, y[i + 1]);
        y[i + 2] = __fsub_rn(t.z, y[i + 2]);
        y[i + 3] = __fsub_rn(t.w, y[i + 3]);
        res_ok = res_ok && pkv_finite(y[i]) && pkv_finite(y[i + 1]) && pkv_finite(y[i + 2]) &&
                 pkv_finite(y[i + 3]);
      }
      if (!code && !res_ok) code = PKV_VEC_NONFINITE_RESIDUAL;  // qjl.rs:210
      // QjlQuantizer::sketch, qjl.rs:214-217: sequential f32 dot per row, sign = dot >= 0
      uint32_t* sw = w + (tp.radii_words + tp.angle_words) * K::WS;
      uint32_t bits = 0;
#pragma unroll 1
      for (int p = 0; p < tp.projections; p++) {
        const float* grow = s_g + p * D;
        float dot = 0.0f;
#pragma unroll
        for (int j = 0; j < D; j += 4) {
          const float4 gg = *reinterpret_cast<const float4*>(grow + j);
          dot = __fadd_rn(dot, __fmul_rn(gg.x, y[j]));
          dot = __fadd_rn(dot, __fmul_rn(gg.y, y[j + 1]));
          dot = __fadd_rn(dot, __fmul_rn(gg.z, y[j + 2]));
          dot = __fadd_rn(dot, __fmul_rn(gg.w, y[j + 3]));
        }
        bits |= (dot >= 0.0f ? 1u : 0u) << (p & 31);
        if ((p & 31) == 31) {
          sw[(p >> 5) * K::WS] = bits;
          bits = 0;
        }
      }
    }
    if (tp.lossy) {
      // CompressedRadiiV1::compress, BlockLogU8 (radius.rs:58-77), min/max after the bytes (wire.rs:368-371)
      float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
#pragma unroll 4
      for (int i = 0; i < K::P; i++) {
        float r = s_rad[i * K::WS + v];
        r = (code || !(r > PKV_FLT_MIN)) ? PKV_FLT_MIN : r;
        const float l = pkv_logf_portable(r);
        s_rad[i * K::WS + v] = l;
        mn = l < mn ? l : mn;
        mx = l > mx ? l : mx;
      }
      float span = __fsub_rn(mx, mn);
      if (!(span > PKV_FLT_EPS)) span = PKV_FLT_EPS;
#pragma unroll 2
      for (int k = 0; k < K::P / 4; k++) {
        uint32_t q4 = 0;
#pragma unroll
        for (int b = 0; b < 4; b++) {
          float nrm = __fdiv_rn(__fsub_rn(s_rad[(4 * k + b) * K::WS + v], mn), span);
          nrm = nrm < 0.0f ? 0.0f : (nrm > 1.0f ? 1.0f : nrm);
          q4 |= ((uint32_t)roundf(__fmul_rn(nrm, 255.0f)) & 0xffu) << (8 * b);
        }
        w[k * K::WS] = q4;
      }
      w[(K::P / 4) * K::WS] = __float_as_uint(mn);
      w[(K::P / 4 + 1) * K::WS] = __float_as_uint(mx);
    }
    if (code) pkv_report(err, 0, gvec, code);
  }
  __syncthreads();
  stage_records_out<D>(payload + (int64_t)batch * g.payload_batch_stride + (int64_t)v0 * g.rec_bytes,
                       s_w, nv, tp.rec_words);
}

template <int D>
size_t turbo_encode_smem(const TurboParams& tp) {
  using K = Turbo<D>;
  return sizeof(float) * K::TV * K::XS + sizeof(float) * tp.projections * D +
         sizeof(float) * 2 * (1 << tp.polar_bits) + sizeof(uint32_t) * tp.rec_words * K::WS +
         (tp.lossy ? sizeof(float) * K::P * K::WS : 0);
}

TurboParams make_params(const pkv_turbo_profile* p) {
  TurboParams tp;
  tp.polar_bits = p->polar_bits;
  tp.mode = p->cfg.mode;
  tp.projections = p->cfg.mode == PKV_TURBO_POLAR_WITH_QJL ? p->cfg.projections : 0;
  tp.lossy = p->cfg.radii_codec == PKV_RADII_BLOCK_LOG_U8;
  tp.radii_words = p->radii_words;
  tp.angle_words = p->angle_words;
  tp.sign_words = p->sign_words;
  tp.rec_words = p->rec_bytes / 4;
  tp.scale = p->scale;
  for (int i = 0; i < 4; i++) tp.sign_mask[i] = p->sign_mask[i];
  tp.qjl = p->qjl_dev;
  tp.lut = p->lut_dev;
  return tp;
}

template <typename F>
int set_smem(F kernel, size_t bytes) {
  if (bytes > 48 * 1024)
    return pkv_cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return PKV_OK;
}

}  // namespace

int pkv_turbo_tile_vectors(int dim) { return dim == 64 ? Turbo<64>::TV : dim == 128 ? Turbo<128>::TV : 0; }

int pkv_launch_turbo_encode(const pkv_turbo_profile* p, const float* x, const PkvGeom& g,
                            uint8_t* payload, uint64_t* err, cudaStream_t s) {
  const int64_t grid = (int64_t)g.n_batches * g.tiles_per_batch;
  if (grid == 0) return PKV_OK;
  if (grid > 0x7fffffff) return PKV_ERR_UNSUPPORTED;
  const TurboParams tp = make_params(p);
  int st;
#define PKV_TURBO_ENC(DIM)                                                              \
  {                                                                                     \
    const size_t sm = turbo_encode_smem<DIM>(tp);                                       \
    if ((st = set_smem(turbo_encode_kernel<DIM>, sm)) != PKV_OK) return st;             \
    turbo_encode_kernel<DIM><<<(unsigned)grid, Turbo<DIM>::TV, sm, s>>>(g, tp, x, payload, err); \
  }
  if (p->cfg.dim == 64) PKV_TURBO_ENC(64)
  else if (p->cfg.dim == 128) PKV_TURBO_ENC(128)
  else return PKV_ERR_UNSUPPORTED;
#undef PKV_TURBO_ENC
  pkv_count_launch();
  return pkv_cuda_status(cudaGetLastError());
}

int pkv_launch_turbo_decode(const pkv_turbo_profile* p, const uint8_t* payload, const PkvGeom& g,
                            float* cache, uint64_t* err, cudaStream_t s) {
  const int64_t grid = (int64_t)g.n_batches * g.tiles_per_batch;
  if (grid == 0) return PKV_OK;
  if (grid > 0x7fffffff) return PKV_ERR_UNSUPPORTED;
  const TurboParams tp = make_params(p);
  int st;
#define PKV_TURBO_DEC(DIM)                                                              \
  {                                                                                     \
    const size_t sm = turbo_decode_smem<DIM>(tp);                                       \
    if ((st = set_smem(turbo_decode_patch_kernel<DIM>, sm)) != PKV_OK) return st;       \
    turbo_decode_patch_kernel<DIM><<<(unsigned)grid, Turbo<DIM>::TV, sm, s>>>(g, tp, payload, cache, err); \
  }
  if (p->cfg.dim == 64) PKV_TURBO_DEC(64)
  else if (p->cfg.dim == 128) PKV_TURBO_DEC(128)
  else return PKV_ERR_UNSUPPORTED;
#undef PKV_TURBO_DEC
  pkv_count_launch();
  return pkv_cuda_status(cudaGetLastError());
}
