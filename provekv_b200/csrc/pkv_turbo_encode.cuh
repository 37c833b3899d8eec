// turbo-quant encode: one thread per vector.
//  turbo-quant/src/turbo.rs:256-288, polar.rs:246-266,413-421, rotation.rs:202-221,379-398,
//  qjl.rs:203-220, radius.rs:58-77, bitpack.rs:21-62, wire.rs:350-396
//
// The per-pair and per-projection work is written as straight-line unrolled passes without
// calls or data-dependent branches, so the compiler can interleave independent pairs; the
// decisions a shortcut could not certify are collected in bit masks and settled afterwards
// by two out-of-line routines that run the exact operation sequence.
#pragma once

#include "pkv_turbo_common.cuh"

namespace pkv_turbo {

// Replace angle index i in the shared angle words (LSB-first stream, bitpack.rs:135-143).
__device__ __forceinline__ void patch_angle(uint32_t* aw, int ws, int i, int pb, uint32_t idx) {
  const int pos = i * pb, wi = pos >> 5, sh = pos & 31;
  const uint32_t m = (1u << pb) - 1u;
  aw[wi * ws] = (aw[wi * ws] & ~(m << sh)) | (idx << sh);
  if (sh + pb > 32) {
    const int s2 = 32 - sh;
    aw[(wi + 1) * ws] = (aw[(wi + 1) * ws] & ~(m >> s2)) | (idx >> s2);
  }
}

// Exact angle buckets for the pairs in `unc`: the rotated vector is rebuilt in local memory
// with the reference's operation order (signs, butterflies step = 1, 2, 4, ..., scale), then
// each pending pair takes atan2f + the bucket expression of polar.rs:415-420.
__device__ __noinline__ void fix_pairs(const float* xrow, int dim, const uint32_t* sign_mask,
                                       float scale, unsigned long long unc, uint32_t* aw, int ws,
                                       int pb) {
  float t[PKV_MAX_DIM];
  for (int i = 0; i < dim; i++)
    t[i] = __uint_as_float(__float_as_uint(xrow[i]) ^ (((sign_mask[i >> 5] >> (i & 31)) & 1u) << 31));
  for (int step = 1; step < dim; step <<= 1)
    for (int start = 0; start < dim; start += 2 * step)
      for (int o = 0; o < step; o++) {
        const float a = t[start + o], b = t[start + o + step];
        t[start + o] = __fadd_rn(a, b);
        t[start + o + step] = __fsub_rn(a, b);
      }
  while (unc) {
    const int i = __ffsll((long long)unc) - 1;
    unc &= unc - 1;
    const float a = __fmul_rn(t[2 * i], scale), b = __fmul_rn(t[2 * i + 1], scale);
    patch_angle(aw, ws, i, pb, exact_bucket(b, a, 1u << pb));
  }
}

// Exact QJL signs for the projections in `unc` (qjl.rs:214-217); `res` is the residual row.
__device__ __noinline__ void fix_signs(const float* g, const float* res, int dim,
                                       unsigned long long unc, uint32_t* sw, int ws) {
  while (unc) {
    const int p = __ffsll((long long)unc) - 1;
    unc &= unc - 1;
    const float dot = exact_dot(g + p * dim, res, dim);
    const uint32_t bit = 1u << (p & 31);
    uint32_t w = sw[(p >> 5) * ws];
    w = dot >= 0.0f ? (w | bit) : (w & ~bit);
    sw[(p >> 5) * ws] = w;
  }
}

template <int D, int PB>
__global__ void __launch_bounds__(Turbo<D>::TV)
turbo_encode_kernel(PkvGeom g, TurboParams tp, const float* __restrict__ x,
                    uint8_t* __restrict__ payload, uint64_t* err) {
  using K = Turbo<D>;
  extern __shared__ __align__(16) uint8_t smem[];
  float* s_x = reinterpret_cast<float*>(smem);                 // [TV][XS]
  float* s_g = s_x + K::TV * K::XS;                            // [m][D]
  float* s_thr = s_g + tp.projections * D;                     // [m] sign-shortcut thresholds
  float* s_lut = s_thr + tp.projections;                       // cos, sin, ray_cos, ray_sin
  const int pb = PB ? PB : tp.polar_bits;
  const int levels = 1 << pb;
  const int lut_len = 2 * levels + 2 * tp.ray_count;
  const float* s_ray_cos = s_lut + 2 * levels;
  const float* s_ray_sin = s_ray_cos + tp.ray_count;
  uint32_t* s_w = reinterpret_cast<uint32_t*>(s_lut + lut_len);          // [rec_words][WS]
  float* s_rad = reinterpret_cast<float*>(s_w + tp.rec_words * K::WS);   // [P][WS], lossy only
  int64_t* s_off = reinterpret_cast<int64_t*>(
      s_rad + (tp.lossy ? K::P * K::WS : 0) + ((tp.rec_words * K::WS) & 1));  // 8-byte aligned

  const int tile = blockIdx.x % g.tiles_per_batch;
  const int batch = blockIdx.x / g.tiles_per_batch;
  const int v0 = tile * K::TV;
  const int nv = min(K::TV, g.vpb - v0);
  const int v = threadIdx.x;

  if (v < nv) s_off[v] = pkv_vec_offset(g.L, batch, v0 + v);
  for (int i = threadIdx.x; i < tp.projections * (D + 1) / 4; i += K::TV)
    pkv_cp_async16(reinterpret_cast<float4*>(s_g) + i, reinterpret_cast<const float4*>(tp.qjl) + i);
  for (int i = threadIdx.x; i < lut_len; i += K::TV) pkv_cp_async4(s_lut + i, tp.lut + i);
  __syncthreads();
  for (int i = threadIdx.x; i < nv * K::LPV; i += K::TV) {
    const int vv = i / K::LPV, q = i % K::LPV;
    pkv_cp_async16(s_x + vv * K::XS + 4 * q, reinterpret_cast<const float4*>(x + s_off[vv]) + q);
  }
  pkv_cp_async_wait_all();
  __syncthreads();

  if (v < nv) {
    float* row = s_x + v * K::XS;
    uint32_t* w = s_w + v;
    uint32_t* aw = w + tp.radii_words * K::WS;
    int code = 0;
    float y[D];
#pragma unroll
    for (int i = 0; i < D; i += 4) {
      const float4 t = *reinterpret_cast<const float4*>(row + i);
      y[i] = t.x; y[i + 1] = t.y; y[i + 2] = t.z; y[i + 3] = t.w;
    }
    bool finite = true;
#pragma unroll
    for (int i = 0; i < D; i++) finite = finite && pkv_finite(y[i]);
    if (!finite) code = PKV_VEC_NONFINITE_INPUT;  // turbo.rs:263
    // FastHadamardRotation::apply, rotation.rs:202-210
    apply_signs<D>(y, tp.sign_mask);
    fwht_regs<D>(y, tp.scale);

    // Pass 1, encode_pair (polar.rs:413-421): radius exactly, bucket by the shortcut.  Radii go
    // to the record (f32 codec) or to s_rad (BlockLogU8); undecided pairs are noted in `unc`.
    float* radp = tp.lossy ? (s_rad + v) : reinterpret_cast<float*>(w);
    constexpr int NW = PB ? K::P * PB / 32 : 1;
    unsigned long long unc = 0;
    {
      uint32_t words[NW];
#pragma unroll
      for (int k = 0; k < NW; k++) words[k] = 0;
      uint64_t bitbuf = 0;
      int nbits = 0, wk = 0;
      bool rad_ok = true;
#pragma unroll
      for (int i = 0; i < K::P; i++) {
        const float a = y[2 * i], b = y[2 * i + 1];
        const float r = __fsqrt_rn(__fadd_rn(__fmul_rn(a, a), __fmul_rn(b, b)));
        int certain = 0;
        uint32_t idx = 0;
        if (tp.fast_bucket) idx = pkv_fast_bucket(a, b, pb, s_ray_cos, s_ray_sin, &certain);
        unc |= (unsigned long long)(certain ? 0u : 1u) << i;
        rad_ok = rad_ok && pkv_finite(r);
        radp[i * K::WS] = r;
        if constexpr (PB != 0) {
          const int pos = i * PB, wi = pos >> 5, sh = pos & 31;
          words[wi] |= idx << sh;
          if (sh + PB > 32) words[wi + 1] |= idx >> (32 - sh);
        } else {
          bitbuf |= (uint64_t)idx << nbits;
          nbits += pb;
          if (nbits >= 32) {
            aw[wk * K::WS] = (uint32_t)bitbuf;
            wk++;
            bitbuf >>= 32;
            nbits -= 32;
          }
        }
      }
      if constexpr (PB != 0) {
#pragma unroll
        for (int k = 0; k < NW; k++) aw[k * K::WS] = words[k];
      } else if (nbits > 0) {
        aw[wk * K::WS] = (uint32_t)bitbuf;
      }
      if (!code && !rad_ok) code = PKV_VEC_BAD_RADIUS;  // PolarCode::from_parts, polar.rs:127-133
    }
    if (unc) fix_pairs(row, D, tp.sign_mask, tp.scale, unc, aw, K::WS, pb);

    if (tp.mode == PKV_TURBO_POLAR_WITH_QJL) {
      // polar.decode (polar.rs:272-278,306-316): de-quantised pairs from the final indices
      {
        const uint32_t mask = (uint32_t)levels - 1u;
        uint32_t words[NW];
        uint64_t bitbuf = 0;
        int nbits = 0, wk = 0;
        if constexpr (PB != 0) {
#pragma unroll
          for (int k = 0; k < NW; k++) words[k] = aw[k * K::WS];
        }
#pragma unroll
        for (int i = 0; i < K::P; i++) {
          uint32_t idx;
          if constexpr (PB != 0) {
            const int pos = i * PB, wi = pos >> 5, sh = pos & 31;
            idx = words[wi] >> sh;
            if (sh + PB > 32) idx |= words[wi + 1] << (32 - sh);
            idx &= mask;
          } else {
            if (nbits < pb) {
              bitbuf |= (uint64_t)aw[wk * K::WS] << nbits;
              wk++;
              nbits += 32;
            }
            idx = (uint32_t)bitbuf & mask;
            bitbuf >>= pb;
            nbits -= pb;
          }
          const float r = radp[i * K::WS];
          y[2 * i] = __fmul_rn(r, s_lut[idx]);
          y[2 * i + 1] = __fmul_rn(r, s_lut[levels + idx]);
        }
      }
      // inverse rotation (rotation.rs:212-221), residual = vector - reconstruction (turbo.rs:268-273)
      fwht_regs<D>(y, tp.scale);
      apply_signs<D>(y, tp.sign_mask);
      bool res_ok = true;
      float2 n2 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int i = 0; i < D; i += 4) {
        const float4 t = *reinterpret_cast<const float4*>(row + i);
        y[i] = __fsub_rn(t.x, y[i]);
        y[i + 1] = __fsub_rn(t.y, y[i + 1]);
        y[i + 2] = __fsub_rn(t.z, y[i + 2]);
        y[i + 3] = __fsub_rn(t.w, y[i + 3]);
        n2 = ffma2(make_float2(y[i], y[i + 1]), make_float2(y[i], y[i + 1]), n2);
        n2 = ffma2(make_float2(y[i + 2], y[i + 3]), make_float2(y[i + 2], y[i + 3]), n2);
        // the residual replaces x in the tile: the exact dot of an undecided row reads it there
        *reinterpret_cast<float4*>(row + i) = make_float4(y[i], y[i + 1], y[i + 2], y[i + 3]);
      }
#pragma unroll
      for (int i = 0; i < D; i++) res_ok = res_ok && pkv_finite(y[i]);
      if (!code && !res_ok) code = PKV_VEC_NONFINITE_RESIDUAL;  // qjl.rs:210
      // QjlQuantizer::sketch, qjl.rs:214-217: sign of the sequential f32 dot per row.  The dot is
      // first taken with packed fused multiply-adds in four chains; its sign is the reference's
      // whenever |dot| clears the rounding bound (pkv_fast_paths.h), else fix_signs decides.
      uint32_t* sw = w + (tp.radii_words + tp.angle_words) * K::WS;
      const float rnorm = __fmul_rn(__fsqrt_rn(n2.x + n2.y), 1.0001f);
      unsigned long long uncq = 0;
      uint32_t bits = 0;
#pragma unroll 4
      for (int p = 0; p < tp.projections; p++) {
        const float* grow = s_g + p * D;
        float2 d0 = make_float2(0.0f, 0.0f), d1 = d0;
#pragma unroll
        for (int j = 0; j < D; j += 4) {
          const float4 gg = *reinterpret_cast<const float4*>(grow + j);
          d0 = ffma2(make_float2(gg.x, gg.y), make_float2(y[j], y[j + 1]), d0);
          d1 = ffma2(make_float2(gg.z, gg.w), make_float2(y[j + 2], y[j + 3]), d1);
        }
        const float dot = (d0.x + d0.y) + (d1.x + d1.y);
        const float tau = fmaf(s_thr[p], rnorm, PKV_QJL_ABS_BOUND);
        uncq |= (unsigned long long)(fabsf(dot) > tau ? 0u : 1u) << p;
        bits |= (dot >= 0.0f ? 1u : 0u) << (p & 31);
        if ((p & 31) == 31) {
          sw[(p >> 5) * K::WS] = bits;
          bits = 0;
        }
      }
      if (uncq) fix_signs(s_g, row, D, uncq, sw, K::WS);
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
    if (code) pkv_report(err, 0, (int64_t)batch * g.vpb + v0 + v, code);
  }
  __syncthreads();
  stage_records<D, false>(
      s_w, reinterpret_cast<uint32_t*>(payload + (int64_t)batch * g.payload_batch_stride +
                                       (int64_t)v0 * g.rec_bytes),
      nv, tp.rec_words);
}

template <int D>
size_t turbo_encode_smem(const TurboParams& tp) {
  using K = Turbo<D>;
  return sizeof(float) * K::TV * K::XS + sizeof(float) * tp.projections * (D + 1) +
         sizeof(float) * (2 * (1 << tp.polar_bits) + 2 * tp.ray_count) +
         sizeof(uint32_t) * tp.rec_words * K::WS + (tp.lossy ? sizeof(float) * K::P * K::WS : 0) +
         sizeof(int64_t) * (K::TV + 1);
}

}  // namespace pkv_turbo
