// Compressed-domain scoring: the inner-product estimate of a prepared query against every stored
// record, without reconstructing the vectors.
//  turbo-quant/src/turbo.rs:340-381 (score_batch_prepared: polar estimate + QJL correction),
//  polar.rs:346-370 (sum over pairs of r (q_a cos + q_b sin), binary32, pair order),
//  qjl.rs:294-330 (sqrt(pi/2) / m * sum_j sign_j p_j), wire.rs:497-565 (record), radius.rs:81-147
// One thread per record; the record tile is staged exactly as in the decode kernel.  Each score is
// the reference's operation sequence (separately rounded multiplies and adds, ascending order), so
// the result is the reference's binary32 value given the same cos / sin table.
#pragma once

#include "pkv_turbo_common.cuh"

namespace pkv_turbo {

template <int D>
struct TurboScoreSmem {
  using K = Turbo<D>;
  static __host__ __device__ size_t warp_bytes(int rec_words) {
    return ((sizeof(uint32_t) * rec_words * K::WS) + 15) & ~(size_t)15;
  }
  static __host__ __device__ size_t table_bytes(int levels) { return sizeof(float) * (256 + 2 * levels + D + 64); }
};

template <int D, int PB>
__global__ void __launch_bounds__(Turbo<D>::THREADS)
turbo_score_kernel(PkvGeom g, TurboParams tp, const uint8_t* __restrict__ payload,
                   const float* __restrict__ rotated_query, const float* __restrict__ projected_query,
                   float qjl_scale, float* __restrict__ scores, uint64_t* err) {
  using K = Turbo<D>;
  extern __shared__ __align__(128) uint8_t smem[];
  const int pb = PB ? PB : tp.polar_bits;
  const int levels = 1 << pb;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* s_q255 = reinterpret_cast<float*>(smem);  // [256]
  float* s_lut = s_q255 + 256;                     // (cos, sin)[L]
  float* s_q = s_lut + 2 * levels;                 // [D] rotated query
  float* s_p = s_q + D;                            // [64] projected query
  uint32_t* s_w = reinterpret_cast<uint32_t*>(smem + TurboScoreSmem<D>::table_bytes(levels) +
                                              warp * TurboScoreSmem<D>::warp_bytes(tp.rec_words));

  const int64_t tile_id = (int64_t)blockIdx.x * K::NWARPS + warp;
  const bool active = tile_id < (int64_t)g.n_batches * g.tiles_per_batch;
  const int tile = active ? (int)(tile_id % g.tiles_per_batch) : 0;
  const int batch = active ? (int)(tile_id / g.tiles_per_batch) : 0;
  const int v0 = tile * K::TV;
  const int nv = active ? min(K::TV, g.vpb - v0) : 0;
  const int v = lane;

  stage_records<D, true>(
      s_w, reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(
               payload + (int64_t)batch * g.payload_batch_stride + (int64_t)v0 * g.rec_bytes)),
      nv, tp.rec_words, lane);
  for (int i = threadIdx.x; i < 2 * levels; i += K::THREADS)
    pkv_cp_async4(s_lut + (i < levels ? 2 * i : 2 * (i - levels) + 1), tp.lut + i);
  for (int i = threadIdx.x; i < D; i += K::THREADS) pkv_cp_async4(s_q + i, rotated_query + i);
  for (int i = threadIdx.x; i < tp.projections; i += K::THREADS) pkv_cp_async4(s_p + i, projected_query + i);
  if (tp.lossy)
    for (int i = threadIdx.x; i < 256; i += K::THREADS) s_q255[i] = __fdiv_rn((float)i, 255.0f);
  pkv_cp_async_wait_all();
  __syncthreads();

  if (v >= nv) return;
  const uint32_t* w = s_w + v;
  int code = 0;
  float rad[K::P];
  if (!tp.lossy) {
#pragma unroll
    for (int i = 0; i < K::P; i++) {
      rad[i] = __uint_as_float(w[i * K::WS]);
      if (!code && (!pkv_finite(rad[i]) || rad[i] < 0.0f)) code = PKV_VEC_BAD_RADIUS;  // radius.rs:98-103
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
        rad[4 * k + b] = r;
      }
    }
  }
  // polar estimate, polar.rs:355-362: estimate += r * (q_a * cos + q_b * sin)
  const uint32_t* aw = w + tp.radii_words * K::WS;
  const uint32_t mask = (uint32_t)levels - 1u;
  float est = 0.0f;
  {
    uint64_t bitbuf = 0;
    int nbits = 0, wk = 0;
#pragma unroll
    for (int i = 0; i < K::P; i++) {
      if (nbits < pb) {
        bitbuf |= (uint64_t)aw[wk * K::WS] << nbits;
        wk++;
        nbits += 32;
      }
      const uint32_t idx = (uint32_t)bitbuf & mask;
      bitbuf >>= pb;
      nbits -= pb;
      const float2 cs = *reinterpret_cast<const float2*>(s_lut + 2 * idx);
      const float2 q = *reinterpret_cast<const float2*>(s_q + 2 * i);
      const float inner = __fadd_rn(__fmul_rn(q.x, cs.x), __fmul_rn(q.y, cs.y));
      est = __fadd_rn(est, __fmul_rn(rad[i], inner));
    }
  }
  if (!code && !pkv_finite(est)) code = PKV_VEC_NONFINITE_OUTPUT;  // "polar score is not finite"
  float score = est;
  if (tp.mode == PKV_TURBO_POLAR_WITH_QJL) {
    // qjl.rs:316-330: sum of sign_j * p_j in order, then the scale
    const uint32_t* sw = aw + tp.angle_words * K::WS;
    float sum = 0.0f;
    for (int j = 0; j < tp.projections; j++) {
      const uint32_t bit = (sw[(j >> 5) * K::WS] >> (j & 31)) & 1u;
      const float p = s_p[j];
      sum = __fadd_rn(sum, bit ? p : -p);
    }
    const float corr = __fmul_rn(qjl_scale, sum);
    if (!code && !pkv_finite(corr)) code = PKV_VEC_NONFINITE_OUTPUT;  // "qjl score is not finite"
    score = __fadd_rn(est, corr);
    if (!code && !pkv_finite(score)) code = PKV_VEC_NONFINITE_OUTPUT;  // "turbo score is not finite"
  }
  const int64_t gvec = (int64_t)batch * g.vpb + v0 + v;
  if (code) pkv_report(err, 0, gvec, code);
  scores[gvec] = score;
}

template <int D>
size_t turbo_score_smem(const TurboParams& tp) {
  return TurboScoreSmem<D>::table_bytes(1 << tp.polar_bits) +
         Turbo<D>::NWARPS * TurboScoreSmem<D>::warp_bytes(tp.rec_words);
}

}  // namespace pkv_turbo
