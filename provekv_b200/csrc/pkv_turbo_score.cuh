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
  // the per-pair table of q_a cos_k + q_b sin_k is kept for up to 128 angle levels (16 KB at d = 64)
  static __host__ __device__ bool has_inner_table(int levels) { return levels <= 128; }
  // per query: the rotated query, the projected query and the inner table
  static __host__ __device__ size_t query_floats(int levels) {
    return D + 64 + (has_inner_table(levels) ? (D / 2) * levels : 0);
  }
  static __host__ __device__ size_t table_bytes(int levels, int n_queries) {
    return sizeof(float) * (256 + 2 * levels + (size_t)n_queries * query_floats(levels));
  }
};

// One record -> score.  W(k) returns word k of the record.  FIXED: f32 radii and a compile-time angle
// width, so every k is a compile-time constant after unrolling and W may index registers.
template <int D, int PB, bool FIXED, typename W>
__device__ __forceinline__ float score_record(const W& w, const TurboParams& tp, int pb, int levels,
                                              const float* s_q255, const float* s_lut, const float* s_q,
                                              const float* s_p, const float* s_inner, bool inner_table,
                                              float qjl_scale, int& code) {
  using K = Turbo<D>;
  bool lossy = false;
  if constexpr (!FIXED) lossy = tp.lossy;
  // radius i: f32 word i (finite and non-negative, radius.rs:98-103: sign clear and exponent not all
  // ones; -0.0 is looked at again below), or the BlockLogU8 byte i through expf (radius.rs:128-145)
  uint32_t bad = 0;
  float mn = 0.0f, span = 0.0f;
  if (lossy) {
    if constexpr (!FIXED) {
      mn = __uint_as_float(w(K::P / 4));
      const float mx = __uint_as_float(w(K::P / 4 + 1));
      if (!pkv_finite(mn) || !pkv_finite(mx) || mn > mx) code = PKV_VEC_BAD_RADIUS_RANGE;
      span = __fsub_rn(mx, mn);
    }
  }
  auto radius = [&](int i) -> float {
    if (!lossy) {
      const uint32_t u = w(i);
      bad |= (u >> 31) | (uint32_t)((u & 0x7f800000u) == 0x7f800000u);
      return __uint_as_float(u);
    }
    float r = 0.0f;
    if constexpr (!FIXED) {
      const float t = __fadd_rn(mn, __fmul_rn(span, s_q255[(w(i >> 2) >> (8 * (i & 3))) & 0xffu]));
      r = code ? 0.0f : pkv_ulp_adjust(tp.expf_table, t, pkv_expf_portable(t));
      if (!code && !pkv_finite(r)) code = PKV_VEC_BAD_RADIUS;  // polar.rs:127-133
    }
    return r;
  };
  // polar estimate, polar.rs:355-362: estimate += r * (q_a * cos + q_b * sin)
  const int a0 = FIXED ? K::P : tp.radii_words;  // first angle word
  const uint32_t mask = (uint32_t)levels - 1u;
  float est = 0.0f;
  auto add_pair = [&](int i, uint32_t idx) {
    float inner;
    if (inner_table) {
      inner = s_inner[i * levels + idx];
    } else {
      const float2 cs = *reinterpret_cast<const float2*>(s_lut + 2 * idx);
      const float2 q = *reinterpret_cast<const float2*>(s_q + 2 * i);
      inner = __fadd_rn(__fmul_rn(q.x, cs.x), __fmul_rn(q.y, cs.y));
    }
    est = __fadd_rn(est, __fmul_rn(radius(i), inner));
  };
  if constexpr (PB != 0) {
    constexpr int NW = K::P * PB / 32;
    uint32_t words[NW];
#pragma unroll
    for (int k = 0; k < NW; k++) words[k] = w(a0 + k);
#pragma unroll
    for (int i = 0; i < K::P; i++) {
      const int pos = i * PB, wi = pos >> 5, sh = pos & 31;
      uint32_t idx = words[wi] >> sh;
      if (sh + PB > 32) idx |= words[wi + 1] << (32 - sh);
      add_pair(i, idx & mask);
    }
  } else {
    uint64_t bitbuf = 0;
    int nbits = 0, wk = 0;
#pragma unroll
    for (int i = 0; i < K::P; i++) {
      if (nbits < pb) {
        bitbuf |= (uint64_t)w(a0 + wk) << nbits;
        wk++;
        nbits += 32;
      }
      const uint32_t idx = (uint32_t)bitbuf & mask;
      bitbuf >>= pb;
      nbits -= pb;
      add_pair(i, idx);
    }
  }
  if (bad) {  // a set sign bit or an all-ones exponent: decide exactly (-0.0 passes `value < 0.0`)
#pragma unroll
    for (int i = 0; i < K::P; i++) {
      const float r = __uint_as_float(w(i));
      if (!code && (!pkv_finite(r) || r < 0.0f)) code = PKV_VEC_BAD_RADIUS;
    }
  }
  if (!code && !pkv_finite(est)) code = PKV_VEC_NONFINITE_OUTPUT;  // "polar score is not finite"
  float score = est;
  if (tp.mode == PKV_TURBO_POLAR_WITH_QJL) {
    // qjl.rs:316-330: sum of sign_j * p_j in order, then the scale
    const int s0 = FIXED ? K::P + K::P * (PB ? PB : 1) / 32 : a0 + tp.angle_words;
    float sum = 0.0f;
#pragma unroll
    for (int h = 0; h < 2; h++) {  // projections is 32 or 64
      if (h * 32 < tp.projections) {
        const uint32_t flip = ~w(s0 + h);
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 p4 = *reinterpret_cast<const float4*>(s_p + h * 32 + j);
          const float pv[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
          for (int t = 0; t < 4; t++)  // sign as f32 * p is exactly +-p
            sum = __fadd_rn(sum, __uint_as_float(__float_as_uint(pv[t]) ^ (((flip >> (j + t)) & 1u) << 31)));
        }
      }
    }
    const float corr = __fmul_rn(qjl_scale, sum);
    if (!code && !pkv_finite(corr)) code = PKV_VEC_NONFINITE_OUTPUT;  // "qjl score is not finite"
    score = __fadd_rn(est, corr);
    if (!code && !pkv_finite(score)) code = PKV_VEC_NONFINITE_OUTPUT;  // "turbo score is not finite"
  }
  return score;
}

// MULTI = false is the one-query launch: without the loop over the queries the compiler keeps the kernel
// at 72 registers (seven CTAs per SM); with it, it holds the unpacked record across the queries (155).
template <int D, int PB, int RAW, bool MULTI>
__global__ void __launch_bounds__(Turbo<D>::THREADS)
turbo_score_kernel(PkvGeom g, TurboParams tp, const uint8_t* __restrict__ payload,
                   const float* __restrict__ rotated_query, const float* __restrict__ projected_query,
                   int n_queries, int64_t score_stride, float qjl_scale, float* __restrict__ scores, uint64_t* err) {
  using K = Turbo<D>;
  extern __shared__ __align__(128) uint8_t smem[];
  const int pb = PB ? PB : tp.polar_bits;
  const int levels = 1 << pb;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if constexpr (!MULTI) n_queries = 1;
  float* s_q255 = reinterpret_cast<float*>(smem);  // [256]
  float* s_lut = s_q255 + 256;                     // (cos, sin)[L]
  // per query, QF floats apart: [D] rotated query, [64] projected query, [P][L] q_a cos_k + q_b sin_k (the
  // part of a pair's term that is the same for every record)
  float* s_qbase = s_lut + 2 * levels;
  const int QF = (int)TurboScoreSmem<D>::query_floats(levels);
  const bool inner_table = TurboScoreSmem<D>::has_inner_table(levels);
  uint32_t* s_w = reinterpret_cast<uint32_t*>(smem + TurboScoreSmem<D>::table_bytes(levels, n_queries) +
                                              warp * TurboScoreSmem<D>::warp_bytes(tp.rec_words));

  const int64_t tile_id = (int64_t)blockIdx.x * K::NWARPS + warp;
  const bool active = tile_id < (int64_t)g.n_batches * g.tiles_per_batch;
  const int tile = active ? (int)(tile_id % g.tiles_per_batch) : 0;
  const int batch = active ? (int)(tile_id / g.tiles_per_batch) : 0;
  const int v0 = tile * K::TV;
  const int nv = active ? min(K::TV, g.vpb - v0) : 0;
  const int v = lane;

  // f32 radii in records that are a multiple of 16 bytes (fixed angle width): the warp's run of records
  // is copied as it lies, 16 bytes per copy, and every lane reads its own record with 16-byte loads
  // (conflict-free: consecutive records start an odd number of 16-byte units apart or the quarter-warps
  // cover distinct bank groups); otherwise the word-transposed tile of the decode kernel.
  // the launcher checks: PB != 0, f32 radii; RAW 1: rec_words % 4 == 0 (register loads), 2: rec_words odd
  constexpr int raw = RAW;
  const uint8_t* src = payload + (int64_t)batch * g.payload_batch_stride + (int64_t)v0 * g.rec_bytes;
  if constexpr (raw != 0) {
    const int nw = nv * tp.rec_words, n16 = nw / 4;  // a full tile of 32 records is a multiple of 16 bytes
    for (int i = lane; i < n16; i += 32)
      pkv_cp_async16(reinterpret_cast<uint4*>(s_w) + i, reinterpret_cast<const uint4*>(src) + i);
    for (int i = 4 * n16 + lane; i < nw; i += 32) pkv_cp_async4(s_w + i, reinterpret_cast<const uint32_t*>(src) + i);
  } else {
    stage_records<D, true>(s_w, reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(src)), nv, tp.rec_words, lane);
  }
  for (int i = threadIdx.x; i < 2 * levels; i += K::THREADS)
    pkv_cp_async4(s_lut + (i < levels ? 2 * i : 2 * (i - levels) + 1), tp.lut + i);
  for (int i = threadIdx.x; i < n_queries * D; i += K::THREADS)
    pkv_cp_async4(s_qbase + (i / D) * QF + (i % D), rotated_query + i);
  for (int i = threadIdx.x; i < n_queries * tp.projections; i += K::THREADS)
    pkv_cp_async4(s_qbase + (i / tp.projections) * QF + D + (i % tp.projections), projected_query + i);
  if (tp.lossy)
    for (int i = threadIdx.x; i < 256; i += K::THREADS) s_q255[i] = __fdiv_rn((float)i, 255.0f);
  pkv_cp_async_wait_all();
  __syncthreads();
  if (inner_table) {  // polar.rs:361: (q_a * theta.cos() + q_b * theta.sin()), the record-independent part
    for (int e = threadIdx.x; e < n_queries * K::P * levels; e += K::THREADS) {
      const int qi = e / (K::P * levels), r = e - qi * (K::P * levels);
      const int i = r / levels, k = r - i * levels;
      const float* s_q = s_qbase + qi * QF;
      s_qbase[qi * QF + D + 64 + r] =
          __fadd_rn(__fmul_rn(s_q[2 * i], s_lut[2 * k]), __fmul_rn(s_q[2 * i + 1], s_lut[2 * k + 1]));
    }
    __syncthreads();
  }

  if (v >= nv) return;
  const int64_t gvec = (int64_t)batch * g.vpb + v0 + v;
  // the record stays where it is (registers or the tile) while the queries take their turns
  if constexpr (raw == 1) {
    // the record in registers: RW words loaded 16 bytes at a time from this lane's run of the raw tile
    constexpr int NWT = K::P * (PB ? PB : 1) / 32 + 2;  // angle words + up to two sign words
    constexpr int RW = (K::P + NWT + 3) & ~3;
    uint32_t rw[RW];
    const uint4* w4 = reinterpret_cast<const uint4*>(s_w + v * tp.rec_words);
#pragma unroll
    for (int k = 0; k < RW / 4; k++) {
      const uint4 u = 4 * k < tp.rec_words ? w4[k] : make_uint4(0u, 0u, 0u, 0u);
      rw[4 * k] = u.x; rw[4 * k + 1] = u.y; rw[4 * k + 2] = u.z; rw[4 * k + 3] = u.w;
    }
#pragma unroll 1
    for (int qi = 0; qi < n_queries; qi++) {
      const float* s_q = s_qbase + qi * QF;
      int code = 0;
      const float score = score_record<D, PB, true>([&](int k) { return rw[k]; }, tp, pb, levels, s_q255, s_lut, s_q,
                                                    s_q + D, s_q + D + 64, inner_table, qjl_scale, code);
      if (code) pkv_report(err, 0, gvec, code);
      scores[(int64_t)qi * score_stride + gvec] = score;
    }
  } else {
#pragma unroll 1
    for (int qi = 0; qi < n_queries; qi++) {
      const float* s_q = s_qbase + qi * QF;
      int code = 0;
      float score;
      if constexpr (raw == 2) {  // odd record stride: word reads of the raw tile are conflict-free
        const uint32_t* wr = s_w + v * tp.rec_words;
        score = score_record<D, PB, true>([&](int k) { return wr[k]; }, tp, pb, levels, s_q255, s_lut, s_q, s_q + D,
                                          s_q + D + 64, inner_table, qjl_scale, code);
      } else {
        const uint32_t* w = s_w + v;
        score = score_record<D, PB, false>([&](int k) { return w[k * K::WS]; }, tp, pb, levels, s_q255, s_lut, s_q,
                                           s_q + D, s_q + D + 64, inner_table, qjl_scale, code);
      }
      if (code) pkv_report(err, 0, gvec, code);
      scores[(int64_t)qi * score_stride + gvec] = score;
    }
  }
}

// TurboQuantizer::prepare_query (turbo-quant/src/turbo.rs:322-337) for a batch of queries, one CTA of 64
// threads per query.  Thread 0 runs FastHadamardRotation::apply (polar.rs:336-343) with the encoder's own
// transform; thread j < projections sums row j of the QJL matrix against the query in order, every product
// rounded (qjl.rs:275-279).  A query, a rotated query or a projection that is not finite is reported with the
// query's index (the reference's check_finite_vector at each of the three places).
template <int D>
__global__ void __launch_bounds__(64)
turbo_prepare_query_kernel(TurboParams tp, const float* __restrict__ queries, float* __restrict__ rotated,
                           float* __restrict__ projected, uint64_t* err) {
  __shared__ float s_x[D];
  const int64_t qi = blockIdx.x;
  const float* q = queries + qi * D;
  for (int i = threadIdx.x; i < D; i += 64) s_x[i] = q[i];
  __syncthreads();
  bool bad = false;
  if (threadIdx.x == 0) {
    float y[D];
#pragma unroll
    for (int i = 0; i < D; i++) {
      y[i] = s_x[i];
      bad = bad || !pkv_finite(y[i]);
    }
    fwht_forward_signed<D>(y, tp.sgn, tp.scale);
#pragma unroll
    for (int i = 0; i < D; i++) {
      bad = bad || !pkv_finite(y[i]);
      rotated[qi * D + i] = y[i];
    }
  }
  if ((int)threadIdx.x < tp.projections) {
    const float* grow = tp.qjl + (size_t)threadIdx.x * D;
    float sum = 0.0f;
#pragma unroll 8
    for (int k = 0; k < D; k++) sum = __fadd_rn(sum, __fmul_rn(__ldg(grow + k), s_x[k]));
    projected[qi * tp.projections + threadIdx.x] = sum;
    bad = bad || !pkv_finite(sum);
  }
  if (bad) pkv_report(err, 0, qi, PKV_VEC_NONFINITE_INPUT);
}

template <int D>
size_t turbo_score_smem(const TurboParams& tp, int n_queries) {
  return TurboScoreSmem<D>::table_bytes(1 << tp.polar_bits, n_queries) +
         Turbo<D>::NWARPS * TurboScoreSmem<D>::warp_bytes(tp.rec_words);
}

}  // namespace pkv_turbo

namespace pkv_turbo {
inline int turbo_score_raw(const TurboParams& tp, int pb_template) {
  if (pb_template == 0 || tp.lossy) return 0;
  return (tp.rec_words % 4) == 0 ? 1 : (tp.rec_words & 1) ? 2 : 0;
}
}  // namespace pkv_turbo
