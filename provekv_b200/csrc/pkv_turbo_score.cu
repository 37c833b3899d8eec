// turbo-quant hot-shell kernels for sm_100a: randomised Hadamard transform
// (Rademacher signs, FWHT held in registers), polar decomposition with b-bit
// angle buckets, f32 or BlockLogU8 radii, optional QJL residual sign sketch,
// and the inverse fused with the write into the KV cache.
//
// One thread owns one vector and one warp owns a tile of 32 vectors, staged through its own
// slice of shared memory (f32 tile with padded rows; records word-transposed, so record word k
// of vector v sits at [k][v]) so that every global access is coalesced.
// The kernels (pkv_turbo_encode.cuh, pkv_turbo_decode.cuh) are templated on the
// dimension and on the angle width: 3, 4 and 7 bits are compiled with static bit
// positions, any other width runs the generic variant (PB = 0).
#include "pkv_turbo_score.cuh"
#include "pkv_turbo_launch.cuh"

using namespace pkv_turbo;

namespace {

template <int D, int PB>
int launch_score(const TurboParams& tp, const uint8_t* payload, const PkvGeom& g, const float* rotated,
                 const float* projected, int n_queries, int64_t score_stride, float qjl_scale, float* scores,
                 uint64_t* err, unsigned grid, cudaStream_t s) {
  const size_t sm = turbo_score_smem<D>(tp, n_queries);
  const unsigned ctas = (grid + Turbo<D>::NWARPS - 1) / Turbo<D>::NWARPS;
  int st;
#define PKV_SCORE_LAUNCH(RAW, MULTI)                                                                     \
  {                                                                                                      \
    if ((st = set_smem(turbo_score_kernel<D, PB, RAW, MULTI>, sm)) != PKV_OK) return st;                 \
    turbo_score_kernel<D, PB, RAW, MULTI><<<ctas, Turbo<D>::THREADS, sm, s>>>(                          \
        g, tp, payload, rotated, projected, n_queries, score_stride, qjl_scale, scores, err);            \
    return PKV_OK;                                                                                       \
  }
  if constexpr (PB != 0) {
    const int raw = turbo_score_raw(tp, PB);
    if (raw == 1) {
      if (n_queries > 1) PKV_SCORE_LAUNCH(1, true) else PKV_SCORE_LAUNCH(1, false)
    }
    if (raw == 2) {
      if (n_queries > 1) PKV_SCORE_LAUNCH(2, true) else PKV_SCORE_LAUNCH(2, false)
    }
  }
  if (n_queries > 1) PKV_SCORE_LAUNCH(0, true) else PKV_SCORE_LAUNCH(0, false)
#undef PKV_SCORE_LAUNCH
}

}  // namespace

// Queries per launch: the per-query tables (rotated and projected query, inner table) of one launch stay
// below 64 KB of shared memory, and at most 8 queries share a pass over the records.
template <int D>
static int score_queries_per_launch(const TurboParams& tp) {
  const size_t per_query = sizeof(float) * TurboScoreSmem<D>::query_floats(1 << tp.polar_bits);
  const size_t fit = (64 * 1024) / per_query;
  return (int)(fit < 1 ? 1 : fit > 8 ? 8 : fit);
}

int pkv_launch_turbo_score(const pkv_turbo_profile* p, const uint8_t* payload, const PkvGeom& g,
                           const float* rotated, const float* projected, int64_t n_queries, float* scores,
                           uint64_t* err, cudaStream_t s) {
  const int64_t grid = (int64_t)g.n_batches * g.tiles_per_batch;
  if (grid == 0 || n_queries == 0) return PKV_OK;
  if (grid > 0x7fffffff) return PKV_ERR_UNSUPPORTED;
  const TurboParams tp = make_params(p);
  // (PI / 2.0).sqrt() * source_norm / m with source_norm = 1, turbo-quant/src/qjl.rs:316-317
  volatile float half_pi_root = sqrtf(3.14159274101257324f / 2.0f);
  const float qjl_scale = p->cfg.projections > 0 ? (half_pi_root * 1.0f) / (float)p->cfg.projections : 0.0f;
  const int64_t score_stride = (int64_t)g.n_batches * g.vpb;
  const int per = p->cfg.dim == 64 ? score_queries_per_launch<64>(tp) : score_queries_per_launch<128>(tp);
  for (int64_t q0 = 0; q0 < n_queries; q0 += per) {
    const int nq = (int)(n_queries - q0 < per ? n_queries - q0 : per);
    const float* rq = rotated + q0 * p->cfg.dim;
    const float* pq = projected ? projected + q0 * p->cfg.projections : projected;
    float* sc = scores + q0 * score_stride;
    int st;
    if (p->cfg.dim == 64) {
      PKV_DISPATCH_PB(launch_score, 64, tp, payload, g, rq, pq, nq, score_stride, qjl_scale, sc, err, (unsigned)grid, s)
    } else if (p->cfg.dim == 128) {
      PKV_DISPATCH_PB(launch_score, 128, tp, payload, g, rq, pq, nq, score_stride, qjl_scale, sc, err, (unsigned)grid, s)
    } else {
      return PKV_ERR_UNSUPPORTED;
    }
    if (st != PKV_OK) return st;
    pkv_count_launch();
    if (cudaError_t ce = cudaGetLastError()) return pkv_cuda_status(ce);
  }
  return PKV_OK;
}

int pkv_launch_turbo_prepare_queries(const pkv_turbo_profile* p, const float* queries, int64_t n_queries,
                                     float* rotated, float* projected, uint64_t* err, cudaStream_t s) {
  if (n_queries == 0) return PKV_OK;
  if (n_queries > 0x7fffffff) return PKV_ERR_UNSUPPORTED;
  const TurboParams tp = make_params(p);
  if (p->cfg.dim == 64)
    turbo_prepare_query_kernel<64><<<(unsigned)n_queries, 64, 0, s>>>(tp, queries, rotated, projected, err);
  else if (p->cfg.dim == 128)
    turbo_prepare_query_kernel<128><<<(unsigned)n_queries, 64, 0, s>>>(tp, queries, rotated, projected, err);
  else
    return PKV_ERR_UNSUPPORTED;
  pkv_count_launch();
  return pkv_cuda_status(cudaGetLastError());
}
