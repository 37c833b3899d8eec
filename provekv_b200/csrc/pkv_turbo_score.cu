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
                 const float* projected, float qjl_scale, float* scores, uint64_t* err, unsigned grid,
                 cudaStream_t s) {
  const size_t sm = turbo_score_smem<D>(tp);
  const unsigned ctas = (grid + Turbo<D>::NWARPS - 1) / Turbo<D>::NWARPS;
  int st;
  if constexpr (PB != 0) {
    const int raw = turbo_score_raw(tp, PB);
    if (raw == 1) {
      if ((st = set_smem(turbo_score_kernel<D, PB, 1>, sm)) != PKV_OK) return st;
      turbo_score_kernel<D, PB, 1><<<ctas, Turbo<D>::THREADS, sm, s>>>(g, tp, payload, rotated, projected,
                                                                      qjl_scale, scores, err);
      return PKV_OK;
    }
    if (raw == 2) {
      if ((st = set_smem(turbo_score_kernel<D, PB, 2>, sm)) != PKV_OK) return st;
      turbo_score_kernel<D, PB, 2><<<ctas, Turbo<D>::THREADS, sm, s>>>(g, tp, payload, rotated, projected,
                                                                      qjl_scale, scores, err);
      return PKV_OK;
    }
  }
  if ((st = set_smem(turbo_score_kernel<D, PB, 0>, sm)) != PKV_OK) return st;
  turbo_score_kernel<D, PB, 0><<<ctas, Turbo<D>::THREADS, sm, s>>>(g, tp, payload, rotated, projected,
                                                                  qjl_scale, scores, err);
  return PKV_OK;
}

}  // namespace

int pkv_launch_turbo_score(const pkv_turbo_profile* p, const uint8_t* payload, const PkvGeom& g,
                           const float* rotated, const float* projected, float* scores, uint64_t* err,
                           cudaStream_t s) {
  const int64_t grid = (int64_t)g.n_batches * g.tiles_per_batch;
  if (grid == 0) return PKV_OK;
  if (grid > 0x7fffffff) return PKV_ERR_UNSUPPORTED;
  const TurboParams tp = make_params(p);
  // (PI / 2.0).sqrt() * source_norm / m with source_norm = 1, turbo-quant/src/qjl.rs:316-317
  volatile float half_pi_root = sqrtf(3.14159274101257324f / 2.0f);
  const float qjl_scale = p->cfg.projections > 0 ? (half_pi_root * 1.0f) / (float)p->cfg.projections : 0.0f;
  int st;
  if (p->cfg.dim == 64) {
    PKV_DISPATCH_PB(launch_score, 64, tp, payload, g, rotated, projected, qjl_scale, scores, err, (unsigned)grid, s)
  } else if (p->cfg.dim == 128) {
    PKV_DISPATCH_PB(launch_score, 128, tp, payload, g, rotated, projected, qjl_scale, scores, err, (unsigned)grid, s)
  } else {
    return PKV_ERR_UNSUPPORTED;
  }
  if (st != PKV_OK) return st;
  pkv_count_launch();
  return pkv_cuda_status(cudaGetLastError());
}
