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
#include "pkv_turbo_decode.cuh"
#include "pkv_turbo_score.cuh"
#include "pkv_turbo_encode.cuh"

using namespace pkv_turbo;

namespace {

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
  for (int i = 0; i < 128; i++) {
    const bool neg = (p->sign_mask[i >> 5] >> (i & 31)) & 1u;
    tp.sgn[i] = neg ? -1.0f : 1.0f;
    tp.sgn_scale[i] = neg ? -p->scale : p->scale;
  }
  for (int i = 0; i < 64; i++) {
    tp.qjl_thr_tf32[i] = i < tp.projections ? p->qjl_thr_tf32[i] : 0.0f;
  }
  tp.fast_bucket = p->fast_bucket;
  tp.ray_count = p->ray_count;
  tp.skip_issue = pkv_skip_tensor_issue();
  tp.qjl = p->qjl_dev;
  tp.lut = p->lut_dev;
  return tp;
}

template <typename F>
int set_smem(F kernel, size_t bytes) {
  if (bytes > 48 * 1024)
    return pkv_cuda_status(
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return PKV_OK;
}

template <int D, int PB>
int launch_encode(const TurboParams& tp, const float* x, const PkvGeom& g, uint8_t* payload,
                  uint64_t* err, unsigned grid, cudaStream_t s) {
  const size_t sm = turbo_encode_smem<D>(tp);
  const unsigned ctas = (grid + TurboEnc<D>::NWARPS - 1) / TurboEnc<D>::NWARPS;  // one warp per 32-vector tile
  int st;
  if (turbo_encode_direct(tp)) {
    if ((st = set_smem(turbo_encode_kernel<D, PB, true>, sm)) != PKV_OK) return st;
    turbo_encode_kernel<D, PB, true><<<ctas, TurboEnc<D>::THREADS, sm, s>>>(g, tp, x, payload, err);
  } else {
    if ((st = set_smem(turbo_encode_kernel<D, PB, false>, sm)) != PKV_OK) return st;
    turbo_encode_kernel<D, PB, false><<<ctas, TurboEnc<D>::THREADS, sm, s>>>(g, tp, x, payload, err);
  }
  return PKV_OK;
}

template <int D, int PB, int DST>
int launch_decode_as(const TurboParams& tp, const uint8_t* payload, const PkvGeom& g, void* cache,
                     uint64_t* err, unsigned grid, cudaStream_t s) {
  const size_t sm = turbo_decode_smem<D>(tp);
  const unsigned ctas = (grid + Turbo<D>::NWARPS - 1) / Turbo<D>::NWARPS;
  int st;
  if constexpr (PB != 0) {
    const int raw = turbo_decode_raw(tp, PB);
    if (raw == 1) {
      if ((st = set_smem(turbo_decode_patch_kernel<D, PB, DST, 1>, sm)) != PKV_OK) return st;
      turbo_decode_patch_kernel<D, PB, DST, 1><<<ctas, Turbo<D>::THREADS, sm, s>>>(
          g, tp, payload, static_cast<typename PkvDst<DST>::type*>(cache), err);
      return PKV_OK;
    }
    if (raw == 2) {
      if ((st = set_smem(turbo_decode_patch_kernel<D, PB, DST, 2>, sm)) != PKV_OK) return st;
      turbo_decode_patch_kernel<D, PB, DST, 2><<<ctas, Turbo<D>::THREADS, sm, s>>>(
          g, tp, payload, static_cast<typename PkvDst<DST>::type*>(cache), err);
      return PKV_OK;
    }
  }
  if ((st = set_smem(turbo_decode_patch_kernel<D, PB, DST, 0>, sm)) != PKV_OK) return st;
  turbo_decode_patch_kernel<D, PB, DST, 0><<<ctas, Turbo<D>::THREADS, sm, s>>>(
      g, tp, payload, static_cast<typename PkvDst<DST>::type*>(cache), err);
  return PKV_OK;
}

template <int D, int PB>
int launch_decode(const TurboParams& tp, const uint8_t* payload, const PkvGeom& g, void* cache, int dst,
                  uint64_t* err, unsigned grid, cudaStream_t s) {
  switch (dst) {
    case PKV_DST_F32: return launch_decode_as<D, PB, PKV_DST_F32>(tp, payload, g, cache, err, grid, s);
    case PKV_DST_F16: return launch_decode_as<D, PB, PKV_DST_F16>(tp, payload, g, cache, err, grid, s);
    case PKV_DST_BF16: return launch_decode_as<D, PB, PKV_DST_BF16>(tp, payload, g, cache, err, grid, s);
    default: return PKV_ERR_INVALID_ARGUMENT;
  }
}

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

int pkv_turbo_tile_vectors(int dim) { return (dim == 64 || dim == 128) ? 32 : 0; }

#define PKV_DISPATCH_PB(FN, DIM, ...)                         \
  switch (tp.polar_bits) {                                    \
    case 3: st = FN<DIM, 3>(__VA_ARGS__); break;              \
    case 4: st = FN<DIM, 4>(__VA_ARGS__); break;              \
    case 7: st = FN<DIM, 7>(__VA_ARGS__); break;              \
    default: st = FN<DIM, 0>(__VA_ARGS__); break;             \
  }

int pkv_launch_turbo_encode(const pkv_turbo_profile* p, const float* x, const PkvGeom& g,
                            uint8_t* payload, uint64_t* err, cudaStream_t s) {
  const int64_t grid = (int64_t)g.n_batches * g.tiles_per_batch;
  if (grid == 0) return PKV_OK;
  if (grid > 0x7fffffff) return PKV_ERR_UNSUPPORTED;
  const TurboParams tp = make_params(p);
  int st;
  if (p->cfg.dim == 64) {
    PKV_DISPATCH_PB(launch_encode, 64, tp, x, g, payload, err, (unsigned)grid, s)
  } else if (p->cfg.dim == 128) {
    PKV_DISPATCH_PB(launch_encode, 128, tp, x, g, payload, err, (unsigned)grid, s)
  } else {
    return PKV_ERR_UNSUPPORTED;
  }
  if (st != PKV_OK) return st;
  pkv_count_launch();
  return pkv_cuda_status(cudaGetLastError());
}

int pkv_launch_turbo_decode(const pkv_turbo_profile* p, const uint8_t* payload, const PkvGeom& g,
                            void* cache, int dst, uint64_t* err, cudaStream_t s) {
  const int64_t grid = (int64_t)g.n_batches * g.tiles_per_batch;
  if (grid == 0) return PKV_OK;
  if (grid > 0x7fffffff) return PKV_ERR_UNSUPPORTED;
  const TurboParams tp = make_params(p);
  int st;
  if (p->cfg.dim == 64) {
    PKV_DISPATCH_PB(launch_decode, 64, tp, payload, g, cache, dst, err, (unsigned)grid, s)
  } else if (p->cfg.dim == 128) {
    PKV_DISPATCH_PB(launch_decode, 128, tp, payload, g, cache, dst, err, (unsigned)grid, s)
  } else {
    return PKV_ERR_UNSUPPORTED;
  }
  if (st != PKV_OK) return st;
  pkv_count_launch();
  return pkv_cuda_status(cudaGetLastError());
}

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
