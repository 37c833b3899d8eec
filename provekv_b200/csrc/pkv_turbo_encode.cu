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
#include "pkv_turbo_encode.cuh"
#include "pkv_turbo_launch.cuh"

using namespace pkv_turbo;

namespace {

// ROT: the sketch in the rotated domain (PolarWithQjl, f32 radii, validated ray table, G'' present).
template <int D, int PB>
int launch_encode(const TurboParams& tp, const float* x, const PkvGeom& g, uint8_t* payload,
                  uint64_t* err, unsigned grid, cudaStream_t s) {
  const size_t sm = turbo_encode_smem<D>(tp);
  const unsigned ctas = (grid + TurboEnc<D>::NWARPS - 1) / TurboEnc<D>::NWARPS;  // one warp per 32-vector tile
  const bool rot = tp.mode == PKV_TURBO_POLAR_WITH_QJL && !tp.lossy && tp.fast_bucket && tp.qjl_rot != nullptr &&
                   !pkv_turbo_encode_legacy();
  int st;
  uint32_t* fix = nullptr;  // rot: counter + one entry per (vector, block of 32 projections), from the stream's pool
  const int64_t entries = (int64_t)g.n_batches * g.vpb * ((tp.projections + 31) / 32);
  if (rot) {
    cudaMemPool_t pool = pkv_scratch_pool();
    if (!pool) return PKV_ERR_CUDA;
    if (cudaError_t ce = cudaMallocFromPoolAsync((void**)&fix, sizeof(uint2) * (size_t)(entries + 1), pool, s))
      return pkv_cuda_status(ce);
    if (cudaError_t ce = cudaMemsetAsync(fix, 0, sizeof(uint32_t), s)) {
      cudaFreeAsync(fix, s);
      return pkv_cuda_status(ce);
    }
  }
  uint2* fix_list = reinterpret_cast<uint2*>(fix) + 1;
#define PKV_TURBO_ENC(DIRECT, ROT)                                                                        \
  {                                                                                                       \
    if ((st = set_smem(turbo_encode_kernel<D, PB, DIRECT, ROT>, sm)) != PKV_OK) return st;                \
    turbo_encode_kernel<D, PB, DIRECT, ROT><<<ctas, TurboEnc<D>::THREADS, sm, s>>>(g, tp, x, payload, err, fix, \
                                                                                    fix_list);             \
  }
  if (turbo_encode_direct(tp)) {
    if (rot) PKV_TURBO_ENC(true, true) else PKV_TURBO_ENC(true, false)
  } else {
    if (rot) PKV_TURBO_ENC(false, true) else PKV_TURBO_ENC(false, false)
  }
  if (rot) {
    const size_t fsm = sizeof(float) * ((size_t)tp.projections * (D + 1) + 2 * (1u << tp.polar_bits) + 4 * D);
    turbo_encode_fix_kernel<D><<<148 * 4, 128, fsm, s>>>(g, tp, x, payload, err, fix, fix_list);
    pkv_count_launch();
    if (cudaError_t ce = cudaFreeAsync(fix, s)) return pkv_cuda_status(ce);
  }
#undef PKV_TURBO_ENC
  return PKV_OK;
}

}  // namespace

int pkv_turbo_tile_vectors(int dim) { return (dim == 64 || dim == 128) ? 32 : 0; }

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

int pkv_turbo_stats_copy(unsigned long long* out, int reset) {
  static const unsigned long long zeros[4] = {0, 0, 0, 0};
  if (out && cudaMemcpyFromSymbol(out, pkv_turbo::g_turbo_stats, sizeof(zeros)) != cudaSuccess) return PKV_ERR_CUDA;
  if (reset && cudaMemcpyToSymbol(pkv_turbo::g_turbo_stats, zeros, sizeof(zeros)) != cudaSuccess) return PKV_ERR_CUDA;
  return PKV_OK;
}
