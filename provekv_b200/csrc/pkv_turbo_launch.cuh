// Host-side pieces shared by the three turbo-quant translation units (encode, decode, score):
// kernel parameters from a profile, the dynamic shared-memory opt-in, the dispatch on the angle width.
#pragma once

#include "pkv_turbo_common.cuh"

namespace pkv_turbo {

inline TurboParams make_params(const pkv_turbo_profile* p) {
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
  tp.qjl_rot = p->qjl_rot_dev;
  tp.lut = p->lut_dev;
  tp.logf_table = p->logf_table;
  tp.expf_table = p->expf_table;
  return tp;
}


template <typename F>
int set_smem(F kernel, size_t bytes) {
  if (bytes > 48 * 1024)
    return pkv_cuda_status(
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return PKV_OK;
}


}  // namespace pkv_turbo

#define PKV_DISPATCH_PB(FN, DIM, ...)                         \
  switch (tp.polar_bits) {                                    \
    case 3: st = FN<DIM, 3>(__VA_ARGS__); break;              \
    case 4: st = FN<DIM, 4>(__VA_ARGS__); break;              \
    case 7: st = FN<DIM, 7>(__VA_ARGS__); break;              \
    default: st = FN<DIM, 0>(__VA_ARGS__); break;             \
  }

