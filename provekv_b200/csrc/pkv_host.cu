// Host side of the C ABI (include/provekv_b200.h): profiles, launch geometry,
// the host-buffer "*_batch_compact" calls and the FB2 / TQB1 headers.
#include <math.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <new>

#include "pkv_common.cuh"
#include "pkv_fast_paths.h"

namespace {

std::atomic<int64_t> g_launches{0};
std::atomic<int> g_skip_tensor_issue{0};
std::atomic<float*> g_rotated_capture{nullptr};
std::atomic<int> g_turbo_encode_legacy{0};

int grow(void** ptr, int64_t* cap, int64_t need) {
  if (need <= *cap) return PKV_OK;
  if (*ptr) cudaFree(*ptr);
  *ptr = nullptr;
  *cap = 0;
  int64_t want = need + need / 4 + 256;
  cudaError_t e = cudaMalloc(ptr, (size_t)want);
  if (e != cudaSuccess) return pkv_cuda_status(e);
  *cap = want;
  return PKV_OK;
}

}  // namespace

int pkv_ws_prepare(PkvWorkspace* ws, int64_t in_bytes, int64_t out_bytes) {
  int st;
  if ((st = grow(&ws->in, &ws->in_cap, in_bytes)) != PKV_OK) return st;
  if ((st = grow(&ws->out, &ws->out_cap, out_bytes)) != PKV_OK) return st;
  if (!ws->err) {
    cudaError_t e = cudaMalloc((void**)&ws->err, sizeof(uint64_t) * PKV_WS_ERR_WORDS);
    if (e != cudaSuccess) return pkv_cuda_status(e);
  }
  return PKV_OK;
}

namespace {

void ws_release(PkvWorkspace* ws) {
  if (ws->in) cudaFree(ws->in);
  if (ws->out) cudaFree(ws->out);
  if (ws->err) cudaFree(ws->err);
  for (int i = 0; i < PKV_WS_STREAMS; i++)
    if (ws->streams[i]) cudaStreamDestroy(ws->streams[i]);
  *ws = PkvWorkspace();
}


// Validate a layout and derive the launch geometry for tiles of `tile` vectors.
int make_geom(const pkv_layout* L, int rec_bytes, int64_t payload_batch_stride, int tile,
              bool encode, PkvGeom* g) {
  if (!L) return PKV_ERR_INVALID_ARGUMENT;
  if (L->n_tokens < 0 || L->n_heads <= 0 || L->n_replicas < 1) return PKV_ERR_INVALID_ARGUMENT;
  if (encode && L->n_replicas != 1) return PKV_ERR_INVALID_ARGUMENT;
  int64_t nb = 1;
  for (int i = 0; i < 3; i++) {
    if (L->n_batches[i] < 1) return PKV_ERR_INVALID_ARGUMENT;
    nb *= L->n_batches[i];
    if (L->batch_stride[i] % 4) return PKV_ERR_INVALID_ARGUMENT;
  }
  if (L->base % 4 || L->token_stride % 4 || L->head_stride % 4 || L->replica_stride % 4)
    return PKV_ERR_INVALID_ARGUMENT;
  const int64_t vpb = (int64_t)L->n_tokens * L->n_heads;
  if (vpb * nb >= (int64_t)1 << 31 || nb >= (int64_t)1 << 31) return PKV_ERR_UNSUPPORTED;
  if (payload_batch_stride % 16 || payload_batch_stride < vpb * rec_bytes)
    return PKV_ERR_INVALID_ARGUMENT;
  g->L = *L;
  g->payload_batch_stride = payload_batch_stride;
  g->vpb = (int32_t)vpb;
  g->tiles_per_batch = (int32_t)((vpb + tile - 1) / tile);
  g->n_batches = (int32_t)nb;
  g->rec_bytes = rec_bytes;
  g->batch_offsets = nullptr;
  return PKV_OK;
}

// 16-bit caches are written 16 bytes at a time: offsets in multiples of 8 elements.
int check_dst(const pkv_layout* L, int dst) {
  if (dst == PKV_DST_F32) return PKV_OK;
  if (dst != PKV_DST_F16 && dst != PKV_DST_BF16) return PKV_ERR_INVALID_ARGUMENT;
  int64_t all = L->base | L->token_stride | L->head_stride | L->replica_stride;
  for (int i = 0; i < 3; i++) all |= L->batch_stride[i];
  return (all % 8) ? PKV_ERR_INVALID_ARGUMENT : PKV_OK;
}

pkv_layout flat_layout(int64_t n, int dim) {
  pkv_layout L;
  memset(&L, 0, sizeof(L));
  L.n_batches[0] = L.n_batches[1] = L.n_batches[2] = 1;
  L.n_tokens = (int32_t)n;
  L.n_heads = 1;
  L.token_stride = dim;
  L.head_stride = dim;
  L.n_replicas = 1;
  return L;
}

int decode_err_word(uint64_t w, int32_t* code, int64_t* index) {
  if (w == PKV_ERR_NONE) {
    if (code) *code = 0;
    if (index) *index = -1;
    return PKV_OK;
  }
  const int c = (int)(w & 0xff);
  if (code) *code = c;
  if (index) *index = (int64_t)((w >> 8) & 0xFFFFFFFFFFFFull);
  return c;
}

// encode_pair's bucket before the modulo (turbo-quant/src/polar.rs:415-420), on the host.
uint32_t raw_bucket_host(float theta, uint32_t levels) {
  const float pi = 3.14159274101257324f;
  volatile float sum = theta + pi;
  volatile float normalized = sum / (2.0f * pi);
  volatile float scaled = normalized * (float)levels;
  const float fl = floorf(scaled);
  return fl <= 0.0f ? 0u : (uint32_t)fl;
}

// For k = 1..levels find T_k, the smallest binary32 theta whose raw bucket is >= k (the bucket
// is monotone in theta), and check that the point where a correctly rounded angle crosses it --
// the midpoint of T_k and its predecessor -- is within 2e-6 rad of the ideal ray -pi + 2 pi k / L.
bool turbo_bucket_boundaries_ok(int levels) {
  auto key = [](float f) {  // order-preserving map of binary32 to int64
    uint32_t u;
    memcpy(&u, &f, 4);
    return (u & 0x80000000u) ? -(int64_t)(u & 0x7fffffffu) : (int64_t)u;
  };
  auto unkey = [](int64_t k) {
    uint32_t u = k < 0 ? (0x80000000u | (uint32_t)(-k)) : (uint32_t)k;
    float f;
    memcpy(&f, &u, 4);
    return f;
  };
  for (int k = 1; k <= levels; k++) {
    int64_t lo = key(-3.2f), hi = key(3.2f);  // bucket(lo) < k <= bucket(hi)
    if (raw_bucket_host(unkey(hi), (uint32_t)levels) < (uint32_t)k) return false;
    while (hi - lo > 1) {
      const int64_t mid = lo + (hi - lo) / 2;
      if (raw_bucket_host(unkey(mid), (uint32_t)levels) >= (uint32_t)k) hi = mid;
      else lo = mid;
    }
    const double boundary = 0.5 * ((double)unkey(lo) + (double)unkey(hi));
    const double ideal = -M_PI + 2.0 * M_PI * (double)k / (double)levels;
    if (fabs(boundary - ideal) > 2.0e-6) return false;
  }
  return true;
}

int fib_index_bits(int n) {  // fib-quant/src/profile.rs:268-274
  int b = 1;
  while ((1 << b) < n) b++;
  return b;
}

}  // namespace

namespace {
thread_local cudaError_t t_last_cuda_error = cudaSuccess;
}
// The library's own stream-ordered memory pool, one per device, created on first use.  Its
// release threshold is unlimited, so the scratch of one call is recycled by the next instead
// of being returned to the driver at every synchronisation.
cudaMemPool_t pkv_scratch_pool() {
  static std::mutex mu;
  static cudaMemPool_t pools[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!pools[dev]) {
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = dev;
    cudaMemPool_t pool = nullptr;
    if (cudaMemPoolCreate(&pool, &props) != cudaSuccess) return nullptr;
    uint64_t keep = ~0ull;
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    pools[dev] = pool;
  }
  return pools[dev];
}

int pkv_cuda_status(cudaError_t e) {
  if (e == cudaSuccess) return PKV_OK;
  t_last_cuda_error = e;
  return PKV_ERR_CUDA;
}
// A profile's tables live on the device that was current when it was created; a launch from another
// device would hand that device's kernels pointers they cannot reach.  Checked before anything is
// launched or copied.
int pkv_check_device(int profile_device) {
  int cur = -1;
  if (cudaError_t ce = cudaGetDevice(&cur)) return pkv_cuda_status(ce);
  return cur == profile_device ? PKV_OK : PKV_ERR_INVALID_ARGUMENT;
}
int pkv_make_geom(const pkv_layout* L, int rec_bytes, int64_t payload_batch_stride, int tile,
                  bool encode, PkvGeom* g) {
  return make_geom(L, rec_bytes, payload_batch_stride, tile, encode, g);
}
void pkv_count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
int pkv_skip_tensor_issue() { return g_skip_tensor_issue.load(std::memory_order_relaxed); }
float* pkv_rotated_capture() { return g_rotated_capture.load(std::memory_order_relaxed); }
int pkv_turbo_encode_legacy() { return g_turbo_encode_legacy.load(std::memory_order_relaxed); }

extern "C" {

int64_t pkv_launch_count(void) { return g_launches.load(); }
const char* pkv_last_cuda_error(void) {
  return t_last_cuda_error == cudaSuccess ? "" : cudaGetErrorString(t_last_cuda_error);
}
int pkv_test_turbo_encode_legacy(int on) {
  g_turbo_encode_legacy.store(on ? 1 : 0);
  return PKV_OK;
}
int pkv_test_capture_rotated(float* rotated_dev) {
  g_rotated_capture.store(rotated_dev, std::memory_order_relaxed);
  return PKV_OK;
}

int pkv_test_skip_tensor_issue(int on) {
  g_skip_tensor_issue.store(on ? 1 : 0);
  return PKV_OK;
}
int pkv_version(void) { return 100; }

const char* pkv_status_string(int s) {
  switch (s) {
    case PKV_OK: return "ok";
    case PKV_ERR_INVALID_ARGUMENT: return "invalid argument";
    case PKV_ERR_CUDA: return "CUDA error (no usable device, out of memory or launch failure)";
    case PKV_ERR_UNSUPPORTED: return "shape not supported by the kernels";
    case PKV_ERR_EMPTY_BATCH: return "empty batch";
    case PKV_ERR_CORRUPT_HEADER: return "corrupt or mismatching wire header";
    case PKV_ERR_BUFFER_TOO_SMALL: return "output buffer too small";
    case PKV_ERR_STATIC_SCRATCH_TOO_SMALL:
      return "too many vectors for the fixed scratch array of pkv_fib_encode_dev_static";
    case PKV_VEC_MISALIGNED_DST:
      return "cache tensor offset is negative or not a multiple of 16 bytes";
    case PKV_VEC_NONFINITE_INPUT: return "non-finite input value";
    case PKV_VEC_ZERO_NORM: return "zero-norm vector";
    case PKV_VEC_BAD_RADIUS: return "radius is not finite and non-negative";
    case PKV_VEC_BAD_RADIUS_RANGE: return "radius codec range is malformed";
    case PKV_VEC_PADDING_BITS: return "nonzero padding bits";
    case PKV_VEC_INDEX_RANGE: return "codeword index out of range";
    case PKV_VEC_BAD_NORM: return "invalid stored norm";
    case PKV_VEC_NONFINITE_OUTPUT: return "non-finite decoded value";
    case PKV_VEC_NONFINITE_RESIDUAL: return "non-finite residual";
    case PKV_VEC_NORM_RANGE: return "norm not representable in the wire norm format";
    case PKV_VEC_DEVICE_WAIT: return "a wait inside a kernel ran out; the output is not valid";
    default: return "unknown status";
  }
}

int pkv_device_count(int* count) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (count) *count = e == cudaSuccess ? n : 0;
  return pkv_cuda_status(e);
}
int pkv_set_device(int device) { return pkv_cuda_status(cudaSetDevice(device)); }
int pkv_host_alloc(void** ptr, int64_t bytes) { return pkv_cuda_status(cudaMallocHost(ptr, (size_t)bytes)); }
int pkv_host_free(void* ptr) { return pkv_cuda_status(cudaFreeHost(ptr)); }
int pkv_dev_alloc(void** ptr, int64_t bytes) { return pkv_cuda_status(cudaMalloc(ptr, (size_t)bytes)); }
int pkv_dev_free(void* ptr) { return pkv_cuda_status(cudaFree(ptr)); }
int pkv_memcpy_h2d(void* d, const void* s, int64_t n, void* stream) {
  return pkv_cuda_status(cudaMemcpyAsync(d, s, (size_t)n, cudaMemcpyHostToDevice, (cudaStream_t)stream));
}
int pkv_memcpy_d2h(void* d, const void* s, int64_t n, void* stream) {
  return pkv_cuda_status(cudaMemcpyAsync(d, s, (size_t)n, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
}
int pkv_stream_synchronize(void* stream) { return pkv_cuda_status(cudaStreamSynchronize((cudaStream_t)stream)); }

// Records of `n_batches` wire blobs between host memory (blob b at blobs_host + b * blob_bytes, its
// records after header_bytes) and a device payload buffer (batch b at payload_dev + b * stride).
int pkv_payload_upload(const uint8_t* blobs_host, int64_t blob_bytes, int32_t header_bytes, int64_t n_batches,
                       int64_t record_bytes_per_batch, uint8_t* payload_dev, int64_t payload_batch_stride,
                       void* stream) {
  if (!blobs_host || !payload_dev || n_batches < 0 || header_bytes < 0 || record_bytes_per_batch < 0 ||
      blob_bytes < header_bytes + record_bytes_per_batch || payload_batch_stride < record_bytes_per_batch)
    return PKV_ERR_INVALID_ARGUMENT;
  if (n_batches == 0 || record_bytes_per_batch == 0) return PKV_OK;
  return pkv_cuda_status(cudaMemcpy2DAsync(payload_dev, (size_t)payload_batch_stride, blobs_host + header_bytes,
                                           (size_t)blob_bytes, (size_t)record_bytes_per_batch, (size_t)n_batches,
                                           cudaMemcpyHostToDevice, (cudaStream_t)stream));
}
int pkv_payload_download(const uint8_t* payload_dev, int64_t payload_batch_stride, int64_t n_batches,
                         int64_t record_bytes_per_batch, uint8_t* blobs_host, int64_t blob_bytes,
                         int32_t header_bytes, void* stream) {
  if (!blobs_host || !payload_dev || n_batches < 0 || header_bytes < 0 || record_bytes_per_batch < 0 ||
      blob_bytes < header_bytes + record_bytes_per_batch || payload_batch_stride < record_bytes_per_batch)
    return PKV_ERR_INVALID_ARGUMENT;
  if (n_batches == 0 || record_bytes_per_batch == 0) return PKV_OK;
  return pkv_cuda_status(cudaMemcpy2DAsync(blobs_host + header_bytes, (size_t)blob_bytes, payload_dev,
                                           (size_t)payload_batch_stride, (size_t)record_bytes_per_batch,
                                           (size_t)n_batches, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
}

int pkv_error_word_reset(uint64_t* err_dev, void* stream) {
  return pkv_cuda_status(cudaMemsetAsync(err_dev, 0xFF, sizeof(uint64_t), (cudaStream_t)stream));
}
int pkv_error_word_read(const uint64_t* err_dev, void* stream, int32_t* code, int64_t* index) {
  uint64_t w = 0;
  cudaError_t e = cudaMemcpyAsync(&w, err_dev, sizeof(w), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return pkv_cuda_status(e);
  return decode_err_word(w, code, index);
}

// ---------------------------------------------------------------------------
// fib-quant
// ---------------------------------------------------------------------------

int pkv_fib_profile_create(const pkv_fib_config* cfg, const double* rotation, const float* codebook,
                           pkv_fib_profile** out) {
  if (!cfg || !rotation || !codebook || !out) return PKV_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  if (cfg->dim <= 0 || cfg->block_dim <= 0 || cfg->dim % cfg->block_dim || cfg->codebook_size < 2)
    return PKV_ERR_INVALID_ARGUMENT;
  if ((cfg->dim != 64 && cfg->dim != 128) || cfg->block_dim != 4 || cfg->codebook_size > 32)
    return PKV_ERR_UNSUPPORTED;
  if (cfg->norm_format < 0 || cfg->norm_format > 1 || cfg->argmin_order < 0 ||
      cfg->argmin_order > 1 || cfg->numerics < 0 || cfg->numerics > 2)
    return PKV_ERR_INVALID_ARGUMENT;
  pkv_fib_profile* p = new (std::nothrow) pkv_fib_profile();
  if (!p) return PKV_ERR_CUDA;
  p->cfg = *cfg;
  p->blocks = cfg->dim / cfg->block_dim;
  p->idx_bits = fib_index_bits(cfg->codebook_size);
  p->norm_len = cfg->norm_format == PKV_NORM_FP16 ? 2 : 4;
  p->idx_len = (p->blocks * p->idx_bits + 7) / 8;
  p->rec_bytes = p->norm_len + p->idx_len;
  p->rot_t_dev = nullptr;
  p->rot32_dev = nullptr;
  p->codebook_dev = nullptr;
  p->rot_dev = nullptr;
  p->rot32_t_dev = nullptr;
  p->half_norm_dev = nullptr;
  p->rot_hi_dev = nullptr;
  p->rot_lo_dev = nullptr;
  p->hadamard = 0;
  memset(p->wht_sgn_scale, 0, sizeof(p->wht_sgn_scale));
  const int d = cfg->dim;
  // The error bounds of the shortcut encoders (pkv_fast_paths.h) take |M_r|_2 = 1 and an orthogonal
  // M.  A table that is not (scaled, truncated, not a rotation at all) is still a valid input of the
  // reference's arithmetic, so the profile is kept but encodes with the exact f64 kernel only.
  p->orthonormal = 1;
  for (int r = 0; r < d && p->orthonormal; r++)
    for (int q = r; q < d; q++) {
      double dot = 0.0;
      for (int j = 0; j < d; j++) dot += rotation[r * d + j] * rotation[q * d + j];
      if (!(fabs(dot - (r == q ? 1.0 : 0.0)) < 1.0e-6)) {  // also catches NaN
        p->orthonormal = 0;
        break;
      }
    }
  cudaError_t e = cudaGetDevice(&p->device);
  double* rt = new double[d * d];
  float* r32 = new float[d * d];
  float cb[128];
  memset(cb, 0, sizeof(cb));
  for (int r = 0; r < d; r++)
    for (int j = 0; j < d; j++) {
      rt[j * d + r] = rotation[r * d + j];
      r32[r * d + j] = (float)rotation[r * d + j];  // fib-quant/src/rotation.rs:139
    }
  memcpy(cb, codebook, sizeof(float) * 4 * cfg->codebook_size);
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->rot_t_dev, sizeof(double) * d * d);
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->rot32_dev, sizeof(float) * d * d);
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->codebook_dev, sizeof(cb));
  if (e == cudaSuccess) e = cudaMemcpy(p->rot_t_dev, rt, sizeof(double) * d * d, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(p->rot32_dev, r32, sizeof(float) * d * d, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(p->codebook_dev, cb, sizeof(cb), cudaMemcpyHostToDevice);
  // tables of the shortcut encoder: f64 matrix row-major, f32 matrix transposed, |c|^2 / 2
  float hn[32];
  for (int c = 0; c < 32; c++) {
    double s = 0.0;
    for (int j = 0; j < 4; j++) s += (double)cb[4 * c + j] * (double)cb[4 * c + j];
    hn[c] = (float)(0.5 * s);
  }
  p->score_abs = pkv_fib_score_abs(cb, cfg->codebook_size);
  // Bias of the Hadamard encoder's score search (pkv_fast_paths.h (3b)); 2e30 marks a codebook that no
  // binade can hold (pkv_fib_profile_create_hadamard refuses it)
  p->search_off = 2.0e30f;
  p->search_ef = 0.0f;
  p->search_quick_gap = 0xffffffffu;
  if (!pkv_fib_search_bias(cb, cfg->codebook_size, 0.0, &p->search_off, &p->search_ef, &p->search_quick_gap))
    p->search_off = 2.0e30f;
  for (int r = 0; r < d; r++)
    for (int j = 0; j < d; j++) r32[j * d + r] = (float)rotation[r * d + j];
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->rot_dev, sizeof(double) * d * d);
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->rot32_t_dev, sizeof(float) * d * d);
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->half_norm_dev, sizeof(hn));
  if (e == cudaSuccess) e = cudaMemcpy(p->rot_dev, rotation, sizeof(double) * d * d, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(p->rot32_t_dev, r32, sizeof(float) * d * d, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(p->half_norm_dev, hn, sizeof(hn), cudaMemcpyHostToDevice);
  {  // split of the f32 matrix for the tensor-core rotation: hi keeps 11 significant bits, lo is exact
    float* hi = new float[d * d];
    float* lo = new float[d * d];
    for (int i = 0; i < d * d; i++) {
      const float m = (float)rotation[i];
      uint32_t u;
      memcpy(&u, &m, 4);
      u &= 0xffffe000u;
      memcpy(&hi[i], &u, 4);
      lo[i] = m - hi[i];
    }
    if (e == cudaSuccess) e = cudaMalloc((void**)&p->rot_hi_dev, sizeof(float) * d * d);
    if (e == cudaSuccess) e = cudaMalloc((void**)&p->rot_lo_dev, sizeof(float) * d * d);
    if (e == cudaSuccess) e = cudaMemcpy(p->rot_hi_dev, hi, sizeof(float) * d * d, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(p->rot_lo_dev, lo, sizeof(float) * d * d, cudaMemcpyHostToDevice);
    delete[] hi;
    delete[] lo;
  }
  delete[] rt;
  delete[] r32;
  if (e != cudaSuccess) {
    pkv_fib_profile_destroy(p);
    return PKV_ERR_CUDA;
  }
  *out = p;
  return PKV_OK;
}

// generate_signs_impl, gpu-backend/src/fallback.rs:76-88: one step of the 64-bit LCG per coordinate,
// bit 32 of the state picks the sign; the scale is `1.0 / (dim as f32).sqrt()` (:52).
static void wht_signed_scale(int dim, uint64_t seed, float* out) {
  const float scale = 1.0f / sqrtf((float)dim);
  uint64_t state = seed;
  for (int i = 0; i < dim; i++) {
    state = state * 6364136223846793005ull + 1442695040888963407ull;
    out[i] = ((state >> 32) & 1) ? scale : -scale;
  }
}

int pkv_fib_profile_create_hadamard(const pkv_fib_config* cfg, uint64_t rotation_seed, const double* rotation,
                                    const float* codebook, pkv_fib_profile** out) {
  if (!cfg || !codebook || !out) return PKV_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  if (cfg->numerics == PKV_FIB_NUMERICS_SINGLE) return PKV_ERR_INVALID_ARGUMENT;  // the transform exists in encode_batch only
  if (cfg->dim != 64 && cfg->dim != 128) return cfg->dim > 0 ? PKV_ERR_UNSUPPORTED : PKV_ERR_INVALID_ARGUMENT;
  const int d = cfg->dim;
  float ss[128];
  wht_signed_scale(d, rotation_seed, ss);
  double* own = nullptr;
  if (!rotation) {
    // the transform written out as a matrix, M[r][j] = ss[r] * (-1)^popcount(r & j), so that the decoders
    // invert what this profile's encoder applied
    own = new (std::nothrow) double[(size_t)d * d];
    if (!own) return PKV_ERR_CUDA;
    for (int r = 0; r < d; r++)
      for (int j = 0; j < d; j++) own[r * d + j] = (__builtin_popcount(r & j) & 1) ? -(double)ss[r] : (double)ss[r];
  }
  const int st = pkv_fib_profile_create(cfg, rotation ? rotation : own, codebook, out);
  delete[] own;
  if (st != PKV_OK) return st;
  if (!((*out)->search_off < 1.0e30f)) {  // no bias fits this codebook, and this encoder has no exact kernel behind it
    pkv_fib_profile_destroy(*out);
    *out = nullptr;
    return PKV_ERR_UNSUPPORTED;
  }
  (*out)->hadamard = 1;
  memcpy((*out)->wht_sgn_scale, ss, sizeof(float) * d);
  return PKV_OK;
}

int pkv_fib_profile_destroy(pkv_fib_profile* p) {
  if (!p) return PKV_OK;
  if (p->rot_t_dev) cudaFree(p->rot_t_dev);
  if (p->rot32_dev) cudaFree(p->rot32_dev);
  if (p->codebook_dev) cudaFree(p->codebook_dev);
  if (p->rot_dev) cudaFree(p->rot_dev);
  if (p->rot32_t_dev) cudaFree(p->rot32_t_dev);
  if (p->half_norm_dev) cudaFree(p->half_norm_dev);
  if (p->rot_hi_dev) cudaFree(p->rot_hi_dev);
  if (p->rot_lo_dev) cudaFree(p->rot_lo_dev);
  ws_release(&p->ws);
  delete p;
  return PKV_OK;
}

int32_t pkv_fib_record_bytes(const pkv_fib_profile* p) { return p ? p->rec_bytes : 0; }

int pkv_fib_encode_dev(const pkv_fib_profile* p, const float* x_dev, const pkv_layout* layout,
                       uint8_t* payload_dev, int64_t payload_batch_stride, uint64_t* err_dev,
                       void* stream) {
  if (!p || !x_dev || !payload_dev || !err_dev) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (((uintptr_t)x_dev | (uintptr_t)payload_dev) & 15) return PKV_ERR_INVALID_ARGUMENT;
  PkvGeom g;
  int st = make_geom(layout, p->rec_bytes, payload_batch_stride, pkv_fib_tile_vectors(p->cfg.dim, 1), true, &g);
  if (st != PKV_OK) return st;
  if (g.vpb == 0) return PKV_ERR_EMPTY_BATCH;
  const int batch_numerics = p->cfg.numerics == PKV_FIB_NUMERICS_BATCH ||
                             (p->cfg.numerics == PKV_FIB_NUMERICS_AUTO && g.vpb >= 4);
  return pkv_launch_fib_encode(p, x_dev, g, payload_dev, err_dev, batch_numerics, (cudaStream_t)stream);
}

int pkv_fib_decode_patch_dev(const pkv_fib_profile* p, const uint8_t* payload_dev,
                             int64_t payload_batch_stride, const pkv_layout* layout,
                             float* cache_dev, uint64_t* err_dev, void* stream) {
  if (!p || !cache_dev || !payload_dev || !err_dev) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (((uintptr_t)cache_dev | (uintptr_t)payload_dev) & 15) return PKV_ERR_INVALID_ARGUMENT;
  PkvGeom g;
  int st = make_geom(layout, p->rec_bytes, payload_batch_stride, pkv_fib_tile_vectors(p->cfg.dim, 0), false, &g);
  if (st != PKV_OK) return st;
  return pkv_launch_fib_decode(p, payload_dev, g, cache_dev, PKV_DST_F32, err_dev, (cudaStream_t)stream);
}

int pkv_fib_decode_patch_dev_as(const pkv_fib_profile* p, const uint8_t* payload_dev,
                                int64_t payload_batch_stride, const pkv_layout* layout,
                                void* cache_dev, int32_t dst_dtype, uint64_t* err_dev, void* stream) {
  if (!p || !cache_dev || !payload_dev || !err_dev) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (((uintptr_t)cache_dev | (uintptr_t)payload_dev) & 15) return PKV_ERR_INVALID_ARGUMENT;
  PkvGeom g;
  int st = make_geom(layout, p->rec_bytes, payload_batch_stride, pkv_fib_tile_vectors(p->cfg.dim, 0), false, &g);
  if (st == PKV_OK) st = check_dst(layout, dst_dtype);
  if (st != PKV_OK) return st;
  return pkv_launch_fib_decode(p, payload_dev, g, cache_dev, dst_dtype, err_dev, (cudaStream_t)stream);
}

int pkv_fib_decode_patch_dev_multi(const pkv_fib_profile* p, const uint8_t* payload_dev,
                                   int64_t payload_batch_stride, const pkv_layout* layout,
                                   void* cache_dev, const int64_t* batch_offsets_dev, int32_t dst_dtype,
                                   uint64_t* err_dev, void* stream) {
  if (!p || !cache_dev || !payload_dev || !err_dev || !batch_offsets_dev) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (((uintptr_t)cache_dev | (uintptr_t)payload_dev) & 15) return PKV_ERR_INVALID_ARGUMENT;
  PkvGeom g;
  int st = make_geom(layout, p->rec_bytes, payload_batch_stride, pkv_fib_tile_vectors(p->cfg.dim, 0), false, &g);
  if (st == PKV_OK) st = check_dst(layout, dst_dtype);
  if (st != PKV_OK) return st;
  g.batch_offsets = batch_offsets_dev;
  return pkv_launch_fib_decode(p, payload_dev, g, cache_dev, dst_dtype, err_dev, (cudaStream_t)stream);
}

int pkv_fib_decode_exact_dev(const pkv_fib_profile* p, const uint8_t* payload_dev, int64_t payload_batch_stride,
                             const pkv_layout* layout, float* out_dev, uint64_t* err_dev, void* stream) {
  if (!p || !out_dev || !payload_dev || !err_dev) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (((uintptr_t)out_dev | (uintptr_t)payload_dev) & 15) return PKV_ERR_INVALID_ARGUMENT;
  PkvGeom g;
  int st = make_geom(layout, p->rec_bytes, payload_batch_stride, pkv_fib_tile_vectors(p->cfg.dim, 0), false, &g);
  if (st != PKV_OK) return st;
  if (layout->n_replicas != 1) return PKV_ERR_INVALID_ARGUMENT;
  return pkv_launch_fib_decode_exact(p, payload_dev, g, out_dev, err_dev, (cudaStream_t)stream);
}

// FibQuantizer::decode for n records in host memory (no header), n small: one upload, one launch.
int pkv_fib_decode_exact(const pkv_fib_profile* cp, const uint8_t* records_host, int64_t n, float* out_host,
                         int32_t* vec_code, int64_t* vec_index) {
  pkv_fib_profile* p = const_cast<pkv_fib_profile*>(cp);
  if (!p || !records_host || !out_host || n < 0) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (vec_code) *vec_code = 0;
  if (vec_index) *vec_index = -1;
  if (n == 0) return PKV_OK;
  if (n >= (int64_t)1 << 31) return PKV_ERR_UNSUPPORTED;
  const int d = p->cfg.dim;
  std::lock_guard<std::mutex> lock(p->ws_mutex);
  int st = pkv_ws_prepare(&p->ws, n * p->rec_bytes + 16, n * d * 4);
  if (st != PKV_OK) return st;
  cudaStream_t s = 0;
  pkv_layout L = flat_layout(n, d);
  const int64_t stride = (n * p->rec_bytes + 15) / 16 * 16;
  if (cudaError_t ce = cudaMemcpyAsync(p->ws.in, records_host, (size_t)n * p->rec_bytes, cudaMemcpyHostToDevice, s))
    return pkv_cuda_status(ce);
  pkv_error_word_reset(p->ws.err, s);
  st = pkv_fib_decode_exact_dev(p, (const uint8_t*)p->ws.in, stride, &L, (float*)p->ws.out, p->ws.err, s);
  if (st != PKV_OK) return st;
  if (cudaError_t ce = cudaMemcpyAsync(out_host, p->ws.out, (size_t)n * d * 4, cudaMemcpyDeviceToHost, s))
    return pkv_cuda_status(ce);
  return pkv_error_word_read(p->ws.err, s, vec_code, vec_index);
}

int pkv_fb2_header_write(const pkv_fib_profile* p, uint32_t n_vectors, uint8_t* out) {
  if (!p || !out) return PKV_ERR_INVALID_ARGUMENT;
  const uint32_t blocks = (uint32_t)p->blocks;
  const uint16_t nl = (uint16_t)p->norm_len, il = (uint16_t)p->idx_len;
  out[0] = 'F'; out[1] = 'B'; out[2] = '2'; out[3] = 1;
  out[4] = (uint8_t)p->idx_bits;
  out[5] = 0;
  memcpy(out + 6, &blocks, 4);
  memcpy(out + 10, &n_vectors, 4);
  out[14] = (uint8_t)p->cfg.norm_format;
  memcpy(out + 15, &nl, 2);
  memcpy(out + 17, &il, 2);
  return PKV_OK;
}

int pkv_fb2_header_parse(const pkv_fib_profile* p, const uint8_t* b, int64_t len, uint32_t* n_vectors) {
  if (!p || !b || !n_vectors) return PKV_ERR_INVALID_ARGUMENT;
  if (len < PKV_FB2_HEADER_BYTES) return PKV_ERR_CORRUPT_HEADER;
  if (b[0] != 'F' || b[1] != 'B' || b[2] != '2' || b[3] != 1) return PKV_ERR_CORRUPT_HEADER;
  uint32_t blocks, n;
  uint16_t nl, il;
  memcpy(&blocks, b + 6, 4);
  memcpy(&n, b + 10, 4);
  memcpy(&nl, b + 15, 2);
  memcpy(&il, b + 17, 2);
  if (b[4] != p->idx_bits || blocks != (uint32_t)p->blocks) return PKV_ERR_CORRUPT_HEADER;
  if (b[14] != p->cfg.norm_format) return PKV_ERR_CORRUPT_HEADER;
  if (nl != p->norm_len || il != p->idx_len) return PKV_ERR_CORRUPT_HEADER;
  if (len < PKV_FB2_HEADER_BYTES + (int64_t)n * (nl + il)) return PKV_ERR_CORRUPT_HEADER;
  *n_vectors = n;
  return PKV_OK;
}

int pkv_fib_encode_batch_compact(const pkv_fib_profile* cp, const float* vectors_host, int64_t n,
                                 uint8_t* out_host, int64_t out_capacity, int64_t* out_len,
                                 int32_t* vec_code, int64_t* vec_index) {
  pkv_fib_profile* p = const_cast<pkv_fib_profile*>(cp);
  if (!p || !out_host || !out_len || n < 0 || (n > 0 && !vectors_host)) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (vec_code) *vec_code = 0;
  if (vec_index) *vec_index = -1;
  *out_len = 0;
  if (n == 0) return PKV_ERR_EMPTY_BATCH;  // FibCodeV1::encode_batch, fib-quant/src/codec.rs:226
  if (n >= (int64_t)1 << 31) return PKV_ERR_UNSUPPORTED;
  const int d = p->cfg.dim;
  const int64_t total = PKV_FB2_HEADER_BYTES + n * p->rec_bytes;
  if (out_capacity < total) return PKV_ERR_BUFFER_TOO_SMALL;
  std::lock_guard<std::mutex> lock(p->ws_mutex);
  int st = pkv_ws_prepare(&p->ws, n * d * 4, n * p->rec_bytes + 16);
  if (st != PKV_OK) return st;
  cudaStream_t s = 0;
  pkv_layout L = flat_layout(n, d);
  const int64_t stride = (n * p->rec_bytes + 15) / 16 * 16;
  if (cudaError_t ce = cudaMemcpyAsync(p->ws.in, vectors_host, (size_t)n * d * 4, cudaMemcpyHostToDevice, s)) return pkv_cuda_status(ce);
  pkv_error_word_reset(p->ws.err, s);
  st = pkv_fib_encode_dev(p, (const float*)p->ws.in, &L, (uint8_t*)p->ws.out, stride, p->ws.err, s);
  if (st != PKV_OK) return st;
  if (cudaError_t ce = cudaMemcpyAsync(out_host + PKV_FB2_HEADER_BYTES, p->ws.out, (size_t)n * p->rec_bytes,
                      cudaMemcpyDeviceToHost, s)) return pkv_cuda_status(ce);
  st = pkv_error_word_read(p->ws.err, s, vec_code, vec_index);
  if (st != PKV_OK) return st;
  pkv_fb2_header_write(p, (uint32_t)n, out_host);
  *out_len = total;
  return PKV_OK;
}

int pkv_fib_decode_batch_compact(const pkv_fib_profile* cp, const uint8_t* bytes_host, int64_t len,
                                 float* out_host, int64_t out_capacity_floats, int64_t* n_vectors,
                                 int32_t* vec_code, int64_t* vec_index) {
  pkv_fib_profile* p = const_cast<pkv_fib_profile*>(cp);
  if (!p || !bytes_host || !n_vectors) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (vec_code) *vec_code = 0;
  if (vec_index) *vec_index = -1;
  *n_vectors = 0;
  uint32_t n32 = 0;
  int st = pkv_fb2_header_parse(p, bytes_host, len, &n32);
  if (st != PKV_OK) return st;
  const int64_t n = n32;
  const int d = p->cfg.dim;
  if (n == 0) return PKV_OK;  // decode_batch_fast of no codes, fib-quant/src/codec.rs:798
  if (!out_host || out_capacity_floats < n * d) return PKV_ERR_BUFFER_TOO_SMALL;
  std::lock_guard<std::mutex> lock(p->ws_mutex);
  st = pkv_ws_prepare(&p->ws, n * p->rec_bytes + 16, n * d * 4);
  if (st != PKV_OK) return st;
  cudaStream_t s = 0;
  pkv_layout L = flat_layout(n, d);
  const int64_t stride = (n * p->rec_bytes + 15) / 16 * 16;
  if (cudaError_t ce = cudaMemcpyAsync(p->ws.in, bytes_host + PKV_FB2_HEADER_BYTES, (size_t)n * p->rec_bytes,
                      cudaMemcpyHostToDevice, s)) return pkv_cuda_status(ce);
  pkv_error_word_reset(p->ws.err, s);
  st = pkv_fib_decode_patch_dev(p, (const uint8_t*)p->ws.in, stride, &L, (float*)p->ws.out, p->ws.err, s);
  if (st != PKV_OK) return st;
  if (cudaError_t ce = cudaMemcpyAsync(out_host, p->ws.out, (size_t)n * d * 4, cudaMemcpyDeviceToHost, s)) return pkv_cuda_status(ce);
  st = pkv_error_word_read(p->ws.err, s, vec_code, vec_index);
  if (st != PKV_OK) return st;
  *n_vectors = n;
  return PKV_OK;
}


// ---------------------------------------------------------------------------
// turbo-quant
// ---------------------------------------------------------------------------

int pkv_turbo_profile_create(const pkv_turbo_config* cfg, const float* signs, const float* qjl,
                             const float* cos_lut, const float* sin_lut, pkv_turbo_profile** out) {
  if (!cfg || !signs || !out) return PKV_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  const int d = cfg->dim;
  if (d <= 0 || (d & 1)) return PKV_ERR_INVALID_ARGUMENT;
  if (cfg->mode != PKV_TURBO_POLAR_ONLY && cfg->mode != PKV_TURBO_POLAR_WITH_QJL)
    return PKV_ERR_INVALID_ARGUMENT;
  const bool with_qjl = cfg->mode == PKV_TURBO_POLAR_WITH_QJL;
  // TurboQuantizer::new_with_mode_and_rotation, turbo-quant/src/turbo.rs:153-162
  if (with_qjl ? (cfg->bits < 2 || cfg->bits > 16) : (cfg->bits < 1 || cfg->bits > 16))
    return PKV_ERR_INVALID_ARGUMENT;
  if (with_qjl && (cfg->projections <= 0 || !qjl)) return PKV_ERR_INVALID_ARGUMENT;
  if (cfg->radii_codec != PKV_RADII_F32 && cfg->radii_codec != PKV_RADII_BLOCK_LOG_U8)
    return PKV_ERR_INVALID_ARGUMENT;
  if (cfg->libm != PKV_LIBM_PORTABLE && cfg->libm != PKV_LIBM_PLATFORM) return PKV_ERR_INVALID_ARGUMENT;
  const int pb = with_qjl ? cfg->bits - 1 : cfg->bits;
  if ((d != 64 && d != 128) || pb > 8) return PKV_ERR_UNSUPPORTED;
  if (with_qjl && (cfg->projections % 32 || cfg->projections > 64)) return PKV_ERR_UNSUPPORTED;
  for (int i = 0; i < d; i++)
    if (signs[i] != 1.0f && signs[i] != -1.0f) return PKV_ERR_INVALID_ARGUMENT;

  pkv_turbo_profile* p = new (std::nothrow) pkv_turbo_profile();
  if (!p) return PKV_ERR_CUDA;
  p->cfg = *cfg;
  p->polar_bits = pb;
  p->pairs = d / 2;
  const int radii_bytes = cfg->radii_codec == PKV_RADII_F32 ? p->pairs * 4 : p->pairs + 8;
  const int angle_bytes = (p->pairs * pb + 7) / 8;
  const int sign_bytes = with_qjl ? (cfg->projections + 7) / 8 : 0;
  p->rec_bytes = radii_bytes + angle_bytes + sign_bytes;  // turbo-quant/src/wire.rs:311-327
  p->radii_words = radii_bytes / 4;
  p->angle_words = angle_bytes / 4;
  p->sign_words = sign_bytes / 4;
  p->scale = 1.0f / sqrtf((float)d);  // (n as f32).sqrt().recip(), rotation.rs:394
  memset(p->sign_mask, 0, sizeof(p->sign_mask));
  for (int i = 0; i < d; i++)
    if (signs[i] < 0.0f) p->sign_mask[i >> 5] |= 1u << (i & 31);
  p->qjl_dev = nullptr;
  p->qjl_rot_dev = nullptr;
  p->lut_dev = nullptr;
  p->logf_table = PkvUlpTable{nullptr, nullptr, nullptr, 0, 0};
  p->expf_table = PkvUlpTable{nullptr, nullptr, nullptr, 0, 0};
  if (cfg->libm == PKV_LIBM_PLATFORM && cfg->radii_codec == PKV_RADII_BLOCK_LOG_U8) {
    int st = pkv_ulp_table_get(PKV_LIBM_FN_LOG, &p->logf_table);
    if (st == PKV_OK) st = pkv_ulp_table_get(PKV_LIBM_FN_EXP, &p->expf_table);
    if (st != PKV_OK) {
      delete p;
      return st;
    }
  }
  const int levels = 1 << pb;
  float lut[1024];
  for (int i = 0; i < levels; i++) {
    if (cos_lut && sin_lut) {
      lut[i] = cos_lut[i];
      lut[levels + i] = sin_lut[i];
    } else {  // PolarCode::dequantize_angle + cosf/sinf of the host libm, polar.rs:91-95,312-313
      const float pi = 3.14159274101257324f;
      volatile float frac = (float)i / (float)levels;
      volatile float scaled = frac * (2.0f * pi);
      const float theta = scaled - pi;
      lut[i] = cosf(theta);
      lut[levels + i] = sinf(theta);
    }
  }
  // Bucket shortcut (pkv_fast_paths.h): rays at 2 pi t / L, t = 0..L/4, usable only if every
  // exact decision boundary lies within 2e-6 rad of its ray.
  p->ray_count = pb >= 2 ? levels / 4 + 1 : 0;
  p->fast_bucket = pb >= 2 && turbo_bucket_boundaries_ok(levels);
  for (int t = 0; t < p->ray_count; t++) {
    const double beta = 2.0 * M_PI * (double)t / (double)levels;
    lut[2 * levels + t] = (float)cos(beta);
    lut[2 * levels + p->ray_count + t] = (float)sin(beta);
  }
  const int lut_len = 2 * levels + 2 * p->ray_count;
  cudaError_t e = cudaGetDevice(&p->device);
  if (e == cudaSuccess) e = cudaMalloc((void**)&p->lut_dev, sizeof(float) * lut_len);
  if (e == cudaSuccess) e = cudaMemcpy(p->lut_dev, lut, sizeof(float) * lut_len, cudaMemcpyHostToDevice);
  if (with_qjl) {
    const int m = cfg->projections;
    float* host = new float[(size_t)m * (d + 1)];
    memcpy(host, qjl, sizeof(float) * (size_t)m * d);
    for (int r = 0; r < m; r++) {  // |g_r| rounded up, times the relative bound of the sign shortcut
      double s2 = 0.0;
      for (int j = 0; j < d; j++) s2 += (double)qjl[r * d + j] * (double)qjl[r * d + j];
      host[(size_t)m * d + r] = (float)(sqrt(s2) * 1.0001) * PKV_QJL_REL_BOUND;
      p->qjl_thr[r] = host[(size_t)m * d + r];
      p->qjl_thr_tf32[r] = (float)(sqrt(s2) * 1.0001) * PKV_QJL_TF32_BOUND;
    }
    const size_t bytes = sizeof(float) * (size_t)m * (d + 1);
    if (e == cudaSuccess) e = cudaMalloc((void**)&p->qjl_dev, bytes);
    if (e == cudaSuccess) e = cudaMemcpy(p->qjl_dev, host, bytes, cudaMemcpyHostToDevice);
    delete[] host;
    {
      // The sketch in the rotated domain: g . (S H~ z) = (g S H~) . z with H~ = scale * H, H the natural-order
      // Walsh-Hadamard matrix the butterflies of turbo-quant/src/rotation.rs:379-398 apply, S the signs.
      // Row r of the table is g_r S H~ / (|g_r| * 1.0001), computed in binary64 and rounded once, so that
      // one bound serves every projection.  A zero row stays zero (its signs come from the exact sequence).
      float* rot = new float[(size_t)m * d];
      for (int r = 0; r < m; r++) {
        double s2 = 0.0;
        for (int j = 0; j < d; j++) s2 += (double)qjl[r * d + j] * (double)qjl[r * d + j];
        const double denom = sqrt(s2) * 1.0001;
        for (int k = 0; k < d; k++) {
          double acc = 0.0;
          for (int j = 0; j < d; j++) {
            const double term = (double)qjl[r * d + j] * (double)signs[j];
            acc += (__builtin_popcount((unsigned)(j & k)) & 1) ? -term : term;
          }
          rot[r * d + k] = denom > 0.0 ? (float)(acc * (double)p->scale / denom) : 0.0f;
        }
      }
      if (e == cudaSuccess) e = cudaMalloc((void**)&p->qjl_rot_dev, sizeof(float) * (size_t)m * d);
      if (e == cudaSuccess) e = cudaMemcpy(p->qjl_rot_dev, rot, sizeof(float) * (size_t)m * d, cudaMemcpyHostToDevice);
      delete[] rot;
    }
  }
  if (e != cudaSuccess) {
    pkv_turbo_profile_destroy(p);
    return PKV_ERR_CUDA;
  }
  *out = p;
  return PKV_OK;
}

int pkv_turbo_profile_destroy(pkv_turbo_profile* p) {
  if (!p) return PKV_OK;
  if (p->qjl_dev) cudaFree(p->qjl_dev);
  if (p->qjl_rot_dev) cudaFree(p->qjl_rot_dev);
  if (p->lut_dev) cudaFree(p->lut_dev);
  ws_release(&p->ws);
  delete p;
  return PKV_OK;
}

int32_t pkv_turbo_record_bytes(const pkv_turbo_profile* p) { return p ? p->rec_bytes : 0; }

int pkv_turbo_encode_dev(const pkv_turbo_profile* p, const float* x_dev, const pkv_layout* layout,
                         uint8_t* payload_dev, int64_t payload_batch_stride, uint64_t* err_dev,
                         void* stream) {
  if (!p || !x_dev || !payload_dev || !err_dev) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (((uintptr_t)x_dev | (uintptr_t)payload_dev) & 15) return PKV_ERR_INVALID_ARGUMENT;
  PkvGeom g;
  int st = make_geom(layout, p->rec_bytes, payload_batch_stride, pkv_turbo_tile_vectors(p->cfg.dim), true, &g);
  if (st != PKV_OK) return st;
  if (g.vpb == 0) return PKV_ERR_EMPTY_BATCH;
  return pkv_launch_turbo_encode(p, x_dev, g, payload_dev, err_dev, (cudaStream_t)stream);
}

int pkv_turbo_decode_patch_dev(const pkv_turbo_profile* p, const uint8_t* payload_dev,
                               int64_t payload_batch_stride, const pkv_layout* layout,
                               float* cache_dev, uint64_t* err_dev, void* stream) {
  if (!p || !cache_dev || !payload_dev || !err_dev) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (((uintptr_t)cache_dev | (uintptr_t)payload_dev) & 15) return PKV_ERR_INVALID_ARGUMENT;
  PkvGeom g;
  int st = make_geom(layout, p->rec_bytes, payload_batch_stride, pkv_turbo_tile_vectors(p->cfg.dim), false, &g);
  if (st != PKV_OK) return st;
  return pkv_launch_turbo_decode(p, payload_dev, g, cache_dev, PKV_DST_F32, err_dev, (cudaStream_t)stream);
}

int pkv_turbo_decode_patch_dev_as(const pkv_turbo_profile* p, const uint8_t* payload_dev,
                                  int64_t payload_batch_stride, const pkv_layout* layout,
                                  void* cache_dev, int32_t dst_dtype, uint64_t* err_dev, void* stream) {
  if (!p || !cache_dev || !payload_dev || !err_dev) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (((uintptr_t)cache_dev | (uintptr_t)payload_dev) & 15) return PKV_ERR_INVALID_ARGUMENT;
  PkvGeom g;
  int st = make_geom(layout, p->rec_bytes, payload_batch_stride, pkv_turbo_tile_vectors(p->cfg.dim), false, &g);
  if (st == PKV_OK) st = check_dst(layout, dst_dtype);
  if (st != PKV_OK) return st;
  return pkv_launch_turbo_decode(p, payload_dev, g, cache_dev, dst_dtype, err_dev, (cudaStream_t)stream);
}

int pkv_turbo_decode_patch_dev_multi(const pkv_turbo_profile* p, const uint8_t* payload_dev,
                                     int64_t payload_batch_stride, const pkv_layout* layout,
                                     void* cache_dev, const int64_t* batch_offsets_dev, int32_t dst_dtype,
                                     uint64_t* err_dev, void* stream) {
  if (!p || !cache_dev || !payload_dev || !err_dev || !batch_offsets_dev) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (((uintptr_t)cache_dev | (uintptr_t)payload_dev) & 15) return PKV_ERR_INVALID_ARGUMENT;
  PkvGeom g;
  int st = make_geom(layout, p->rec_bytes, payload_batch_stride, pkv_turbo_tile_vectors(p->cfg.dim), false, &g);
  if (st == PKV_OK) st = check_dst(layout, dst_dtype);
  if (st != PKV_OK) return st;
  g.batch_offsets = batch_offsets_dev;
  return pkv_launch_turbo_decode(p, payload_dev, g, cache_dev, dst_dtype, err_dev, (cudaStream_t)stream);
}

int pkv_turbo_score_queries_dev(const pkv_turbo_profile* p, const uint8_t* payload_dev,
                                int64_t payload_batch_stride, int64_t n_batches, int64_t vectors_per_batch,
                                const float* rotated_queries_dev, const float* projected_queries_dev,
                                int64_t n_queries, float* scores_dev, uint64_t* err_dev, void* stream) {
  if (!p || !payload_dev || !rotated_queries_dev || !scores_dev || !err_dev) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (p->cfg.mode == PKV_TURBO_POLAR_WITH_QJL && !projected_queries_dev) return PKV_ERR_INVALID_ARGUMENT;
  if (((uintptr_t)payload_dev & 15) || ((uintptr_t)rotated_queries_dev & 3) || ((uintptr_t)scores_dev & 3) ||
      ((uintptr_t)projected_queries_dev & 3))
    return PKV_ERR_INVALID_ARGUMENT;
  if (n_batches < 0 || vectors_per_batch < 0 || n_queries < 0 || n_batches >= ((int64_t)1 << 31) ||
      vectors_per_batch >= ((int64_t)1 << 31))
    return PKV_ERR_INVALID_ARGUMENT;
  if (n_batches == 0 || vectors_per_batch == 0 || n_queries == 0) return PKV_OK;
  pkv_layout L = flat_layout(vectors_per_batch, p->cfg.dim);
  L.n_batches[0] = (int32_t)n_batches;
  PkvGeom g;
  int st = make_geom(&L, p->rec_bytes, payload_batch_stride, pkv_turbo_tile_vectors(p->cfg.dim), false, &g);
  if (st != PKV_OK) return st;
  return pkv_launch_turbo_score(p, payload_dev, g, rotated_queries_dev, projected_queries_dev, n_queries, scores_dev,
                                err_dev, (cudaStream_t)stream);
}

int pkv_turbo_score_dev(const pkv_turbo_profile* p, const uint8_t* payload_dev,
                        int64_t payload_batch_stride, int64_t n_batches, int64_t vectors_per_batch,
                        const float* rotated_query_dev, const float* projected_query_dev,
                        float* scores_dev, uint64_t* err_dev, void* stream) {
  return pkv_turbo_score_queries_dev(p, payload_dev, payload_batch_stride, n_batches, vectors_per_batch,
                                     rotated_query_dev, projected_query_dev, 1, scores_dev, err_dev, stream);
}

int pkv_turbo_prepare_queries_dev(const pkv_turbo_profile* p, const float* queries_dev, int64_t n_queries,
                                  float* rotated_dev, float* projected_dev, uint64_t* err_dev, void* stream) {
  if (!p || !queries_dev || !rotated_dev || !err_dev || n_queries < 0) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (p->cfg.mode == PKV_TURBO_POLAR_WITH_QJL && !projected_dev) return PKV_ERR_INVALID_ARGUMENT;
  if (((uintptr_t)queries_dev | (uintptr_t)rotated_dev | (uintptr_t)projected_dev) & 3) return PKV_ERR_INVALID_ARGUMENT;
  return pkv_launch_turbo_prepare_queries(p, queries_dev, n_queries, rotated_dev, projected_dev, err_dev,
                                          (cudaStream_t)stream);
}

int pkv_stats_read(uint64_t* counts8) {
  if (!counts8) return PKV_ERR_INVALID_ARGUMENT;
  unsigned long long f[4] = {0, 0, 0, 0}, t[4] = {0, 0, 0, 0};
  if (cudaDeviceSynchronize() != cudaSuccess) return PKV_ERR_CUDA;
  if (int st = pkv_fib_stats_copy(f, 0)) return st;
  if (int st = pkv_turbo_stats_copy(t, 0)) return st;
  for (int i = 0; i < 4; i++) {
    counts8[i] = f[i];
    counts8[4 + i] = t[i];
  }
  return PKV_OK;
}

int pkv_stats_reset(void) {
  if (cudaDeviceSynchronize() != cudaSuccess) return PKV_ERR_CUDA;
  if (int st = pkv_fib_stats_copy(nullptr, 1)) return st;
  return pkv_turbo_stats_copy(nullptr, 1);
}

int pkv_tqb1_header_write(const pkv_turbo_profile* p, uint32_t n_vectors, uint8_t* out) {
  if (!p || !out) return PKV_ERR_INVALID_ARGUMENT;
  const uint16_t ver = 1, rot = 1;  // rotation flag 1 = FastHadamard, wire.rs:583-589
  const uint32_t d = (uint32_t)p->cfg.dim, m = (uint32_t)p->cfg.projections;
  const uint32_t rec = (uint32_t)p->rec_bytes;
  memcpy(out, "TQB1", 4);
  memcpy(out + 4, &ver, 2);
  memcpy(out + 6, &rot, 2);
  out[8] = 2;
  out[9] = 0;
  memcpy(out + 10, &d, 4);
  out[14] = (uint8_t)p->polar_bits;
  out[15] = (uint8_t)(p->cfg.radii_codec == PKV_RADII_F32 ? 0 : 1);
  out[16] = 0;
  out[17] = 0;
  memcpy(out + 18, &m, 4);
  memcpy(out + 22, &p->cfg.seed, 8);
  memcpy(out + 30, &n_vectors, 4);
  memcpy(out + 34, &rec, 4);
  return PKV_OK;
}

// The reference decoder takes the radii codec from byte 15 (wire.rs:437-447); a
// profile here is bound to one codec, so a payload written with the other one is
// reported as a header mismatch and the caller picks the matching profile.
int pkv_tqb1_header_parse(const pkv_turbo_profile* p, const uint8_t* b, int64_t len, uint32_t* n_vectors) {
  if (!p || !b || !n_vectors) return PKV_ERR_INVALID_ARGUMENT;
  if (len < PKV_TQB1_HEADER_BYTES) return PKV_ERR_CORRUPT_HEADER;
  uint16_t ver, rot;
  uint32_t d, m, n, rec;
  uint64_t seed;
  if (memcmp(b, "TQB1", 4)) return PKV_ERR_CORRUPT_HEADER;
  memcpy(&ver, b + 4, 2);
  memcpy(&rot, b + 6, 2);
  memcpy(&d, b + 10, 4);
  memcpy(&m, b + 18, 4);
  memcpy(&seed, b + 22, 8);
  memcpy(&n, b + 30, 4);
  memcpy(&rec, b + 34, 4);
  if (ver != 1 || rot != 1 || b[8] != 2) return PKV_ERR_CORRUPT_HEADER;
  if (b[15] != (p->cfg.radii_codec == PKV_RADII_F32 ? 0 : 1)) return PKV_ERR_CORRUPT_HEADER;
  if (d != (uint32_t)p->cfg.dim || m != (uint32_t)p->cfg.projections || seed != p->cfg.seed)
    return PKV_ERR_CORRUPT_HEADER;
  if (b[14] != p->polar_bits || rec != (uint32_t)p->rec_bytes) return PKV_ERR_CORRUPT_HEADER;
  if (len != PKV_TQB1_HEADER_BYTES + (int64_t)n * rec) return PKV_ERR_CORRUPT_HEADER;  // WireCursor::finish
  *n_vectors = n;
  return PKV_OK;
}

int pkv_turbo_encode_batch_compact(const pkv_turbo_profile* cp, const float* vectors_host, int64_t n,
                                   uint8_t* out_host, int64_t out_capacity, int64_t* out_len,
                                   int32_t* vec_code, int64_t* vec_index) {
  pkv_turbo_profile* p = const_cast<pkv_turbo_profile*>(cp);
  if (!p || !out_host || !out_len || n < 0 || (n > 0 && !vectors_host)) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (vec_code) *vec_code = 0;
  if (vec_index) *vec_index = -1;
  *out_len = 0;
  if (n == 0) return PKV_ERR_EMPTY_BATCH;  // turbo-quant/src/wire.rs:302-306
  if (n >= (int64_t)1 << 31) return PKV_ERR_UNSUPPORTED;
  const int d = p->cfg.dim;
  const int64_t total = PKV_TQB1_HEADER_BYTES + n * p->rec_bytes;
  if (out_capacity < total) return PKV_ERR_BUFFER_TOO_SMALL;
  std::lock_guard<std::mutex> lock(p->ws_mutex);
  int st = pkv_ws_prepare(&p->ws, n * d * 4, n * p->rec_bytes + 16);
  if (st != PKV_OK) return st;
  cudaStream_t s = 0;
  pkv_layout L = flat_layout(n, d);
  const int64_t stride = (n * p->rec_bytes + 15) / 16 * 16;
  if (cudaError_t ce = cudaMemcpyAsync(p->ws.in, vectors_host, (size_t)n * d * 4, cudaMemcpyHostToDevice, s)) return pkv_cuda_status(ce);
  pkv_error_word_reset(p->ws.err, s);
  st = pkv_turbo_encode_dev(p, (const float*)p->ws.in, &L, (uint8_t*)p->ws.out, stride, p->ws.err, s);
  if (st != PKV_OK) return st;
  if (cudaError_t ce = cudaMemcpyAsync(out_host + PKV_TQB1_HEADER_BYTES, p->ws.out, (size_t)n * p->rec_bytes,
                      cudaMemcpyDeviceToHost, s)) return pkv_cuda_status(ce);
  st = pkv_error_word_read(p->ws.err, s, vec_code, vec_index);
  if (st != PKV_OK) return st;
  pkv_tqb1_header_write(p, (uint32_t)n, out_host);
  *out_len = total;
  return PKV_OK;
}

int pkv_turbo_decode_batch_compact(const pkv_turbo_profile* cp, const uint8_t* bytes_host,
                                   int64_t len, float* out_host, int64_t out_capacity_floats,
                                   int64_t* n_vectors, int32_t* vec_code, int64_t* vec_index) {
  pkv_turbo_profile* p = const_cast<pkv_turbo_profile*>(cp);
  if (!p || !bytes_host || !n_vectors) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  if (vec_code) *vec_code = 0;
  if (vec_index) *vec_index = -1;
  *n_vectors = 0;
  uint32_t n32 = 0;
  int st = pkv_tqb1_header_parse(p, bytes_host, len, &n32);
  if (st != PKV_OK) return st;
  const int64_t n = n32;
  const int d = p->cfg.dim;
  if (n == 0) return PKV_OK;
  if (!out_host || out_capacity_floats < n * d) return PKV_ERR_BUFFER_TOO_SMALL;
  std::lock_guard<std::mutex> lock(p->ws_mutex);
  st = pkv_ws_prepare(&p->ws, n * p->rec_bytes + 16, n * d * 4);
  if (st != PKV_OK) return st;
  cudaStream_t s = 0;
  pkv_layout L = flat_layout(n, d);
  const int64_t stride = (n * p->rec_bytes + 15) / 16 * 16;
  if (cudaError_t ce = cudaMemcpyAsync(p->ws.in, bytes_host + PKV_TQB1_HEADER_BYTES, (size_t)n * p->rec_bytes,
                      cudaMemcpyHostToDevice, s)) return pkv_cuda_status(ce);
  pkv_error_word_reset(p->ws.err, s);
  st = pkv_turbo_decode_patch_dev(p, (const uint8_t*)p->ws.in, stride, &L, (float*)p->ws.out, p->ws.err, s);
  if (st != PKV_OK) return st;
  if (cudaError_t ce = cudaMemcpyAsync(out_host, p->ws.out, (size_t)n * d * 4, cudaMemcpyDeviceToHost, s)) return pkv_cuda_status(ce);
  st = pkv_error_word_read(p->ws.err, s, vec_code, vec_index);
  if (st != PKV_OK) return st;
  *n_vectors = n;
  return PKV_OK;
}

}  // extern "C"
