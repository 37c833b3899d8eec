// Many batches per call with host buffers: the whole pool / shell of one build in
// one call (proveKV/src/pool.rs:246-309, shell.rs:250-311 issue one codec call per
// (layer, K|V); here the caller hands over all of them).  Batches are cut into
// chunks that run on three streams, so the host->device copy of one chunk, the
// kernel of the previous one and the device->host copy of the one before overlap.
#include <math.h>
#include <string.h>

#include <mutex>

#include "pkv_common.cuh"

namespace {

struct BulkCodec {
  PkvWorkspace* ws;
  std::mutex* mu;  // the profile's staging lock
  int device;      // the device the profile's tables live on
  int dim, rec, hdr;
  const void* profile;
  bool turbo;
};

// On an error exit copies of earlier chunks may still be reading or writing the caller's host
// buffers and the staging area: wait for them before the caller gets control back.  The status
// of the wait itself is dropped; the caller sees the original error.
struct StreamDrain {
  PkvWorkspace* ws;
  bool armed = true;
  ~StreamDrain() {
    if (!armed) return;
    for (int i = 0; i < PKV_WS_STREAMS; i++)
      if (ws->streams[i]) cudaStreamSynchronize(ws->streams[i]);
  }
};

int dev_encode(const BulkCodec& c, const float* x, const pkv_layout* L, uint8_t* pay, int64_t stride,
               uint64_t* err, cudaStream_t s) {
  return c.turbo ? pkv_turbo_encode_dev((const pkv_turbo_profile*)c.profile, x, L, pay, stride, err, s)
                 : pkv_fib_encode_dev((const pkv_fib_profile*)c.profile, x, L, pay, stride, err, s);
}
int dev_decode(const BulkCodec& c, const uint8_t* pay, int64_t stride, const pkv_layout* L, float* out,
               uint64_t* err, cudaStream_t s) {
  return c.turbo ? pkv_turbo_decode_patch_dev((const pkv_turbo_profile*)c.profile, pay, stride, L, out, err, s)
                 : pkv_fib_decode_patch_dev((const pkv_fib_profile*)c.profile, pay, stride, L, out, err, s);
}
void write_header(const BulkCodec& c, uint32_t n, uint8_t* out) {
  if (c.turbo) pkv_tqb1_header_write((const pkv_turbo_profile*)c.profile, n, out);
  else pkv_fb2_header_write((const pkv_fib_profile*)c.profile, n, out);
}
int parse_header(const BulkCodec& c, const uint8_t* b, int64_t len, uint32_t* n) {
  return c.turbo ? pkv_tqb1_header_parse((const pkv_turbo_profile*)c.profile, b, len, n)
                 : pkv_fb2_header_parse((const pkv_fib_profile*)c.profile, b, len, n);
}

// The staging streams get the highest priority the device offers: their kernels are short chunks
// that feed a transfer pipeline, and when the caller has a long kernel of its own in flight on another
// stream (a decode-and-patch of the pool, say) the chunks must not queue behind its blocks.
int prepare_streams(PkvWorkspace* ws) {
  int least = 0, greatest = 0;
  if (cudaDeviceGetStreamPriorityRange(&least, &greatest) != cudaSuccess) return PKV_ERR_CUDA;
  for (int i = 0; i < PKV_WS_STREAMS; i++)
    if (!ws->streams[i] &&
        cudaStreamCreateWithPriority(&ws->streams[i], cudaStreamNonBlocking, greatest) != cudaSuccess)
      return PKV_ERR_CUDA;
  return PKV_OK;
}

// Number of chunks: the shorter of the two transfers of a call is the part that cannot hide behind
// the longer one, 1/n of it stays exposed at the start or the end of the pipeline, and every chunk
// costs about 25 us of copy set-up and launches; n = sqrt(t_short / 25 us) balances the two
// (measured on C2: 6-8 chunks 1.87 ms, 16 chunks 1.96 ms, 32 chunks 2.36 ms per encode call).
int chunk_count(int64_t n_batches, int64_t in_bytes, int64_t out_bytes) {
  const double short_us = (double)(in_bytes < out_bytes ? in_bytes : out_bytes) / 55.0e3;  // 55 GB/s
  int n = (int)(sqrt(short_us / 25.0) + 0.5);
  if (n < 2) n = 2;
  if (n > PKV_WS_ERR_WORDS) n = PKV_WS_ERR_WORDS;
  return (int)(n_batches < n ? n_batches : n);
}

pkv_layout chunk_layout(int64_t b0, int64_t nb, int64_t vpb, int dim) {
  pkv_layout L;
  memset(&L, 0, sizeof(L));
  L.base = b0 * vpb * dim;
  L.n_batches[0] = (int32_t)nb;
  L.n_batches[1] = L.n_batches[2] = 1;
  L.batch_stride[0] = vpb * dim;
  L.n_tokens = (int32_t)vpb;
  L.n_heads = 1;
  L.token_stride = dim;
  L.head_stride = dim;
  L.n_replicas = 1;
  return L;
}

// Collect the chunk error words: the first failing vector in batch-major order.
int finish(const BulkCodec& c, int n_chunks, const int64_t* chunk_b0, int64_t vpb, int32_t* vec_code,
           int64_t* vec_index) {
  uint64_t words[PKV_WS_ERR_WORDS];
  for (int i = 0; i < PKV_WS_STREAMS; i++)
    if (cudaError_t ce = cudaStreamSynchronize(c.ws->streams[i])) return pkv_cuda_status(ce);
  if (cudaError_t ce = cudaMemcpy(words, c.ws->err, sizeof(uint64_t) * n_chunks, cudaMemcpyDeviceToHost)) return pkv_cuda_status(ce);
  uint64_t best = PKV_ERR_NONE;
  for (int k = 0; k < n_chunks; k++) {
    if (words[k] == PKV_ERR_NONE) continue;
    const uint64_t pass = words[k] >> 56, code = words[k] & 0xff;
    const uint64_t idx = ((words[k] >> 8) & 0xFFFFFFFFFFFFull) + (uint64_t)(chunk_b0[k] * vpb);
    const uint64_t w = (pass << 56) | (idx << 8) | code;
    if (w < best) best = w;
  }
  if (best == PKV_ERR_NONE) return PKV_OK;
  if (vec_code) *vec_code = (int32_t)(best & 0xff);
  if (vec_index) *vec_index = (int64_t)((best >> 8) & 0xFFFFFFFFFFFFull);
  return (int)(best & 0xff);
}

int bulk_encode(const BulkCodec& c, const float* x_host, int64_t n_batches, int64_t vpb,
                uint8_t* out_host, int64_t out_capacity, int32_t* vec_code, int64_t* vec_index) {
  if (!x_host || !out_host || n_batches < 0 || vpb < 0) return PKV_ERR_INVALID_ARGUMENT;
  if (vec_code) *vec_code = 0;
  if (vec_index) *vec_index = -1;
  if (n_batches == 0) return PKV_OK;
  if (vpb == 0) return PKV_ERR_EMPTY_BATCH;
  if (n_batches * vpb >= (int64_t)1 << 31) return PKV_ERR_UNSUPPORTED;
  const int64_t blob = c.hdr + vpb * c.rec;
  if (out_capacity < n_batches * blob) return PKV_ERR_BUFFER_TOO_SMALL;
  const int64_t pstride = (vpb * c.rec + 15) / 16 * 16;
  if (int ds = pkv_check_device(c.device)) return ds;
  std::lock_guard<std::mutex> lock(*c.mu);
  int st = pkv_ws_prepare(c.ws, n_batches * vpb * c.dim * 4, n_batches * pstride);
  if (st != PKV_OK) return st;
  if ((st = prepare_streams(c.ws)) != PKV_OK) return st;
  StreamDrain drain{c.ws};
  const int n_chunks = chunk_count(n_batches, n_batches * vpb * c.dim * 4, n_batches * vpb * c.rec);
  int64_t chunk_b0[PKV_WS_ERR_WORDS];
  for (int k = 0; k < n_chunks; k++) {
    const int64_t b0 = n_batches * k / n_chunks, b1 = n_batches * (k + 1) / n_chunks, nb = b1 - b0;
    chunk_b0[k] = b0;
    cudaStream_t s = c.ws->streams[k % PKV_WS_STREAMS];
    if (pkv_error_word_reset(c.ws->err + k, s) != PKV_OK) return PKV_ERR_CUDA;
    const int64_t xoff = b0 * vpb * c.dim;
    if (cudaError_t ce = cudaMemcpyAsync((float*)c.ws->in + xoff, x_host + xoff, (size_t)(nb * vpb * c.dim) * 4,
                        cudaMemcpyHostToDevice, s)) return pkv_cuda_status(ce);
    pkv_layout L = chunk_layout(b0, nb, vpb, c.dim);
    st = dev_encode(c, (const float*)c.ws->in, &L, (uint8_t*)c.ws->out + b0 * pstride, pstride,
                    c.ws->err + k, s);
    if (st != PKV_OK) return st;
    if (cudaError_t ce = cudaMemcpy2DAsync(out_host + b0 * blob + c.hdr, (size_t)blob, (uint8_t*)c.ws->out + b0 * pstride,
                          (size_t)pstride, (size_t)(vpb * c.rec), (size_t)nb, cudaMemcpyDeviceToHost,
                          s)) return pkv_cuda_status(ce);
  }
  for (int64_t b = 0; b < n_batches; b++) write_header(c, (uint32_t)vpb, out_host + b * blob);
  drain.armed = false;  // finish() waits for the streams itself
  return finish(c, n_chunks, chunk_b0, vpb, vec_code, vec_index);
}

int bulk_decode(const BulkCodec& c, const uint8_t* bytes_host, int64_t n_batches, int64_t vpb,
                float* out_host, int64_t out_capacity_floats, int32_t* vec_code, int64_t* vec_index) {
  if (!bytes_host || !out_host || n_batches < 0 || vpb < 0) return PKV_ERR_INVALID_ARGUMENT;
  if (vec_code) *vec_code = 0;
  if (vec_index) *vec_index = -1;
  if (n_batches == 0 || vpb == 0) return PKV_OK;
  if (n_batches * vpb >= (int64_t)1 << 31) return PKV_ERR_UNSUPPORTED;
  const int64_t blob = c.hdr + vpb * c.rec;
  if (out_capacity_floats < n_batches * vpb * c.dim) return PKV_ERR_BUFFER_TOO_SMALL;
  for (int64_t b = 0; b < n_batches; b++) {
    uint32_t n = 0;
    int st = parse_header(c, bytes_host + b * blob, blob, &n);
    if (st != PKV_OK) return st;
    if (n != (uint32_t)vpb) return PKV_ERR_CORRUPT_HEADER;
  }
  const int64_t pstride = (vpb * c.rec + 15) / 16 * 16;
  if (int ds = pkv_check_device(c.device)) return ds;
  std::lock_guard<std::mutex> lock(*c.mu);
  int st = pkv_ws_prepare(c.ws, n_batches * pstride, n_batches * vpb * c.dim * 4);
  if (st != PKV_OK) return st;
  if ((st = prepare_streams(c.ws)) != PKV_OK) return st;
  StreamDrain drain{c.ws};
  const int n_chunks = chunk_count(n_batches, n_batches * vpb * c.rec, n_batches * vpb * c.dim * 4);
  int64_t chunk_b0[PKV_WS_ERR_WORDS];
  for (int k = 0; k < n_chunks; k++) {
    const int64_t b0 = n_batches * k / n_chunks, b1 = n_batches * (k + 1) / n_chunks, nb = b1 - b0;
    chunk_b0[k] = b0;
    cudaStream_t s = c.ws->streams[k % PKV_WS_STREAMS];
    if (pkv_error_word_reset(c.ws->err + k, s) != PKV_OK) return PKV_ERR_CUDA;
    if (cudaError_t ce = cudaMemcpy2DAsync((uint8_t*)c.ws->in + b0 * pstride, (size_t)pstride,
                          bytes_host + b0 * blob + c.hdr, (size_t)blob, (size_t)(vpb * c.rec), (size_t)nb,
                          cudaMemcpyHostToDevice, s)) return pkv_cuda_status(ce);
    pkv_layout L = chunk_layout(b0, nb, vpb, c.dim);
    st = dev_decode(c, (const uint8_t*)c.ws->in + b0 * pstride, pstride, &L, (float*)c.ws->out,
                    c.ws->err + k, s);
    if (st != PKV_OK) return st;
    const int64_t xoff = b0 * vpb * c.dim;
    if (cudaError_t ce = cudaMemcpyAsync(out_host + xoff, (float*)c.ws->out + xoff, (size_t)(nb * vpb * c.dim) * 4,
                        cudaMemcpyDeviceToHost, s)) return pkv_cuda_status(ce);
  }
  drain.armed = false;
  return finish(c, n_chunks, chunk_b0, vpb, vec_code, vec_index);
}

BulkCodec fib_codec(const pkv_fib_profile* p) {
  pkv_fib_profile* q = const_cast<pkv_fib_profile*>(p);
  return BulkCodec{&q->ws, &q->ws_mutex, q->device, q->cfg.dim, q->rec_bytes, PKV_FB2_HEADER_BYTES, q, false};
}
BulkCodec turbo_codec(const pkv_turbo_profile* p) {
  pkv_turbo_profile* q = const_cast<pkv_turbo_profile*>(p);
  return BulkCodec{&q->ws, &q->ws_mutex, q->device, q->cfg.dim, q->rec_bytes, PKV_TQB1_HEADER_BYTES, q, true};
}

}  // namespace

extern "C" {

int pkv_fib_encode_batches_compact(const pkv_fib_profile* p, const float* vectors_host,
                                   int64_t n_batches, int64_t vectors_per_batch, uint8_t* out_host,
                                   int64_t out_capacity, int32_t* vec_code, int64_t* vec_index) {
  if (!p) return PKV_ERR_INVALID_ARGUMENT;
  return bulk_encode(fib_codec(p), vectors_host, n_batches, vectors_per_batch, out_host, out_capacity,
                     vec_code, vec_index);
}
int pkv_fib_decode_batches_compact(const pkv_fib_profile* p, const uint8_t* bytes_host,
                                   int64_t n_batches, int64_t vectors_per_batch, float* out_host,
                                   int64_t out_capacity_floats, int32_t* vec_code, int64_t* vec_index) {
  if (!p) return PKV_ERR_INVALID_ARGUMENT;
  return bulk_decode(fib_codec(p), bytes_host, n_batches, vectors_per_batch, out_host,
                     out_capacity_floats, vec_code, vec_index);
}
int pkv_turbo_encode_batches_compact(const pkv_turbo_profile* p, const float* vectors_host,
                                     int64_t n_batches, int64_t vectors_per_batch, uint8_t* out_host,
                                     int64_t out_capacity, int32_t* vec_code, int64_t* vec_index) {
  if (!p) return PKV_ERR_INVALID_ARGUMENT;
  return bulk_encode(turbo_codec(p), vectors_host, n_batches, vectors_per_batch, out_host, out_capacity,
                     vec_code, vec_index);
}
int pkv_turbo_decode_batches_compact(const pkv_turbo_profile* p, const uint8_t* bytes_host,
                                     int64_t n_batches, int64_t vectors_per_batch, float* out_host,
                                     int64_t out_capacity_floats, int32_t* vec_code, int64_t* vec_index) {
  if (!p) return PKV_ERR_INVALID_ARGUMENT;
  return bulk_decode(turbo_codec(p), bytes_host, n_batches, vectors_per_batch, out_host,
                     out_capacity_floats, vec_code, vec_index);
}

}  // extern "C"
