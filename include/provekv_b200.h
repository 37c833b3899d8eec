/*
 * provekv_b200.h -- C ABI of the B200 (sm_100a) KV-cache codec library.
 *
 * The library replaces one path of RecursiveIntell/proveKV: the batched
 * fib-quant k4 cold-tier codec (FB2 wire), the batched turbo-quant hot-shell
 * codec (TQB1 wire) and the decode step fused with the write into a
 * framework's per-layer KV cache.  Every entry point is `extern "C"`, takes
 * plain pointers and sizes, and returns a status code (0 = ok).  Nothing here
 * falls back to the CPU: when no CUDA device is usable the calls fail with
 * PKV_ERR_CUDA.
 *
 * Two levels are exported.
 *  - "*_batch_compact": host buffers in, host buffers out, FB2 / TQB1 bytes
 *    including the header.  These are what a binding of the reference's
 *    FibQuantAdapter::{encode,decode}_batch_compact (proveKV/src/codec.rs:513-569)
 *    and TurboQuantAdapter::{encode,decode}_batch_compact
 *    (proveKV/src/codec.rs:248-326) calls.
 *  - "*_dev": device pointers in and out, any number of (layer, K|V, agent)
 *    batches per launch addressed through a pkv_layout, payload without
 *    header.  This is the form the pool / shell code drives
 *    (proveKV/src/pool.rs:246-309, proveKV/src/shell.rs:250-311) and the form
 *    the fused decode-and-patch takes (quant-codec-core/src/codec.rs:27-34
 *    `decode_slice` into a caller-owned output).
 *
 * Tables (rotation matrix, codebook, Rademacher signs, QJL matrix) are inputs:
 * the reference derives them from a seed with rand_chacha / nalgebra / statrs,
 * none of which is reproduced here; bit-exactness is defined given equal tables.
 */
#ifndef PROVEKV_B200_H
#define PROVEKV_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------ */
enum {
  PKV_OK = 0,
  PKV_ERR_INVALID_ARGUMENT = 1,
  PKV_ERR_CUDA = 2,
  PKV_ERR_UNSUPPORTED = 3,      /* shape outside what the kernels are built for */
  PKV_ERR_EMPTY_BATCH = 4,      /* fib-quant/src/codec.rs:226, turbo-quant/src/wire.rs:303 */
  PKV_ERR_CORRUPT_HEADER = 5,   /* magic / version / profile mismatch / length */
  PKV_ERR_BUFFER_TOO_SMALL = 6,
  PKV_ERR_STATIC_SCRATCH_TOO_SMALL = 7, /* more vectors than pkv_fib_encode_dev_static can take */
  /* Per-vector codes, reported together with the index of the first failing
   * vector.  Within one vector the smaller code is the check the reference
   * performs first. */
  PKV_VEC_NONFINITE_INPUT = 16,   /* fib-quant/src/codec.rs:1059, turbo-quant/src/polar.rs:401 */
  PKV_VEC_ZERO_NORM = 17,         /* fib-quant/src/codec.rs:603 */
  PKV_VEC_BAD_RADIUS = 18,        /* turbo-quant/src/polar.rs:127, radius.rs:104,161 */
  PKV_VEC_BAD_RADIUS_RANGE = 19,  /* turbo-quant/src/radius.rs:170 */
  PKV_VEC_PADDING_BITS = 20,      /* fib-quant/src/bitpack.rs:66, turbo-quant/src/bitpack.rs:101 */
  PKV_VEC_INDEX_RANGE = 21,       /* fib-quant/src/codec.rs:819 */
  PKV_VEC_BAD_NORM = 22,          /* fib-quant/src/codec.rs:1029 */
  PKV_VEC_NONFINITE_OUTPUT = 23,  /* fib-quant/src/codec.rs:840 */
  PKV_VEC_NONFINITE_RESIDUAL = 24,/* turbo-quant/src/qjl.rs:210 */
  PKV_VEC_NORM_RANGE = 25,        /* fib-quant/src/codec.rs:1003 (second pass of encode_batch) */
  PKV_VEC_DEVICE_WAIT = 26,       /* no counterpart: a bounded wait inside a kernel ran out (the payload is not valid) */
  PKV_VEC_MISALIGNED_DST = 27     /* no counterpart: a per-tensor cache offset of a *_multi call is negative or not
                                     a multiple of 16 bytes (that batch is skipped) */
};

const char* pkv_status_string(int status);
/* Counters of the certify-or-flag tiers on the current device since the last reset (a shortcut's answer is
 * used only where it is proven to be the reference's; these count what was not proven and went on):
 *   counts8[0] fib blocks settled by an encoder's in-kernel exact tier
 *   counts8[1] fib list entries (a block or a whole vector) redone by the exact f64 kernel
 *   counts8[4] turbo pairs whose angle bucket was taken with the exact atan2f
 *   counts8[5] turbo (vector, projection) signs retaken by the binary32 dot
 *   counts8[6] turbo signs or list entries redone with the reference's own sequence
 * the others are zero.  Both calls synchronise the device. */
int pkv_stats_read(uint64_t* counts8);
int pkv_stats_reset(void);

int pkv_version(void);
/* Text of the CUDA runtime error behind the calling thread's most recent PKV_ERR_CUDA ("" if none). */
const char* pkv_last_cuda_error(void);

/* ---- configuration ----------------------------------------------------- */
#define PKV_NORM_FP16 0 /* NormFormat::Fp16Paper, fib-quant/src/codec.rs:1001 */
#define PKV_NORM_F32 1  /* NormFormat::F32Reference */

#define PKV_ARGMIN_PAIRWISE 0   /* AVX2 order, gpu-backend/src/simd_nearest.rs:44-94 */
#define PKV_ARGMIN_SEQUENTIAL 1 /* scalar order, gpu-backend/src/simd_nearest.rs:24-39 */

#define PKV_FIB_NUMERICS_AUTO 0   /* batch numerics for n >= 4, single below: fib-quant/src/codec.rs:586-589 */
#define PKV_FIB_NUMERICS_BATCH 1  /* normalised vector rounded to f32 before rotation, :607-609 */
#define PKV_FIB_NUMERICS_SINGLE 2 /* normalised vector kept in f64, :481 */

#define PKV_TURBO_POLAR_ONLY 0     /* TurboMode::PolarOnly,  polar_bits = bits */
#define PKV_TURBO_POLAR_WITH_QJL 1 /* TurboMode::PolarWithQjl, polar_bits = bits - 1 */

#define PKV_RADII_F32 0        /* RadiusCodecProfileV1::F32 */
#define PKV_RADII_BLOCK_LOG_U8 1 /* RadiusCodecProfileV1::BlockLogU8 */

/* The reference takes ln / exp of the BlockLogU8 radii from the platform libm through Rust std
 * (turbo-quant/src/radius.rs:61,143); glibc's binary32 functions are not correctly rounded, so those
 * bytes are defined by the machine that wrote them.  PKV_LIBM_PORTABLE: the correctly rounded functions
 * of include/pkv_portable_math.h (the same bits on every machine).  PKV_LIBM_PLATFORM: the bits of this
 * host's logf / expf; the first profile created with it scans every binary32 argument on the host cores
 * (a few seconds, once per process and function) and uploads the arguments where the two differ.
 * PKV_ERR_UNSUPPORTED if the host function is ever more than one unit away from correct rounding. */
#define PKV_LIBM_PORTABLE 0
#define PKV_LIBM_PLATFORM 1

typedef struct pkv_fib_config {
  int32_t dim;           /* ambient_dim; kernels: 64 or 128 */
  int32_t block_dim;     /* k; kernels: 4 */
  int32_t codebook_size; /* N <= 32 */
  int32_t norm_format;   /* PKV_NORM_* */
  int32_t argmin_order;  /* PKV_ARGMIN_* */
  int32_t numerics;      /* PKV_FIB_NUMERICS_* */
} pkv_fib_config;

typedef struct pkv_turbo_config {
  int32_t dim;         /* power of two; kernels: 64 or 128 */
  int32_t bits;        /* TurboQuantizer bits (turbo-quant/src/turbo.rs:124) */
  int32_t mode;        /* PKV_TURBO_* */
  int32_t projections; /* QJL rows m (multiple of 8, <= 64 in the kernels) */
  int32_t radii_codec; /* PKV_RADII_* */
  int32_t libm;        /* PKV_LIBM_*: which logf / expf the BlockLogU8 radii use */
  uint64_t seed;       /* written to the TQB1 header only */
} pkv_turbo_config;

/* How the vectors of one launch are laid out in an f32 tensor.
 * A launch covers n_batches[0]*n_batches[1]*n_batches[2] batches (for example
 * agent x layer x {K,V}); batch (b0,b1,b2) holds n_tokens*n_heads vectors and
 * vector v of a batch is (token = v / n_heads, head = v % n_heads), the order
 * proveKV/src/pool.rs:246-257 gathers in.  Element offset of a vector:
 *   base + b0*batch_stride[0] + b1*batch_stride[1] + b2*batch_stride[2]
 *        + token*token_stride + head*head_stride  (+ r*replica_stride on decode)
 * The dim values of a vector are contiguous.  All strides and base are in
 * elements and must be multiples of 4 (16-byte accesses).  n_replicas > 1 makes
 * the decode kernels write every vector to that many destinations (one decode,
 * several caches); encode requires n_replicas == 1. */
typedef struct pkv_layout {
  int64_t base;
  int64_t batch_stride[3];
  int64_t token_stride;
  int64_t head_stride;
  int64_t replica_stride;
  int32_t n_batches[3];
  int32_t n_tokens;
  int32_t n_heads;
  int32_t n_replicas;
} pkv_layout;

/* Element type of the cache a decode-and-patch call writes.  proveKV/scripts/ppl_validate_multi_agent.py:
 * 247-262 stores the decoded f32 values with `dtype=k.dtype`, i.e. rounded to nearest-even to the model's
 * cache type; the *_as calls do the same rounding in the kernel's store (values beyond the half-precision
 * range become infinities, as in that conversion).  For the 16-bit types the layout's base and strides are
 * still in elements and must be multiples of 8. */
#define PKV_DST_F32 0
#define PKV_DST_F16 1
#define PKV_DST_BF16 2

typedef struct pkv_fib_profile pkv_fib_profile;
typedef struct pkv_turbo_profile pkv_turbo_profile;

/* ---- device / memory helpers ------------------------------------------ */
int pkv_device_count(int* count);
int pkv_set_device(int device);
/* Pinned host memory for callers that want full PCIe rate on the compact calls. */
int pkv_host_alloc(void** ptr, int64_t bytes);
int pkv_host_free(void* ptr);
int pkv_dev_alloc(void** ptr, int64_t bytes);
int pkv_dev_free(void* ptr);
int pkv_memcpy_h2d(void* dst_dev, const void* src_host, int64_t bytes, void* stream);
int pkv_memcpy_d2h(void* dst_host, const void* src_dev, int64_t bytes, void* stream);
int pkv_stream_synchronize(void* stream);

/* Wire blobs on the host <-> a device payload buffer, headers skipped: blob b lies at
 * blobs_host + b * blob_bytes with its records after header_bytes (PKV_FB2_HEADER_BYTES /
 * PKV_TQB1_HEADER_BYTES; fib-quant/src/codec.rs:195-220, turbo-quant/src/wire.rs:276-290), batch b of
 * the payload at payload_dev + b * payload_batch_stride.  One strided asynchronous copy on `stream`;
 * pinned host memory keeps it asynchronous.  The download leaves the header bytes of each blob
 * untouched (write them with pkv_fb2_header_write / pkv_tqb1_header_write). */
int pkv_payload_upload(const uint8_t* blobs_host, int64_t blob_bytes, int32_t header_bytes, int64_t n_batches,
                       int64_t record_bytes_per_batch, uint8_t* payload_dev, int64_t payload_batch_stride,
                       void* stream);
int pkv_payload_download(const uint8_t* payload_dev, int64_t payload_batch_stride, int64_t n_batches,
                         int64_t record_bytes_per_batch, uint8_t* blobs_host, int64_t blob_bytes,
                         int32_t header_bytes, void* stream);

/* The device error word: 0xFFFF...F = no error; otherwise the smallest
 * (pass << 56 | vector_index << 8 | code) any thread reported, vector_index counted over the
 * whole launch.  Within one batch this is the error the reference's loops reach first (fib
 * encode checks every vector for finiteness / zero norm in a first pass and the norm range in a
 * second, fib-quant/src/codec.rs:593-608,695-708).  Across the batches of one launch the order
 * is by pass, then by vector: a first-pass error of a later batch is reported in preference to a
 * second-pass error of an earlier one (the reference issues one call per batch from a parallel
 * loop and reports whichever batch fails).  Reset before a launch, read (synchronising the
 * stream) after it. */
int pkv_error_word_reset(uint64_t* err_dev, void* stream);
int pkv_error_word_read(const uint64_t* err_dev, void* stream, int32_t* code, int64_t* vector_index);

/* ---- the gpu-backend crate's operators on the fib encode path ------------ */
/* gpu_backend::hadamard_batch (gpu-backend/src/lib.rs:66-90): data_dev holds n vectors of dim f32, transformed
 * in place with the arithmetic of hadamard_batch_cpu (gpu-backend/src/fallback.rs:12-62): zero-padded to the
 * next power of two, butterflies (a, b) -> (a + b, a - b) for step = 1, 2, 4, .., x sign_i (64-bit LCG from
 * `seed`, :76-88), x 1/sqrt(padded dim), truncated back to dim; bit for bit.  Padded dims up to 1024
 * (PKV_ERR_UNSUPPORTED beyond).  Bound by HBM: every element is read once and written once. */
int pkv_hadamard_batch_dev(float* data_dev, int64_t n, int32_t dim, uint64_t seed, void* stream);
/* gpu_backend::codebook_lookup_batch (gpu-backend/src/lib.rs:196-239) with the arithmetic of
 * codebook_lookup_cpu (fallback.rs:254-305): input_dev n x dim f32, codebook_dev n_codewords x k f32,
 * indices_dev n * (dim / k) u32 in (vector, block) order; per block the squared distances summed in
 * coordinate order, strict less-than scan from index 0 (ties and non-finite distances as the scan leaves
 * them).  k = 4 and n_codewords <= 32 (PKV_ERR_UNSUPPORTED otherwise; the crate's own GPU path has the
 * same limits); all three pointers 16-byte aligned. */
int pkv_codebook_lookup_batch_dev(const float* input_dev, const float* codebook_dev, int64_t n, int32_t dim,
                                  int32_t k, int32_t n_codewords, uint32_t* indices_dev, void* stream);

/* ---- fib-quant --------------------------------------------------------- */
/* rotation: dim x dim f64 row-major (StoredRotation.matrix, fib-quant/src/rotation.rs:51-56);
 * codebook: codebook_size x block_dim f32 row-major (fib-quant/src/codebook.rs:28-29).
 * A profile (fib or turbo) belongs to the CUDA device that is current when it is created: its
 * tables are uploaded there, and every call that takes the profile returns
 * PKV_ERR_INVALID_ARGUMENT, before launching or copying anything, when another device is
 * current.  The shortcut encoders' error bounds assume an orthonormal rotation; the matrix is
 * checked here (rows of unit length, M M^T = I to 1e-6) and a profile whose matrix fails the check
 * encodes with the exact f64 kernel only. */
int pkv_fib_profile_create(const pkv_fib_config* cfg, const double* rotation, const float* codebook,
                           pkv_fib_profile** out);
/* A profile whose batch encoder rotates with the f32 Walsh-Hadamard transform that the reference's
 * `gpu` build applies in FibQuantizer::encode_batch (fib-quant/src/codec.rs:612-656 ->
 * gpu_backend::hadamard_batch; arithmetic of gpu-backend/src/fallback.rs:12-62: butterflies for step =
 * 1, 2, 4, .., then x sign_i from the 64-bit LCG seeded with rotation_seed (:76-88), then x 1/sqrt(dim))
 * instead of the stored matrix.  The transform costs dim*log2(dim) additions per vector instead of
 * 2*dim*dim multiply-adds, and every step is a binary32 operation, so the bytes are the reference's
 * without a second tier.  NOT wire-compatible with pools encoded through the stored matrix: the
 * reference's decoders (and pkv_fib_decode_*) invert `rotation` whatever the encoder applied.
 * As in the reference the transform is taken for batches of at least 16 vectors
 * (GpuContext::GPU_MIN_BATCH_SIZE, gpu-backend/src/lib.rs:61-63) and the stored matrix below that;
 * cfg->numerics = PKV_FIB_NUMERICS_BATCH takes it for every batch size, PKV_FIB_NUMERICS_SINGLE is
 * PKV_ERR_INVALID_ARGUMENT (encode() has no such path).
 * rotation: the stored matrix the decoders use (and small batches encode with); NULL = the transform
 * itself written out as a matrix, so that decode inverts what encode applied. */
int pkv_fib_profile_create_hadamard(const pkv_fib_config* cfg, uint64_t rotation_seed, const double* rotation,
                                    const float* codebook, pkv_fib_profile** out);
int pkv_fib_profile_destroy(pkv_fib_profile* p);
/* Bytes per vector in the FB2 payload: norm (2 or 4) + ceil(5*dim/4/8). */
int32_t pkv_fib_record_bytes(const pkv_fib_profile* p);

/* Replaces FibQuantizer::encode_batch + finish_batch_encode
 * (fib-quant/src/codec.rs:578-729): one record per vector at
 * payload_dev + batch*payload_batch_stride + v*record_bytes. */
int pkv_fib_encode_dev(const pkv_fib_profile* p, const float* x_dev, const pkv_layout* layout,
                       uint8_t* payload_dev, int64_t payload_batch_stride, uint64_t* err_dev,
                       void* stream);
/* No counterpart in the reference.  Same work and same bytes as pkv_fib_encode_dev for callers
 * that must not allocate device memory while encoding (memory fully budgeted at start-up, or an
 * allocator that may not be re-entered): pkv_fib_encode_dev borrows a list of undecided blocks
 * from the stream's memory pool, this call keeps it in a fixed array inside the library image
 * and calls no allocating routine.  Limits: at most PKV_FIB_STATIC_MAX_VECTORS vectors per call
 * (PKV_ERR_STATIC_SCRATCH_TOO_SMALL beyond), batches of at least 4 vectors (PKV_ERR_UNSUPPORTED
 * below, unless the profile forces batch numerics; also for a profile whose matrix is not
 * orthonormal, which only the exact kernel encodes).  The array (4 MiB on every GPU that loads the
 * library) is shared by all calls on a device: calls that can overlap on the GPU race.  The first
 * call on each device looks the array's address up; make that call before any stream capture. */
#define PKV_FIB_STATIC_MAX_VECTORS (1 << 20)
int pkv_fib_encode_dev_static(const pkv_fib_profile* p, const float* x_dev, const pkv_layout* layout,
                              uint8_t* payload_dev, int64_t payload_batch_stride, uint64_t* err_dev,
                              void* stream);

/* Replaces FibQuantizer::decode_batch_fast (fib-quant/src/codec.rs:797-844) fused
 * with the per-head relayout of proveKV/src/pool.rs:538-558 and the cache write of
 * proveKV/scripts/ppl_validate_multi_agent.py:226-271. */
int pkv_fib_decode_patch_dev(const pkv_fib_profile* p, const uint8_t* payload_dev,
                             int64_t payload_batch_stride, const pkv_layout* layout,
                             float* cache_dev, uint64_t* err_dev, void* stream);

/* The same decode with the cache element type chosen by the caller (PKV_DST_*). */
int pkv_fib_decode_patch_dev_as(const pkv_fib_profile* p, const uint8_t* payload_dev,
                                int64_t payload_batch_stride, const pkv_layout* layout,
                                void* cache_dev, int32_t dst_dtype, uint64_t* err_dev, void* stream);

/* FibQuantizer::decode (fib-quant/src/codec.rs:506-537), the binary64 decoder KVecCodec::decode runs on a
 * single FB1 payload (proveKV/src/codec.rs:612-638): widened codewords, StoredRotation::apply_inverse in
 * binary64 (rotation.rs:118-130), `(value * norm) as f32`.  Its output differs from the batched f32 decoder's
 * in the last bits (fib-quant/tests/decode_batch_fast_parity.rs allows 1e-4).  `_dev`: records and output in
 * device memory, addressed like the decode-and-patch calls (n_replicas must be 1).  The host form takes n
 * bare records ([norm][indices], no header) and writes n x dim floats. */
int pkv_fib_decode_exact_dev(const pkv_fib_profile* p, const uint8_t* payload_dev, int64_t payload_batch_stride,
                             const pkv_layout* layout, float* out_dev, uint64_t* err_dev, void* stream);
int pkv_fib_decode_exact(const pkv_fib_profile* p, const uint8_t* records_host, int64_t n, float* out_host,
                         int32_t* vec_code, int64_t* vec_index);

/* One launch for a cache made of separately allocated tensors (a framework's per-layer K and V
 * tensors, proveKV/scripts/ppl_validate_multi_agent.py:282-293): batch b of the launch (flattened
 * n_batches index) is written at cache_dev + batch_offsets_dev[b] elements, plus the layout's base,
 * token and head terms; the layout's batch_stride values are ignored.  batch_offsets_dev is device
 * memory holding one int64 per batch; an offset must be non-negative and a multiple of 4 elements
 * (8 for the 16-bit types).  The kernel checks that: a violating batch is skipped and reported
 * through the error word as PKV_VEC_MISALIGNED_DST. */
int pkv_fib_decode_patch_dev_multi(const pkv_fib_profile* p, const uint8_t* payload_dev,
                                   int64_t payload_batch_stride, const pkv_layout* layout,
                                   void* cache_dev, const int64_t* batch_offsets_dev, int32_t dst_dtype,
                                   uint64_t* err_dev, void* stream);

/* FibQuantAdapter::encode_batch_compact (proveKV/src/codec.rs:513-525): n vectors
 * of dim f32, contiguous, host memory -> FB2 bytes (19-byte header + n records). */
int pkv_fib_encode_batch_compact(const pkv_fib_profile* p, const float* vectors_host, int64_t n,
                                 uint8_t* out_host, int64_t out_capacity, int64_t* out_len,
                                 int32_t* vec_code, int64_t* vec_index);
/* FibQuantAdapter::decode_batch_compact (proveKV/src/codec.rs:530-569), FB2 only. */
int pkv_fib_decode_batch_compact(const pkv_fib_profile* p, const uint8_t* bytes_host, int64_t len,
                                 float* out_host, int64_t out_capacity_floats, int64_t* n_vectors,
                                 int32_t* vec_code, int64_t* vec_index);

/* Many equal-sized batches in one call: vectors_host is [n_batches][vectors_per_batch][dim],
 * out_host receives n_batches FB2 blobs of 19 + vectors_per_batch*record_bytes bytes each, i.e.
 * what proveKV/src/pool.rs:265-266 obtains from one encode_batch_compact call per (layer, K|V).
 * Copies and kernels of successive chunks overlap; vec_index is the global vector index.
 * When the status is a per-vector code (>= 16) out_host is still complete: the record of every vector
 * the encoder refused (zero norm, non-finite input, norm outside the wire format) is all zero bytes -- a
 * norm field no accepted vector can have -- and every other record is the one a call without the refused
 * vectors would have produced.  The reference fails the whole batch (fib-quant/src/codec.rs:594-610);
 * callers that keep refused vectors raw (fib-quant/src/kv/codec.rs:264-286) read the outcome per vector
 * from the records. */
int pkv_fib_encode_batches_compact(const pkv_fib_profile* p, const float* vectors_host,
                                   int64_t n_batches, int64_t vectors_per_batch, uint8_t* out_host,
                                   int64_t out_capacity, int32_t* vec_code, int64_t* vec_index);
int pkv_fib_decode_batches_compact(const pkv_fib_profile* p, const uint8_t* bytes_host,
                                   int64_t n_batches, int64_t vectors_per_batch, float* out_host,
                                   int64_t out_capacity_floats, int32_t* vec_code, int64_t* vec_index);

/* FB2 header, fib-quant/src/codec.rs:195-220 (19 bytes). */
#define PKV_FB2_HEADER_BYTES 19
int pkv_fb2_header_write(const pkv_fib_profile* p, uint32_t n_vectors, uint8_t* out19);
int pkv_fb2_header_parse(const pkv_fib_profile* p, const uint8_t* bytes, int64_t len,
                         uint32_t* n_vectors);

/* ---- turbo-quant ------------------------------------------------------- */
/* signs: dim values of +-1 (FastHadamardRotation.signs, turbo-quant/src/rotation.rs:152-155);
 * qjl: projections x dim f32 row-major (turbo-quant/src/qjl.rs:341-352), NULL for polar-only;
 * cos_lut/sin_lut: 2^polar_bits values of cosf/sinf at the dequantised angles
 * (turbo-quant/src/polar.rs:91-95,312-313), NULL = computed with the host libm. */
int pkv_turbo_profile_create(const pkv_turbo_config* cfg, const float* signs, const float* qjl,
                             const float* cos_lut, const float* sin_lut, pkv_turbo_profile** out);
int pkv_turbo_profile_destroy(pkv_turbo_profile* p);
/* Bytes per vector in the TQB1 payload (turbo-quant/src/wire.rs:311-327). */
int32_t pkv_turbo_record_bytes(const pkv_turbo_profile* p);

/* Replaces TurboQuantizer::encode per vector (turbo-quant/src/turbo.rs:256-288) and
 * the per-vector part of TurboCodeWireV1::encode_batch_with_radii (wire.rs:350-396). */
int pkv_turbo_encode_dev(const pkv_turbo_profile* p, const float* x_dev, const pkv_layout* layout,
                         uint8_t* payload_dev, int64_t payload_batch_stride, uint64_t* err_dev,
                         void* stream);
/* Replaces TurboCodeWireV1::decode_batch's per-vector part (wire.rs:497-565) and
 * decode_approximate_batch (turbo.rs:414-420), fused with the cache write. */
int pkv_turbo_decode_patch_dev(const pkv_turbo_profile* p, const uint8_t* payload_dev,
                               int64_t payload_batch_stride, const pkv_layout* layout,
                               float* cache_dev, uint64_t* err_dev, void* stream);

int pkv_turbo_decode_patch_dev_as(const pkv_turbo_profile* p, const uint8_t* payload_dev,
                                  int64_t payload_batch_stride, const pkv_layout* layout,
                                  void* cache_dev, int32_t dst_dtype, uint64_t* err_dev, void* stream);

int pkv_turbo_decode_patch_dev_multi(const pkv_turbo_profile* p, const uint8_t* payload_dev,
                                     int64_t payload_batch_stride, const pkv_layout* layout,
                                     void* cache_dev, const int64_t* batch_offsets_dev, int32_t dst_dtype,
                                     uint64_t* err_dev, void* stream);

/* Compressed-domain scoring, TurboQuantizer::score_batch_prepared (turbo-quant/src/turbo.rs:340-381):
 * scores_dev[b * vectors_per_batch + v] = polar inner-product estimate (polar.rs:346-370) plus the
 * QJL correction (qjl.rs:294-330) of record v of batch b against one prepared query, computed from
 * the records without reconstructing the vectors.  rotated_query_dev: dim values, the query after
 * FastHadamardRotation::apply (polar.rs:336-343); projected_query_dev: `projections` values G * query
 * (qjl.rs:266-281), ignored for polar-only profiles; both are what TurboQuantizer::prepare_query
 * (turbo.rs:322-337) returns, in device memory.  Records are validated as in the decode call; a
 * non-finite score is reported as PKV_VEC_NONFINITE_OUTPUT. */
int pkv_turbo_score_dev(const pkv_turbo_profile* p, const uint8_t* payload_dev,
                        int64_t payload_batch_stride, int64_t n_batches, int64_t vectors_per_batch,
                        const float* rotated_query_dev, const float* projected_query_dev,
                        float* scores_dev, uint64_t* err_dev, void* stream);

/* The same for n_queries prepared queries in one pass over the records (a group of query heads that
 * share a KV head, or the queries of several positions): rotated_queries_dev is [n_queries][dim],
 * projected_queries_dev [n_queries][projections], scores_dev [n_queries][n_batches * vectors_per_batch].
 * Each score is the value pkv_turbo_score_dev gives for that query alone; up to eight queries share one
 * read of the records. */
int pkv_turbo_score_queries_dev(const pkv_turbo_profile* p, const uint8_t* payload_dev,
                                int64_t payload_batch_stride, int64_t n_batches, int64_t vectors_per_batch,
                                const float* rotated_queries_dev, const float* projected_queries_dev,
                                int64_t n_queries, float* scores_dev, uint64_t* err_dev, void* stream);

/* TurboQuantizer::prepare_query (turbo-quant/src/turbo.rs:322-337) for queries that already live on the
 * device: rotated_dev[q] = FastHadamardRotation::apply(query q) (polar.rs:336-343), projected_dev[q] = the
 * QJL matrix times query q with every product rounded and the row summed in order (qjl.rs:266-281);
 * projected_dev is ignored for polar-only profiles.  A query, rotated query or projection that is not
 * finite is reported as PKV_VEC_NONFINITE_INPUT with the query's index (the reference's
 * check_finite_vector at each of the three places). */
int pkv_turbo_prepare_queries_dev(const pkv_turbo_profile* p, const float* queries_dev, int64_t n_queries,
                                  float* rotated_dev, float* projected_dev, uint64_t* err_dev, void* stream);

/* TurboQuantAdapter::{encode,decode}_batch_compact (proveKV/src/codec.rs:248-326). */
int pkv_turbo_encode_batch_compact(const pkv_turbo_profile* p, const float* vectors_host, int64_t n,
                                   uint8_t* out_host, int64_t out_capacity, int64_t* out_len,
                                   int32_t* vec_code, int64_t* vec_index);
int pkv_turbo_decode_batch_compact(const pkv_turbo_profile* p, const uint8_t* bytes_host,
                                   int64_t len, float* out_host, int64_t out_capacity_floats,
                                   int64_t* n_vectors, int32_t* vec_code, int64_t* vec_index);

/* Many equal-sized batches in one call (proveKV/src/shell.rs:266-267 issues one
 * encode_batch_compact per (layer, K|V)): TQB1 blobs of 38 + vectors_per_batch*record_bytes. */
int pkv_turbo_encode_batches_compact(const pkv_turbo_profile* p, const float* vectors_host,
                                     int64_t n_batches, int64_t vectors_per_batch, uint8_t* out_host,
                                     int64_t out_capacity, int32_t* vec_code, int64_t* vec_index);
int pkv_turbo_decode_batches_compact(const pkv_turbo_profile* p, const uint8_t* bytes_host,
                                     int64_t n_batches, int64_t vectors_per_batch, float* out_host,
                                     int64_t out_capacity_floats, int32_t* vec_code, int64_t* vec_index);

/* TQB1 header, turbo-quant/src/wire.rs:276-290 (38 bytes). */
#define PKV_TQB1_HEADER_BYTES 38
int pkv_tqb1_header_write(const pkv_turbo_profile* p, uint32_t n_vectors, uint8_t* out38);
int pkv_tqb1_header_parse(const pkv_turbo_profile* p, const uint8_t* bytes, int64_t len,
                          uint32_t* n_vectors);

/* The binary32 arguments (bit patterns, ascending) on which this host's logf (function 0, positive
 * normal arguments) or expf (function 1, |x| <= 89) differs from the portable function; host-only,
 * needs no GPU.  keys_out may be null to ask for the count; *all_one_unit = 1 if every difference is
 * one unit in the last place. */
int pkv_host_libm_exceptions(int32_t function, uint32_t* keys_out, int64_t capacity, int64_t* count,
                             int32_t* all_one_unit);

/* Number of kernel launches this process has issued through the library. */
int64_t pkv_launch_count(void);

/* Test hook, no counterpart in the reference.  While switched on, the encoders that use the tensor
 * cores (turbo with QJL, fib d = 64) do not issue their products, so the bounded wait on the
 * completion barrier runs out after a few hundred polls: the launch reports PKV_VEC_DEVICE_WAIT
 * through the error word, releases its tensor memory and returns, with nothing outstanding on the
 * GPU.  The payload of such a launch is not valid.  Process-wide; switch it off again after use. */
int pkv_test_skip_tensor_issue(int on);

/* Test hook, no counterpart in the reference.  While rotated_dev is not NULL the fib encoders that rotate on
 * the tensor cores (fp16 norm, 5-bit indices, d = 64 / 128) also store every vector's rotated values as the
 * tensor cores delivered them, dim f32 per vector in launch order, so that the error bound assumed for the
 * unit's accumulation (PKV_FIB_ROT_ERR_TC) can be measured against the exact rotation.  The buffer must hold
 * n_vectors * dim floats of every launch made while the hook is on.  Process-wide; NULL switches it off. */
int pkv_test_capture_rotated(float* rotated_dev);

/* Test hook, no counterpart in the reference.  For PolarWithQjl profiles with f32 radii the turbo
 * encoder takes the QJL sketch in the rotated domain (no inverse transform in the common case); while
 * this is switched on it takes the sketch of the residual, as every other profile does, so that tests
 * can compare the two routes byte for byte.  Process-wide. */
int pkv_test_turbo_encode_legacy(int on);

#ifdef __cplusplus
}
#endif
#endif /* PROVEKV_B200_H */
