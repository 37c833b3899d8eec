// Shared declarations of the sm_100a codec kernels: launch geometry, vector
// addressing, the device error word and the profile objects behind the C ABI.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/pkv_portable_math.h"
#include "../../include/provekv_b200.h"

#define PKV_MAX_DIM 128
#define PKV_ERR_NONE 0xFFFFFFFFFFFFFFFFull

// Everything a kernel needs to find the vectors and records of one launch.
struct PkvGeom {
  pkv_layout L;
  int64_t payload_batch_stride;  // bytes between the payloads of two batches
  int32_t vpb;                   // vectors per batch = n_tokens * n_heads
  int32_t tiles_per_batch;       // ceil(vpb / tile vectors)
  int32_t n_batches;             // n_batches[0] * [1] * [2]
  int32_t rec_bytes;             // bytes per vector record
  // Decode only, may be null.  Element offset of each batch's tensor from the cache pointer, for
  // caches made of separately allocated tensors; replaces the batch_stride terms of the layout.
  const int64_t* batch_offsets;
};

// Element offset of vector v of batch `batch` (see pkv_layout in the C header).
__device__ __forceinline__ int64_t pkv_vec_offset(const pkv_layout& L, int batch, int v) {
  int token = v / L.n_heads;
  int head = v - token * L.n_heads;
  int b2 = batch % L.n_batches[2];
  int t = batch / L.n_batches[2];
  int b1 = t % L.n_batches[1];
  int b0 = t / L.n_batches[1];
  return L.base + (int64_t)b0 * L.batch_stride[0] + (int64_t)b1 * L.batch_stride[1] +
         (int64_t)b2 * L.batch_stride[2] + (int64_t)token * L.token_stride +
         (int64_t)head * L.head_stride;
}

// Destination of vector v of batch `batch` in a decode kernel.  With a table of per-batch tensor
// offsets the alignment cannot be checked on the host: a batch whose offset is negative or not a
// multiple of `align` elements (16 bytes) is reported and skipped (PKV_SKIP_DST).
#define PKV_SKIP_DST ((int64_t)0x8000000000000000ll)
__device__ __forceinline__ int64_t pkv_dst_offset(const PkvGeom& g, int batch, int v, int align,
                                                  uint64_t* err);

// Error word: the smallest (pass << 56 | global vector index << 8 | code) wins: within a batch
// the error the reference's sequential loops hit first; across the batches of a launch the
// order is by pass, then by vector.
__device__ __forceinline__ void pkv_report(uint64_t* err, int pass, int64_t gvec, int code) {
  unsigned long long w = ((unsigned long long)pass << 56) | ((unsigned long long)gvec << 8) |
                         (unsigned long long)code;
  atomicMin((unsigned long long*)err, w);
}

__device__ __forceinline__ int64_t pkv_dst_offset(const PkvGeom& g, int batch, int v, int align,
                                                  uint64_t* err) {
  if (g.batch_offsets == nullptr) return pkv_vec_offset(g.L, batch, v);
  const int64_t off = g.batch_offsets[batch];
  if (off < 0 || off % align) {
    pkv_report(err, 0, (int64_t)batch * g.vpb + v, PKV_VEC_MISALIGNED_DST);
    return PKV_SKIP_DST;
  }
  const int token = v / g.L.n_heads, head = v - token * g.L.n_heads;
  return off + g.L.base + (int64_t)token * g.L.token_stride + (int64_t)head * g.L.head_stride;
}

__device__ __forceinline__ bool pkv_finite(float x) {
  return (__float_as_uint(x) & 0x7f800000u) != 0x7f800000u;
}

// Asynchronous global -> shared copies (LDGSTS): a thread queues all of its copies and waits
// once, so a tile's loads are all in flight together instead of one round trip per loop step.
__device__ __forceinline__ void pkv_cp_async16(void* smem_dst, const void* gsrc) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void pkv_cp_async4(void* smem_dst, const void* gsrc) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void pkv_cp_async_wait_all() {
  asm volatile("cp.async.wait_all;" ::: "memory");
}

// Asynchronous bulk copies (the copy engine moves a contiguous run of bytes, 16-byte aligned, a multiple
// of 16 long, and signals an mbarrier with the byte count): one instruction stages a whole tile of
// records or a table.  Plain per-CTA forms only.  Waits are bounded.
__device__ __forceinline__ uint32_t pkv_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void pkv_mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(pkv_smem_u32(bar)), "r"(count) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void pkv_mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(pkv_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void pkv_bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   pkv_smem_u32(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"(pkv_smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ bool pkv_mbar_wait(uint64_t* bar, uint32_t parity, int limit = 1 << 20) {
  const uint32_t a = pkv_smem_u32(bar);
  for (int it = 0; it < limit; it++) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(a), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// IEEE binary16 <-> binary32 in integer arithmetic (round to nearest even), the
// conversion half::f16::from_f32 / to_f32 perform (fib-quant/src/codec.rs:1002,1028).
__device__ __forceinline__ uint32_t pkv_f32_to_f16_bits(float f) {
  const uint32_t x = __float_as_uint(f);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const uint32_t exp = (x >> 23) & 0xffu;
  uint32_t man = x & 0x7fffffu;
  if (exp == 0xffu) return sign | 0x7c00u | (man ? (0x200u | (man >> 13)) : 0u);
  const int e = (int)exp - 127 + 15;
  if (e >= 0x1f) return sign | 0x7c00u;
  if (e <= 0) {
    if (e < -10) return sign;
    man |= 0x800000u;
    const uint32_t shift = (uint32_t)(14 - e);
    uint32_t hm = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u);
    const uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (hm & 1u))) hm++;
    return sign | hm;
  }
  uint32_t h = sign | ((uint32_t)e << 10) | (man >> 13);
  const uint32_t rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
  return h;
}

__device__ __forceinline__ float pkv_f16_bits_to_f32(uint32_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  const uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  if (exp == 0) {
    if (man == 0) return __uint_as_float(sign);
    int e = -1;
    do {
      man <<= 1;
      e++;
    } while (!(man & 0x400u));
    return __uint_as_float(sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13));
  }
  if (exp == 0x1f) return __uint_as_float(sign | 0x7f800000u | (man << 13));
  return __uint_as_float(sign | ((exp + 127 - 15) << 23) | (man << 13));
}

// ---- host libm reproduction (pkv_libm.cu) ---------------------------------
// Arguments on which the host libm's logf / expf differs from the portable (correctly rounded)
// function, always by one unit: sorted keys, one direction bit per key, a bitmap in front.
#define PKV_LIBM_FN_LOG 0
#define PKV_LIBM_FN_EXP 1
#define PKV_ULP_HASH_MUL 0x9E3779B1u
struct PkvUlpTable {
  const uint32_t* keys;   // argument bit patterns, ascending (unsigned)
  const uint32_t* dirs;   // bit i set: host bits = portable bits + 1, clear: - 1
  const uint32_t* bloom;  // 2^bloom_log2 bits, bit (key * PKV_ULP_HASH_MUL) >> (32 - bloom_log2) set for every key
  uint32_t n;
  uint32_t bloom_log2;
};
int pkv_ulp_table_get(int kind, PkvUlpTable* out);

// The host libm's value of the function at `arg`, from the portable value.  Out of line and with the
// table passed as scalars: the callers sit in long unrolled loops (one call site per radius), and a
// reference to a member of a kernel's parameter struct would make the compiler copy the whole struct
// to local memory.
static __device__ __noinline__ float pkv_ulp_lookup(const uint32_t* __restrict__ keys, const uint32_t* __restrict__ dirs,
                                             const uint32_t* __restrict__ bloom, uint32_t n, uint32_t bloom_log2,
                                             float arg, float portable) {
  const uint32_t u = __float_as_uint(arg);
  const uint32_t b = (u * PKV_ULP_HASH_MUL) >> (32u - bloom_log2);
  if (!((__ldg(bloom + (b >> 5)) >> (b & 31u)) & 1u)) return portable;
  uint32_t lo = 0, hi = n;  // first key >= u
  while (lo < hi) {
    const uint32_t mid = (lo + hi) >> 1;
    if (__ldg(keys + mid) < u) lo = mid + 1;
    else hi = mid;
  }
  if (lo >= n || __ldg(keys + lo) != u) return portable;
  const bool up = (__ldg(dirs + (lo >> 5)) >> (lo & 31u)) & 1u;
  return __uint_as_float(__float_as_uint(portable) + (up ? 1u : 0xffffffffu));
}
// A null table = the portable value.
__device__ __forceinline__ float pkv_ulp_adjust(const PkvUlpTable t, float arg, float portable) {
  if (t.keys == nullptr) return portable;
  return pkv_ulp_lookup(t.keys, t.dirs, t.bloom, t.n, t.bloom_log2, arg, portable);
}

// ---- host-side objects ---------------------------------------------------

#define PKV_WS_ERR_WORDS 16
#define PKV_WS_STREAMS 3
struct PkvWorkspace {  // device staging of the *_compact calls, grown on demand
  void* in = nullptr;
  void* out = nullptr;
  uint64_t* err = nullptr;  // PKV_WS_ERR_WORDS error words
  int64_t in_cap = 0, out_cap = 0;
  cudaStream_t streams[PKV_WS_STREAMS] = {nullptr, nullptr, nullptr};  // copy/compute pipeline
};

struct pkv_fib_profile {
  pkv_fib_config cfg;
  int device;
  int idx_bits, norm_len, idx_len, rec_bytes, blocks;
  int orthonormal;      // 1: rows of unit length and M M^T = I to 1e-6, the premise of the shortcut bounds
  double* rot_t_dev;    // [j][r]  = M[r][j], f64 (encode: lanes read consecutive rows)
  float* rot32_dev;     // [row][col] = (f32) M[row][col] (decode, fib-quant/src/rotation.rs:139)
  float* codebook_dev;  // 32 x 4 f32, rows >= N zero-filled
  double* rot_dev;      // [r][j] f64 (exact fix-up of undecided blocks)
  float* rot32_t_dev;   // [j][r] = (f32) M[r][j] (shortcut encoder)
  float* half_norm_dev; // |c|^2 / 2 per codeword
  float* rot_hi_dev;    // [r][j] (f32) M[r][j] with the 13 low significand bits cleared (TF32 operand)
  float* rot_lo_dev;    // [r][j] (f32) M[r][j] - rot_hi, exact
  float score_abs;            // rounding of the fused scores of the dense encoders' search (pkv_fast_paths.h (3))
  uint32_t search_quick_gap;  // for a rotation error of 0 (the Hadamard encoder)
  float search_off, search_ef;  // bias of the Hadamard encoder score search and its error bound (pkv_fib_search.cuh)
  int hadamard;         // 1: encode_batch rotates by the f32 Walsh-Hadamard transform (pkv_fib_profile_create_hadamard)
  float wht_sgn_scale[128];  // sign_i / sqrt(dim) of that transform
  PkvWorkspace ws;
  std::mutex ws_mutex;  // the host-buffer calls of one profile share ws; other profiles run alongside
};

struct pkv_turbo_profile {
  pkv_turbo_config cfg;
  int device;
  int polar_bits, pairs, rec_bytes, radii_words, angle_words, sign_words;
  float scale;              // 1 / sqrtf(dim), turbo-quant/src/rotation.rs:394
  uint32_t sign_mask[4];    // bit i set: signs[i] == -1
  int fast_bucket;          // 1: ray table validated, kernels may use the bucket shortcut
  int ray_count;            // 2^polar_bits / 4 + 1, or 0
  float qjl_thr[64];        // per row: |g_r| * PKV_QJL_REL_BOUND (binary32 sign shortcut)
  float qjl_thr_tf32[64];   // per row: |g_r| * PKV_QJL_TF32_BOUND (tensor-core sign shortcut)
  float* qjl_dev;           // projections x dim, then one sign-shortcut threshold per row
  float* qjl_rot_dev;       // projections x dim: G S H~ with unit-length rows (the rotated-domain sketch)
  float* lut_dev;           // cos[L], sin[L], ray_cos[ray_count], ray_sin[ray_count]
  PkvUlpTable logf_table;   // PKV_LIBM_PLATFORM: the host libm's logf / expf (keys null = portable)
  PkvUlpTable expf_table;
  PkvWorkspace ws;
  std::mutex ws_mutex;
};

// Cache element type of a decode kernel and the round-to-nearest-even store conversion.
template <int DST> struct PkvDst { using type = float; };
template <> struct PkvDst<PKV_DST_F16> { using type = __half; };
template <> struct PkvDst<PKV_DST_BF16> { using type = __nv_bfloat16; };
#ifdef __CUDACC__
template <int DST>
__device__ __forceinline__ uint32_t pkv_pack2(float a, float b) {  // a in the low half
  if constexpr (DST == PKV_DST_F16) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
  } else {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
}
#endif

int pkv_cuda_status(cudaError_t e);
int pkv_check_device(int profile_device);
int pkv_make_geom(const pkv_layout* L, int rec_bytes, int64_t payload_batch_stride, int tile,
                  bool encode, PkvGeom* g);
int pkv_ws_prepare(PkvWorkspace* ws, int64_t in_bytes, int64_t out_bytes);
void pkv_count_launch();
cudaMemPool_t pkv_scratch_pool();  // the library's stream-ordered pool of the current device (scratch lists)
int pkv_skip_tensor_issue();  // test hook, see pkv_test_skip_tensor_issue
float* pkv_rotated_capture();  // test hook, see pkv_test_capture_rotated
int pkv_turbo_encode_legacy();  // test hook, see pkv_test_turbo_encode_legacy

// launchers implemented in pkv_fib.cu / pkv_turbo.cu
int pkv_launch_fib_encode(const pkv_fib_profile* p, const float* x, const PkvGeom& g,
                          uint8_t* payload, uint64_t* err, int batch_numerics, cudaStream_t s);
int pkv_launch_fib_encode_fast_with_scratch(const pkv_fib_profile* p, const float* x, const PkvGeom& g,
                                            uint8_t* payload, uint64_t* err, uint32_t* scratch,
                                            cudaStream_t s);
int pkv_launch_fib_decode(const pkv_fib_profile* p, const uint8_t* payload, const PkvGeom& g,
                          void* cache, int dst, uint64_t* err, cudaStream_t s);  // g.batch_offsets honoured
int pkv_launch_fib_decode_exact(const pkv_fib_profile* p, const uint8_t* payload, const PkvGeom& g, float* out,
                                uint64_t* err, cudaStream_t s);
int pkv_launch_turbo_encode(const pkv_turbo_profile* p, const float* x, const PkvGeom& g,
                            uint8_t* payload, uint64_t* err, cudaStream_t s);
int pkv_launch_turbo_decode(const pkv_turbo_profile* p, const uint8_t* payload, const PkvGeom& g,
                            void* cache, int dst, uint64_t* err, cudaStream_t s);
int pkv_launch_turbo_score(const pkv_turbo_profile* p, const uint8_t* payload, const PkvGeom& g,
                           const float* rotated, const float* projected, int64_t n_queries, float* scores,
                           uint64_t* err, cudaStream_t s);
int pkv_fib_stats_copy(unsigned long long* out4, int reset);
int pkv_turbo_stats_copy(unsigned long long* out4, int reset);
int pkv_launch_turbo_prepare_queries(const pkv_turbo_profile* p, const float* queries, int64_t n_queries,
                                     float* rotated, float* projected, uint64_t* err, cudaStream_t s);
int pkv_fib_tile_vectors(int dim, int encode);
int pkv_turbo_tile_vectors(int dim);
