// fib-quant k=4 cold-tier kernels for sm_100a: batched encode (normalise, dense
// f64 rotation, nearest-of-N codeword per 4-block, 5-bit pack, fp16 norm) and
// decode fused with the write into the KV cache.
//
// Both kernels reproduce the reference's arithmetic order exactly:
//  encode  fib-quant/src/codec.rs:578-729, rotation.rs:104-115,
//          gpu-backend/src/simd_nearest.rs:24-94, fib-quant/src/bitpack.rs:4-44
//  decode  fib-quant/src/codec.rs:797-844, rotation.rs:136-149
// The dense rotation makes them ALU-bound, not HBM-bound: decode needs
// 2*dim*dim separately rounded f32 operations per vector, encode the same count
// in f64.
#include <mutex>

#include <string.h>

#include "pkv_common.cuh"
#include "pkv_fast_paths.h"
#include "pkv_turbo_common.cuh"  // the packed butterfly network (pkv_fib_encode_wht.cuh)

namespace {

// Counters of the certify-or-flag tiers since the last reset (pkv_stats_read): [0] blocks settled by an
// encoder's in-kernel exact tier, [1] list entries redone by fib_encode_fix_kernel with the reference's f64
// sequence.  One atomic per warp and tile at most.
__device__ unsigned long long g_fib_stats[4];
__device__ __forceinline__ void fib_count_flagged(uint32_t flagged, int lane) {
  const unsigned n = __reduce_add_sync(0xffffffffu, (unsigned)__popc(flagged));
  if (lane == 0 && n) atomicAdd(&g_fib_stats[0], (unsigned long long)n);
}

constexpr int kThreads = 128;

__device__ __forceinline__ uint32_t load_bits(const uint8_t* bytes, int pos, int width) {
  // bits [pos, pos+width) of an LSB-first stream, width <= 8
  uint32_t lo = bytes[pos >> 3];
  uint32_t hi = bytes[(pos + width - 1) >> 3];
  return (((hi << 8) | lo) >> (pos & 7)) & ((1u << width) - 1u);
}

// Copy `nbytes` from global (16-byte aligned) into shared memory.
__device__ __forceinline__ void stage_in(uint8_t* dst, const uint8_t* src, int nbytes) {
  int n16 = nbytes >> 4;
  for (int i = threadIdx.x; i < n16; i += blockDim.x)
    pkv_cp_async16(reinterpret_cast<uint4*>(dst) + i, reinterpret_cast<const uint4*>(src) + i);
  for (int i = (n16 << 4) + threadIdx.x; i < nbytes; i += blockDim.x) dst[i] = src[i];
}
__device__ __forceinline__ void stage_out(uint8_t* dst, const uint8_t* src, int nbytes) {
  int n16 = nbytes >> 4;
  for (int i = threadIdx.x; i < n16; i += blockDim.x)
    reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  for (int i = (n16 << 4) + threadIdx.x; i < nbytes; i += blockDim.x) dst[i] = src[i];
}

// acc += m * r on two adjacent accumulators, each lane with a separately rounded product and sum:
// a packed multiply (mul.rn.f32x2), then the packed sum t + acc written as fma.rn.f32x2(t, 1, acc),
// which rounds exactly like an add (t * 1 is exact, signed zeros included).  A literal packed add
// after the packed multiply -- or a multiplier the assembler can see is 1 -- gets contracted into a
// fused multiply-add, which changes the bits; so the pair (1.0f, 1.0f) arrives as a kernel argument.
constexpr unsigned long long kPackedOnes = 0x3f8000003f800000ull;
__device__ __forceinline__ void mul_add2(unsigned long long& acc, float2 m, float2 r,
                                         unsigned long long ones) {
  unsigned long long pm, pr, pt;
  pm = *reinterpret_cast<unsigned long long*>(&m);
  pr = *reinterpret_cast<unsigned long long*>(&r);
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(pt) : "l"(pm), "l"(pr));
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(pt), "l"(ones));
}

// ---------------------------------------------------------------------------
// decode + patch
// ---------------------------------------------------------------------------
// One CTA decodes TV vectors.  Thread (cg, vg) owns columns {4cg..4cg+3} and
// {D/2+4cg..+3} of vectors vg*8 .. vg*8+7 and walks the rows in ascending order,
// so each of its 64 accumulators sees the reference's sum
//   x_c = (((0 + m_0c r_0) + m_1c r_1) + ...)   with separately rounded * and +.
template <int D>
struct FibDec {
  static constexpr int CG = D / 8;
  static constexpr int VG = kThreads / CG;
  static constexpr int TV = VG * 8;
  static constexpr int B = D / 4;
};

template <int D, int DST>
__global__ void __launch_bounds__(kThreads)
fib_decode_patch_kernel(PkvGeom g, const uint8_t* __restrict__ payload,
                        const float* __restrict__ rot32, const float* __restrict__ codebook,
                        int n_codewords, int idx_bits, int norm_len,
                        typename PkvDst<DST>::type* __restrict__ cache, uint64_t* err,
                        unsigned long long ones) {
  using K = FibDec<D>;
  extern __shared__ __align__(128) uint8_t smem[];
  float* s_rot = reinterpret_cast<float*>(smem);                 // [D][D]
  float4* s_cb = reinterpret_cast<float4*>(s_rot + D * D);       // [32]
  int64_t* s_dst = reinterpret_cast<int64_t*>(s_cb + 32);        // [TV]
  float* s_norm = reinterpret_cast<float*>(s_dst + K::TV);       // [TV]
  uint8_t* s_idx = reinterpret_cast<uint8_t*>(s_norm + K::TV);   // [TV][B]
  uint8_t* s_rec = s_idx + K::TV * K::B;                         // [TV][rec] (+16 pad)

  const int tile = blockIdx.x % g.tiles_per_batch;
  const int batch = blockIdx.x / g.tiles_per_batch;
  const int v0 = tile * K::TV;
  const int nv = min(K::TV, g.vpb - v0);
  const int rec = g.rec_bytes;

  // The matrix (16 / 64 KB) and the tile's records arrive by asynchronous bulk copies issued by one
  // thread and counted by an mbarrier; a ragged last tile (not a multiple of 16 bytes) is copied piecewise.
  __shared__ __align__(8) uint64_t s_bar;
  const uint8_t* rec_src = payload + (int64_t)batch * g.payload_batch_stride + (int64_t)v0 * rec;
  const bool rec_bulk = ((nv * rec) & 15) == 0;
  if (threadIdx.x == 0) {
    pkv_mbar_init(&s_bar, 1);
    pkv_mbar_expect_tx(&s_bar, (uint32_t)(D * D * 4 + (rec_bulk ? nv * rec : 0)));
    pkv_bulk_load(s_rot, rot32, D * D * 4, &s_bar);
    if (rec_bulk) pkv_bulk_load(s_rec, rec_src, (uint32_t)(nv * rec), &s_bar);
  }
  if (threadIdx.x < 32) s_cb[threadIdx.x] = __ldg(reinterpret_cast<const float4*>(codebook) + threadIdx.x);
  if (!rec_bulk) stage_in(s_rec, rec_src, nv * rec);
  pkv_cp_async_wait_all();
  __syncthreads();  // the barrier is initialised for everyone; piecewise copies and the codebook are in
  if (!__syncthreads_and(pkv_mbar_wait(&s_bar, 0))) {  // the copies never completed: nothing is decoded
    if (threadIdx.x == 0) pkv_report(err, 0, (int64_t)batch * g.vpb + v0, PKV_VEC_DEVICE_WAIT);
    return;
  }

  // unpack + validate: one thread per vector (checks in the reference's order)
  for (int v = threadIdx.x; v < K::TV; v += kThreads) {
    float nf = 0.0f;
    if (v < nv) {
      const uint8_t* r = s_rec + v * rec;
      const int64_t gvec = (int64_t)batch * g.vpb + v0 + v;
      int code = 0;
      const int used = K::B * idx_bits;
      for (int pos = used; pos < (((used + 7) >> 3) << 3); pos++)
        if ((r[norm_len + (pos >> 3)] >> (pos & 7)) & 1) code = PKV_VEC_PADDING_BITS;
      for (int b = 0; b < K::B; b++) {
        uint32_t idx = load_bits(r + norm_len, b * idx_bits, idx_bits);
        if (idx >= (uint32_t)n_codewords) {
          if (!code) code = PKV_VEC_INDEX_RANGE;
          idx = 0;
        }
        s_idx[v * K::B + b] = (uint8_t)idx;
      }
      if (norm_len == 2) {
        nf = pkv_f16_bits_to_f32((uint32_t)r[0] | ((uint32_t)r[1] << 8));
      } else {
        nf = __uint_as_float((uint32_t)r[0] | ((uint32_t)r[1] << 8) | ((uint32_t)r[2] << 16) |
                             ((uint32_t)r[3] << 24));
      }
      if (!(pkv_finite(nf) && nf > 0.0f)) {
        if (!code) code = PKV_VEC_BAD_NORM;
      }
      if (code) pkv_report(err, 0, gvec, code);
      s_dst[v] = pkv_dst_offset(g, batch, v0 + v, DST == PKV_DST_F32 ? 4 : 8, err);
    } else {
      for (int b = 0; b < K::B; b++) s_idx[v * K::B + b] = 0;
      s_dst[v] = 0;
    }
    s_norm[v] = nf;
  }
  __syncthreads();

  const int cg = threadIdx.x % K::CG, vg = threadIdx.x / K::CG;
  const int cA = 4 * cg, cB = D / 2 + 4 * cg;
  unsigned long long acc[8][4];  // packed pairs of adjacent columns
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int c = 0; c < 4; c++) acc[i][c] = 0ull;

#pragma unroll 1
  for (int b = 0; b < K::B; b++) {
    float4 cw[8];
#pragma unroll
    for (int i = 0; i < 8; i++) cw[i] = s_cb[s_idx[(vg * 8 + i) * K::B + b]];
#pragma unroll
    for (int rr = 0; rr < 4; rr++) {
      const float* mrow = s_rot + (4 * b + rr) * D;
      const float4 mA = *reinterpret_cast<const float4*>(mrow + cA);
      const float4 mB = *reinterpret_cast<const float4*>(mrow + cB);
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const float r = rr == 0 ? cw[i].x : rr == 1 ? cw[i].y : rr == 2 ? cw[i].z : cw[i].w;
        // two columns per instruction, each lane rounded on its own: the same two IEEE
        // operations per element as the scalar form
        const float2 rr2 = make_float2(r, r);
        mul_add2(acc[i][0], make_float2(mA.x, mA.y), rr2, ones);
        mul_add2(acc[i][1], make_float2(mA.z, mA.w), rr2, ones);
        mul_add2(acc[i][2], make_float2(mB.x, mB.y), rr2, ones);
        mul_add2(acc[i][3], make_float2(mB.z, mB.w), rr2, ones);
      }
    }
  }

#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int v = vg * 8 + i;
    if (v >= nv || s_dst[v] == PKV_SKIP_DST) continue;
    const float nf = s_norm[v];
    float o[8];
    bool ok = true;
#pragma unroll
    for (int c = 0; c < 8; c++) {
      const uint32_t bits = (uint32_t)(acc[i][c >> 1] >> (32 * (c & 1)));
      o[c] = __fmul_rn(__uint_as_float(bits), nf);
      ok = ok && pkv_finite(o[c]);
    }
    if (!ok) pkv_report(err, 0, (int64_t)batch * g.vpb + v0 + v, PKV_VEC_NONFINITE_OUTPUT);
    typename PkvDst<DST>::type* dst = cache + s_dst[v];
    for (int r = 0; r < g.L.n_replicas; r++) {
      if constexpr (DST == PKV_DST_F32) {
        *reinterpret_cast<float4*>(dst + cA) = make_float4(o[0], o[1], o[2], o[3]);
        *reinterpret_cast<float4*>(dst + cB) = make_float4(o[4], o[5], o[6], o[7]);
      } else {  // the finite check above is on the f32 values, as in the reference; the cast comes after
        *reinterpret_cast<uint2*>(dst + cA) = make_uint2(pkv_pack2<DST>(o[0], o[1]), pkv_pack2<DST>(o[2], o[3]));
        *reinterpret_cast<uint2*>(dst + cB) = make_uint2(pkv_pack2<DST>(o[4], o[5]), pkv_pack2<DST>(o[6], o[7]));
      }
      dst += g.L.replica_stride;
    }
  }
}

// FibQuantizer::decode (fib-quant/src/codec.rs:506-537), the decoder behind KVecCodec::decode for one
// payload (proveKV/src/codec.rs:612-638): binary64 throughout -- codewords widened, x_c = sum over
// rows of M[row][c] * r_row (rows ascending, separately rounded * and +, rotation.rs:118-130), then
// (f32)(x_c * norm).  One thread per (vector, column); 128 / D vectors per CTA.  Not a throughput
// path: the batched decoders above are what pools and shells use.
template <int D>
__global__ void __launch_bounds__(kThreads)
fib_decode_exact_kernel(PkvGeom g, const uint8_t* __restrict__ payload, const double* __restrict__ rot,
                        const float* __restrict__ codebook, int n_codewords, int idx_bits, int norm_len,
                        float* __restrict__ out, uint64_t* err) {
  constexpr int B = D / 4, VPC = kThreads / D == 0 ? 1 : kThreads / D;
  __shared__ double s_r[VPC][D];
  __shared__ double s_norm[VPC];
  __shared__ int s_code[VPC];
  const int vl = threadIdx.x / D, c = threadIdx.x % D;
  const int64_t n = (int64_t)g.n_batches * g.vpb;
  const int64_t gvec = (int64_t)blockIdx.x * VPC + vl;
  const bool active = vl < VPC && gvec < n;
  const int batch = active ? (int)(gvec / g.vpb) : 0, v = active ? (int)(gvec % g.vpb) : 0;
  const uint8_t* r = payload + (int64_t)batch * g.payload_batch_stride + (int64_t)v * g.rec_bytes;
  if (active && c == 0) {
    int code = 0;
    const int used = B * idx_bits;
    for (int pos = used; pos < (((used + 7) >> 3) << 3); pos++)
      if ((r[norm_len + (pos >> 3)] >> (pos & 7)) & 1) code = PKV_VEC_PADDING_BITS;
    for (int b = 0; b < B; b++) {
      uint32_t idx = load_bits(r + norm_len, b * idx_bits, idx_bits);
      if (idx >= (uint32_t)n_codewords) {
        if (!code) code = PKV_VEC_INDEX_RANGE;
        idx = 0;
      }
      for (int j = 0; j < 4; j++) s_r[vl][4 * b + j] = (double)codebook[4 * idx + j];
    }
    float nf;
    if (norm_len == 2) nf = pkv_f16_bits_to_f32((uint32_t)r[0] | ((uint32_t)r[1] << 8));
    else nf = __uint_as_float((uint32_t)r[0] | ((uint32_t)r[1] << 8) | ((uint32_t)r[2] << 16) | ((uint32_t)r[3] << 24));
    if (!code && !(pkv_finite(nf) && nf > 0.0f)) code = PKV_VEC_BAD_NORM;
    s_norm[vl] = (double)nf;
    s_code[vl] = code;
    if (code) pkv_report(err, 0, gvec, code);
  }
  __syncthreads();
  if (!active || s_code[vl]) return;
  double sum = 0.0;
  for (int row = 0; row < D; row++) sum = __dadd_rn(sum, __dmul_rn(rot[row * D + c], s_r[vl][row]));
  const float o = __double2float_rn(__dmul_rn(sum, s_norm[vl]));
  if (!pkv_finite(o)) pkv_report(err, 0, gvec, PKV_VEC_NONFINITE_OUTPUT);
  out[pkv_vec_offset(g.L, batch, v) + c] = o;
}

template <int D>
size_t fib_decode_smem(int rec) {
  using K = FibDec<D>;
  return sizeof(float) * D * D + sizeof(float4) * 32 + sizeof(int64_t) * K::TV +
         sizeof(float) * K::TV + K::TV * K::B + (size_t)K::TV * rec + 16;
}


// ---------------------------------------------------------------------------
// encode
// ---------------------------------------------------------------------------
// One CTA encodes TV vectors in three steps: (A) per-vector f64 norm and the
// normalised vector, (B) rotation + argmin with thread (bg, vg) owning block bg
// (rows 4bg..4bg+3) of vectors vg*8..vg*8+7, (C) per-vector bit packing.
template <int D>
struct FibEnc {
  static constexpr int B = D / 4;
  static constexpr int VG = kThreads / B;
  static constexpr int TV = VG * 8;
  static constexpr int XS = D + 1;  // padded row strides (elements)
};

__device__ __forceinline__ int nearest_codeword(const float4* s_cb, int n, int order, float s0,
                                                float s1, float s2, float s3) {
  int best = 0;
  float best_dist = __int_as_float(0x7f800000);
  const int paired = order == PKV_ARGMIN_PAIRWISE ? (n & ~1) : 0;
  for (int c = 0; c < n; c++) {
    const float4 w = s_cb[c];
    float dist;
    if (c < paired) {  // gpu-backend/src/simd_nearest.rs:62-70: (q0+q1)+(q2+q3), delta = cw - s
      const float d0 = __fsub_rn(w.x, s0), d1 = __fsub_rn(w.y, s1);
      const float d2 = __fsub_rn(w.z, s2), d3 = __fsub_rn(w.w, s3);
      dist = __fadd_rn(__fadd_rn(__fmul_rn(d0, d0), __fmul_rn(d1, d1)),
                       __fadd_rn(__fmul_rn(d2, d2), __fmul_rn(d3, d3)));
    } else {  // :24-39 and the odd tail :82-92: ((q0+q1)+q2)+q3, delta = s - cw
      const float d0 = __fsub_rn(s0, w.x), d1 = __fsub_rn(s1, w.y);
      const float d2 = __fsub_rn(s2, w.z), d3 = __fsub_rn(s3, w.w);
      dist = __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(d0, d0), __fmul_rn(d1, d1)),
                                 __fmul_rn(d2, d2)),
                       __fmul_rn(d3, d3));
    }
    if (dist < best_dist) {
      best_dist = dist;
      best = c;
    }
  }
  return best;
}

template <int D>
__global__ void __launch_bounds__(kThreads)
fib_encode_kernel(PkvGeom g, const float* __restrict__ x, const double* __restrict__ rot_t,
                  const float* __restrict__ codebook, int n_codewords, int idx_bits, int norm_len,
                  int argmin_order, int batch_numerics, uint8_t* __restrict__ payload,
                  uint64_t* err) {
  using K = FibEnc<D>;
  extern __shared__ __align__(128) uint8_t smem[];
  double* s_rot = reinterpret_cast<double*>(smem);                 // [j][r]
  double* s_nrm = s_rot + D * D;                                   // [TV][XS]
  double* s_norm = s_nrm + K::TV * K::XS;                          // [TV]
  float4* s_cb = reinterpret_cast<float4*>(s_norm + K::TV);        // [32]
  float* s_x = reinterpret_cast<float*>(s_cb + 32);                // [TV][XS]
  uint8_t* s_idx = reinterpret_cast<uint8_t*>(s_x + K::TV * K::XS);  // [TV][B]
  uint8_t* s_bad = s_idx + K::TV * K::B;                           // [TV]
  uint8_t* s_rec = s_bad + K::TV;                                  // [TV][rec], 16-aligned below

  const int tile = blockIdx.x % g.tiles_per_batch;
  const int batch = blockIdx.x / g.tiles_per_batch;
  const int v0 = tile * K::TV;
  const int nv = min(K::TV, g.vpb - v0);
  const int rec = g.rec_bytes;
  s_rec += (16 - (reinterpret_cast<uintptr_t>(s_rec) & 15)) & 15;

  for (int i = threadIdx.x; i < D * D / 2; i += kThreads)
    pkv_cp_async16(reinterpret_cast<double2*>(s_rot) + i, reinterpret_cast<const double2*>(rot_t) + i);
  if (threadIdx.x < 32) s_cb[threadIdx.x] = __ldg(reinterpret_cast<const float4*>(codebook) + threadIdx.x);
  // load the tile: D/4 lanes per vector, one float4 each
  for (int i = threadIdx.x; i < K::TV * (D / 4); i += kThreads) {
    const int v = i / (D / 4), q = i % (D / 4);
    float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
    if (v < nv)
      val = __ldg(reinterpret_cast<const float4*>(x + pkv_vec_offset(g.L, batch, v0 + v)) + q);
    float* d = s_x + v * K::XS + 4 * q;
    d[0] = val.x; d[1] = val.y; d[2] = val.z; d[3] = val.w;
  }
  pkv_cp_async_wait_all();
  __syncthreads();

  // (A) check_finite, l2_norm (f64, sequential), fib-quant/src/codec.rs:601-606,1049-1064
  for (int v = threadIdx.x; v < K::TV; v += kThreads) {
    const float* xv = s_x + v * K::XS;
    bool finite = true;
    double acc = 0.0;
    for (int j = 0; j < D; j++) {
      const float f = xv[j];
      finite = finite && pkv_finite(f);
      const double t = (double)f;
      acc = __dadd_rn(acc, __dmul_rn(t, t));
    }
    double norm = __dsqrt_rn(acc);
    int bad = 0;
    if (v < nv) {
      if (!finite) bad = PKV_VEC_NONFINITE_INPUT;
      else if (norm == 0.0) bad = PKV_VEC_ZERO_NORM;
      if (bad) pkv_report(err, 0, (int64_t)batch * g.vpb + v0 + v, bad);
    }
    if (bad || v >= nv) norm = 1.0;
    s_norm[v] = norm;
    s_bad[v] = (uint8_t)(bad || v >= nv);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < K::TV * D; i += kThreads) {
    const int v = i / D, j = i % D;
    double q = __ddiv_rn((double)s_x[v * K::XS + j], s_norm[v]);
    if (batch_numerics) q = (double)__double2float_rn(q);  // :607-609 then :662
    if (s_bad[v]) q = 0.0;
    s_nrm[v * K::XS + j] = q;
  }
  __syncthreads();

  // (B) StoredRotation::apply (rotation.rs:104-115): y_r = sum_j M[r][j] n_j, j ascending, f64
  const int bg = threadIdx.x % K::B, vg = threadIdx.x / K::B;
  double acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int r = 0; r < 4; r++) acc[i][r] = 0.0;
#pragma unroll 2
  for (int j = 0; j < D; j++) {
    const double2 m01 = *reinterpret_cast<const double2*>(s_rot + j * D + 4 * bg);
    const double2 m23 = *reinterpret_cast<const double2*>(s_rot + j * D + 4 * bg + 2);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const double nj = s_nrm[(vg * 8 + i) * K::XS + j];
      acc[i][0] = __dadd_rn(acc[i][0], __dmul_rn(m01.x, nj));
      acc[i][1] = __dadd_rn(acc[i][1], __dmul_rn(m01.y, nj));
      acc[i][2] = __dadd_rn(acc[i][2], __dmul_rn(m23.x, nj));
      acc[i][3] = __dadd_rn(acc[i][3], __dmul_rn(m23.y, nj));
    }
  }
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int idx = nearest_codeword(s_cb, n_codewords, argmin_order, __double2float_rn(acc[i][0]),
                                     __double2float_rn(acc[i][1]), __double2float_rn(acc[i][2]),
                                     __double2float_rn(acc[i][3]));
    s_idx[(vg * 8 + i) * K::B + bg] = (uint8_t)idx;
  }
  __syncthreads();

  // (C) encode_norm (:994-1020) + pack_indices (bitpack.rs:4-44)
  for (int v = threadIdx.x; v < nv; v += kThreads) {
    uint8_t* r = s_rec + v * rec;
    for (int i = 0; i < rec; i++) r[i] = 0;
    if (s_bad[v]) continue;
    const float nf = __double2float_rn(s_norm[v]);
    bool ok;
    if (norm_len == 2) {
      const uint32_t h = pkv_f32_to_f16_bits(nf);
      ok = (h & 0x7fffu) < 0x7c00u && (h & 0x7fffu) != 0;
      r[0] = (uint8_t)(h & 0xff);
      r[1] = (uint8_t)(h >> 8);
    } else {
      const uint32_t u = __float_as_uint(nf);
      ok = pkv_finite(nf) && nf > 0.0f;
      r[0] = (uint8_t)u; r[1] = (uint8_t)(u >> 8); r[2] = (uint8_t)(u >> 16); r[3] = (uint8_t)(u >> 24);
    }
    if (!ok) {
      pkv_report(err, 1, (int64_t)batch * g.vpb + v0 + v, PKV_VEC_NORM_RANGE);
      for (int i = 0; i < norm_len; i++) r[i] = 0;
      continue;
    }
    for (int b = 0; b < K::B; b++) {
      const int pos = b * idx_bits;
      const uint32_t val = (uint32_t)s_idx[v * K::B + b] << (pos & 7);
      r[norm_len + (pos >> 3)] |= (uint8_t)val;
      if (val >> 8) r[norm_len + (pos >> 3) + 1] |= (uint8_t)(val >> 8);
    }
  }
  __syncthreads();
  stage_out(payload + (int64_t)batch * g.payload_batch_stride + (int64_t)v0 * rec, s_rec, nv * rec);
}

template <int D>
size_t fib_encode_smem(int rec) {
  using K = FibEnc<D>;
  return sizeof(double) * D * D + sizeof(double) * K::TV * K::XS + sizeof(double) * K::TV +
         sizeof(float4) * 32 + sizeof(float) * K::TV * K::XS + K::TV * K::B + K::TV +
         (size_t)K::TV * rec + 32;
}

#include "pkv_fib_search.cuh"
#include "pkv_fib_encode_fast.cuh"
#include "pkv_fib_encode_tc.cuh"
#include "pkv_fib_encode_tc128.cuh"
#include "pkv_fib_encode_wht.cuh"

template <typename F>
int set_smem(F kernel, size_t bytes) {
  if (bytes > 48 * 1024)
    return pkv_cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return PKV_OK;
}

}  // namespace

int pkv_fib_tile_vectors(int dim, int encode) {
  if (dim == 64) return encode ? FibEnc<64>::TV : FibDec<64>::TV;
  if (dim == 128) return encode ? FibEnc<128>::TV : FibDec<128>::TV;
  return 0;
}

// Shortcut path: fast kernel over all vectors, then the exact fix-up of the listed entries.  The
// list (one counter + at most one entry per vector) is scratch memory taken from the pool above,
// ordered on the caller's stream, for the duration of the two launches.
template <int D>
int launch_fib_encode_fast(const pkv_fib_profile* p, const float* x, const PkvGeom& g,
                           uint8_t* payload, uint64_t* err, cudaStream_t s) {
  const int64_t n = (int64_t)g.n_batches * g.vpb;
  cudaMemPool_t pool = pkv_scratch_pool();
  if (!pool) return PKV_ERR_CUDA;
  uint32_t* scratch = nullptr;
  if (cudaError_t ce = cudaMallocFromPoolAsync((void**)&scratch, sizeof(uint32_t) * (size_t)(n + 1), pool, s)) return pkv_cuda_status(ce);
  int st = pkv_launch_fib_encode_fast_with_scratch(p, x, g, payload, err, scratch, s);
  if (cudaFreeAsync(scratch, s) != cudaSuccess && st == PKV_OK) st = PKV_ERR_CUDA;
  return st;
}

int pkv_launch_fib_encode(const pkv_fib_profile* p, const float* x, const PkvGeom& g,
                          uint8_t* payload, uint64_t* err, int batch_numerics, cudaStream_t s) {
  const int64_t grid = (int64_t)g.n_batches * g.tiles_per_batch;
  if (grid == 0) return PKV_OK;
  if (grid > 0x7fffffff) return PKV_ERR_UNSUPPORTED;
  // A Hadamard profile: the reference's `gpu` build takes the transform for batches of at least 16
  // vectors (GpuContext::GPU_MIN_BATCH_SIZE, gpu-backend/src/lib.rs:61-63; dim >= 64 always holds here)
  // and the stored matrix below that; PKV_FIB_NUMERICS_BATCH forces the transform for every size.
  if (p->hadamard && (p->cfg.numerics == PKV_FIB_NUMERICS_BATCH || g.vpb >= 16)) {
    FibWhtParams prm;
    memcpy(prm.sgn_scale, p->wht_sgn_scale, sizeof(prm.sgn_scale));
    PkvGeom gf = g;
    int st;
#define PKV_FIB_WHT(DIM)                                                                              \
  {                                                                                                   \
    gf.tiles_per_batch = (g.vpb + FibWht<DIM>::TV - 1) / FibWht<DIM>::TV;                             \
    const int64_t tiles = (int64_t)g.n_batches * gf.tiles_per_batch;                                  \
    if (tiles > 0x7fffffff) return PKV_ERR_UNSUPPORTED;                                               \
    const size_t sm = FibWht<DIM>::smem(g.rec_bytes);                                                 \
    if ((st = set_smem(fib_encode_wht_kernel<DIM>, sm)) != PKV_OK) return st;                         \
    fib_encode_wht_kernel<DIM><<<(unsigned)tiles, FibWht<DIM>::THREADS, sm, s>>>(                     \
        gf, x, prm, p->codebook_dev, p->half_norm_dev, p->cfg.codebook_size, p->idx_bits, p->norm_len, \
        p->cfg.argmin_order, FibSearchBias{p->search_off, p->search_ef, 32u, p->search_quick_gap}, payload, err); \
  }
    if (p->cfg.dim == 64) PKV_FIB_WHT(64)
    else if (p->cfg.dim == 128) PKV_FIB_WHT(128)
    else return PKV_ERR_UNSUPPORTED;
#undef PKV_FIB_WHT
    pkv_count_launch();
    return pkv_cuda_status(cudaGetLastError());
  }
  // The shortcuts are proven for the batch numerics; list entries hold 27-bit vector indices.
  if (batch_numerics && p->orthonormal && (int64_t)g.n_batches * g.vpb <= ((int64_t)1 << 27)) {
    if (p->cfg.dim == 64) return launch_fib_encode_fast<64>(p, x, g, payload, err, s);
    if (p->cfg.dim == 128) return launch_fib_encode_fast<128>(p, x, g, payload, err, s);
    return PKV_ERR_UNSUPPORTED;
  }
  int st;
#define PKV_FIB_ENC(DIM)                                                                          \
  {                                                                                               \
    const size_t sm = fib_encode_smem<DIM>(g.rec_bytes);                                          \
    if ((st = set_smem(fib_encode_kernel<DIM>, sm)) != PKV_OK) return st;                         \
    fib_encode_kernel<DIM><<<(unsigned)grid, kThreads, sm, s>>>(                                  \
        g, x, p->rot_t_dev, p->codebook_dev, p->cfg.codebook_size, p->idx_bits, p->norm_len,      \
        p->cfg.argmin_order, batch_numerics, payload, err);                                       \
  }
  if (p->cfg.dim == 64) PKV_FIB_ENC(64)
  else if (p->cfg.dim == 128) PKV_FIB_ENC(128)
  else return PKV_ERR_UNSUPPORTED;
#undef PKV_FIB_ENC
  pkv_count_launch();
  return pkv_cuda_status(cudaGetLastError());
}

// scratch: uint32 counter followed by room for one uint32 entry per vector of the launch.
int pkv_launch_fib_encode_fast_with_scratch(const pkv_fib_profile* p, const float* x, const PkvGeom& g,
                                            uint8_t* payload, uint64_t* err, uint32_t* scratch,
                                            cudaStream_t s) {
  if (cudaError_t ce = cudaMemsetAsync(scratch, 0, sizeof(uint32_t), s)) return pkv_cuda_status(ce);
  int st;
  // the cold-tier default shape takes the tensor-core kernel
  if (p->cfg.dim == 64 && p->norm_len == 2 && p->idx_bits == 5) {
    PkvGeom gf = g;
    gf.tiles_per_batch = (g.vpb + FibTc::TV - 1) / FibTc::TV;
    const int64_t tiles = (int64_t)g.n_batches * gf.tiles_per_batch;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t quads = (tiles + FibTc::NWARPS - 1) / FibTc::NWARPS;
    const int64_t grid = quads < (int64_t)sms * 3 ? quads : (int64_t)sms * 3;  // persistent: 3 CTAs per SM
    if ((st = set_smem(fib_encode_tc_kernel, FibTc::SMEM)) != PKV_OK) return st;
    fib_encode_tc_kernel<<<(unsigned)grid, FibTc::THREADS, FibTc::SMEM, s>>>(
        gf, x, p->rot_hi_dev, p->rot_lo_dev, p->codebook_dev, p->half_norm_dev, p->cfg.codebook_size, p->rot_dev,
        p->cfg.argmin_order, p->score_abs, payload, err, scratch, scratch + 1, pkv_skip_tensor_issue(), pkv_rotated_capture());
    pkv_count_launch();
    // the in-kernel exact tier leaves only boundary cases on the list: one CTA per SM is plenty
    fib_encode_fix_kernel<64><<<sms, kThreads, 0, s>>>(
        gf, x, p->rot_dev, p->codebook_dev, p->cfg.codebook_size, p->idx_bits, p->norm_len,
        p->cfg.argmin_order, payload, scratch, scratch + 1);
    pkv_count_launch();
    return pkv_cuda_status(cudaGetLastError());
  }
  if (p->cfg.dim == 128 && p->norm_len == 2 && p->idx_bits == 5) {
    PkvGeom gf = g;
    gf.tiles_per_batch = (g.vpb + FibTc128::ROWS - 1) / FibTc128::ROWS;
    const int64_t tiles = (int64_t)g.n_batches * gf.tiles_per_batch;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int64_t grid = tiles < (int64_t)sms ? tiles : (int64_t)sms;  // persistent: one CTA per SM
    if ((st = set_smem(fib_encode_tc128_kernel, FibTc128::SMEM)) != PKV_OK) return st;
    fib_encode_tc128_kernel<<<(unsigned)grid, FibTc128::THREADS, FibTc128::SMEM, s>>>(
        gf, x, p->rot_hi_dev, p->rot_lo_dev, p->codebook_dev, p->half_norm_dev, p->cfg.codebook_size, p->rot_dev,
        p->cfg.argmin_order, p->score_abs, payload, err, scratch, scratch + 1, pkv_skip_tensor_issue(), pkv_rotated_capture());
    pkv_count_launch();
    fib_encode_fix_kernel<128><<<sms, kThreads, 0, s>>>(
        gf, x, p->rot_dev, p->codebook_dev, p->cfg.codebook_size, p->idx_bits, p->norm_len,
        p->cfg.argmin_order, payload, scratch, scratch + 1);
    pkv_count_launch();
    return pkv_cuda_status(cudaGetLastError());
  }
#define PKV_FIB_FAST(DIM)                                                                           \
  {                                                                                                 \
    PkvGeom gf = g;                                                                                 \
    gf.tiles_per_batch = (g.vpb + FibFast<DIM>::TV - 1) / FibFast<DIM>::TV;                         \
    const int64_t grid = (int64_t)g.n_batches * gf.tiles_per_batch;                                 \
    if (grid > 0x7fffffff) return PKV_ERR_UNSUPPORTED;                                              \
    const size_t sm = fib_encode_fast_smem<DIM>(g.rec_bytes);                                       \
    if ((st = set_smem(fib_encode_fast_kernel<DIM>, sm)) != PKV_OK) return st;                      \
    fib_encode_fast_kernel<DIM><<<(unsigned)grid, FibFast<DIM>::THREADS, sm, s>>>(                             \
        gf, x, p->rot32_t_dev, p->codebook_dev, p->half_norm_dev, p->cfg.codebook_size, p->idx_bits, \
        p->norm_len, p->score_abs, payload, err, scratch, scratch + 1);                             \
    pkv_count_launch();                                                                             \
    fib_encode_fix_kernel<DIM><<<148 * 8, kThreads, 0, s>>>(                                            \
        gf, x, p->rot_dev, p->codebook_dev, p->cfg.codebook_size, p->idx_bits, p->norm_len,         \
        p->cfg.argmin_order, payload, scratch, scratch + 1);                                        \
    pkv_count_launch();                                                                             \
  }
  if (p->cfg.dim == 64) PKV_FIB_FAST(64)
  else if (p->cfg.dim == 128) PKV_FIB_FAST(128)
  else return PKV_ERR_UNSUPPORTED;
#undef PKV_FIB_FAST
  return pkv_cuda_status(cudaGetLastError());
}

int pkv_launch_fib_decode(const pkv_fib_profile* p, const uint8_t* payload, const PkvGeom& g,
                          void* cache, int dst, uint64_t* err, cudaStream_t s) {
  const int64_t grid = (int64_t)g.n_batches * g.tiles_per_batch;
  if (grid == 0) return PKV_OK;
  if (grid > 0x7fffffff) return PKV_ERR_UNSUPPORTED;
  int st;
#define PKV_FIB_DEC(DIM, DST)                                                                     \
  {                                                                                               \
    const size_t sm = fib_decode_smem<DIM>(g.rec_bytes);                                          \
    if ((st = set_smem(fib_decode_patch_kernel<DIM, DST>, sm)) != PKV_OK) return st;              \
    fib_decode_patch_kernel<DIM, DST><<<(unsigned)grid, kThreads, sm, s>>>(                       \
        g, payload, p->rot32_dev, p->codebook_dev, p->cfg.codebook_size, p->idx_bits,             \
        p->norm_len, static_cast<PkvDst<DST>::type*>(cache), err, kPackedOnes);                   \
  }
#define PKV_FIB_DEC_DST(DIM)                                                                      \
  switch (dst) {                                                                                  \
    case PKV_DST_F32: PKV_FIB_DEC(DIM, PKV_DST_F32) break;                                        \
    case PKV_DST_F16: PKV_FIB_DEC(DIM, PKV_DST_F16) break;                                        \
    case PKV_DST_BF16: PKV_FIB_DEC(DIM, PKV_DST_BF16) break;                                      \
    default: return PKV_ERR_INVALID_ARGUMENT;                                                     \
  }
  if (p->cfg.dim == 64) PKV_FIB_DEC_DST(64)
  else if (p->cfg.dim == 128) PKV_FIB_DEC_DST(128)
  else return PKV_ERR_UNSUPPORTED;
#undef PKV_FIB_DEC_DST
#undef PKV_FIB_DEC
  pkv_count_launch();
  return pkv_cuda_status(cudaGetLastError());
}

int pkv_launch_fib_decode_exact(const pkv_fib_profile* p, const uint8_t* payload, const PkvGeom& g, float* out,
                                uint64_t* err, cudaStream_t s) {
  const int64_t n = (int64_t)g.n_batches * g.vpb;
  if (n == 0) return PKV_OK;
  const int vpc = p->cfg.dim == 64 ? 2 : 1;
  const int64_t grid = (n + vpc - 1) / vpc;
  if (grid > 0x7fffffff) return PKV_ERR_UNSUPPORTED;
  if (p->cfg.dim == 64)
    fib_decode_exact_kernel<64><<<(unsigned)grid, kThreads, 0, s>>>(g, payload, p->rot_dev, p->codebook_dev,
                                                                   p->cfg.codebook_size, p->idx_bits, p->norm_len, out, err);
  else if (p->cfg.dim == 128)
    fib_decode_exact_kernel<128><<<(unsigned)grid, kThreads, 0, s>>>(g, payload, p->rot_dev, p->codebook_dev,
                                                                    p->cfg.codebook_size, p->idx_bits, p->norm_len, out, err);
  else return PKV_ERR_UNSUPPORTED;
  pkv_count_launch();
  return pkv_cuda_status(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// fib encode without any allocation
// ---------------------------------------------------------------------------
// Some embedders may not allocate device memory on the call path at all: a serving process
// whose memory is fully budgeted up front (every byte of HBM handed to the KV cache and the
// weights at start-up), a caller running under an allocator it must not re-enter, or code that
// has already frozen its memory layout.  pkv_fib_encode_dev takes the undecided-block list of the
// shortcut encoder from the stream's memory pool; the entry point below uses a fixed array that
// is part of the loaded library image instead, so it calls no allocating routine whatsoever.
//
// The array holds one counter and one entry per vector, which bounds a call to
// PKV_FIB_STATIC_MAX_VECTORS vectors.  Every GPU that loads the library carries these 4 MiB until
// the process exits.  All calls on a device share the array and it keeps the previous call's
// contents: the counter is zeroed at the start of each call, and two calls whose kernels overlap
// on the GPU (different streams, no ordering) would corrupt each other's list.
static __device__ __align__(256) uint32_t g_fib_static_scratch[PKV_FIB_STATIC_MAX_VECTORS + 64];

namespace {
std::mutex g_static_mutex;
uint32_t* g_static_scratch_ptr[64] = {};  // device address of the array, per device ordinal
}  // namespace

extern "C" int pkv_fib_encode_dev_static(const pkv_fib_profile* p, const float* x_dev,
                                         const pkv_layout* layout, uint8_t* payload_dev,
                                         int64_t payload_batch_stride, uint64_t* err_dev,
                                         void* stream) {
  if (!p || !x_dev || !payload_dev || !err_dev) return PKV_ERR_INVALID_ARGUMENT;
  if (((uintptr_t)x_dev | (uintptr_t)payload_dev) & 15) return PKV_ERR_INVALID_ARGUMENT;
  if (int ds = pkv_check_device(p->device)) return ds;
  PkvGeom g;
  int st = pkv_make_geom(layout, p->rec_bytes, payload_batch_stride, pkv_fib_tile_vectors(p->cfg.dim, 1),
                         true, &g);
  if (st != PKV_OK) return st;
  if (g.vpb == 0) return PKV_ERR_EMPTY_BATCH;
  // the shortcut encoder implements the batch numerics only (fib-quant/src/codec.rs:586-589)
  const bool batch_numerics = p->cfg.numerics == PKV_FIB_NUMERICS_BATCH ||
                              (p->cfg.numerics == PKV_FIB_NUMERICS_AUTO && g.vpb >= 4);
  if (p->hadamard)  // that encoder keeps no list, so it allocates nothing anyway
    return pkv_launch_fib_encode(p, x_dev, g, payload_dev, err_dev, batch_numerics, (cudaStream_t)stream);
  if (!batch_numerics || !p->orthonormal) return PKV_ERR_UNSUPPORTED;
  if ((int64_t)g.n_batches * g.vpb > PKV_FIB_STATIC_MAX_VECTORS) return PKV_ERR_STATIC_SCRATCH_TOO_SMALL;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return PKV_ERR_CUDA;
  uint32_t* scratch;
  {
    // Set-up, once per device: in host code the array's name is only a handle, the address a
    // kernel can use comes from cudaGetSymbolAddress with that device current.
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_scratch_ptr[dev]) {
      void* addr = nullptr;
      if (cudaGetSymbolAddress(&addr, g_fib_static_scratch) != cudaSuccess || !addr) return PKV_ERR_CUDA;
      g_static_scratch_ptr[dev] = static_cast<uint32_t*>(addr);
    }
    scratch = g_static_scratch_ptr[dev];
  }
  return pkv_launch_fib_encode_fast_with_scratch(p, x_dev, g, payload_dev, err_dev, scratch,
                                                 (cudaStream_t)stream);
}

int pkv_fib_stats_copy(unsigned long long* out, int reset) {
  static const unsigned long long zeros[4] = {0, 0, 0, 0};
  if (out && cudaMemcpyFromSymbol(out, g_fib_stats, sizeof(zeros)) != cudaSuccess) return PKV_ERR_CUDA;
  if (reset && cudaMemcpyToSymbol(g_fib_stats, zeros, sizeof(zeros)) != cudaSuccess) return PKV_ERR_CUDA;
  return PKV_OK;
}
