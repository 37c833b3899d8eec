// turbo-quant encode: one thread per vector, one warp per tile of 32 vectors.
//  turbo-quant/src/turbo.rs:256-288, polar.rs:246-266,413-421, rotation.rs:202-221,379-398,
//  qjl.rs:203-220, radius.rs:58-77, bitpack.rs:21-62, wire.rs:350-396
//
// The per-pair and per-projection work is written as straight-line unrolled passes without
// calls or data-dependent branches, so the compiler can interleave independent pairs; the
// decisions a shortcut could not certify are collected in bit masks and settled afterwards
// by out-of-line routines that run the exact operation sequence.
//
// Shared-memory tile of the CTA's 128 vectors (4 warps x 32): the tensor cores' K-major layout with
// the 128-byte swizzle -- one slab of [128 rows][128 bytes] per 32 columns, the eight 16-byte
// pieces of a row's 128 bytes permuted by (piece ^ (row & 7)) -- so that a 128-byte line of a
// vector in global memory stays one line in shared memory (efficient staging copies) and the
// thread-per-row accesses of a quarter warp still fall in eight different bank groups.  The
// QJL sketch (32 or 64 dot products per vector) is one 128 x m x D TF32 product on the tensor
// cores (tcgen05.mma, accumulator in tensor memory); its signs are accepted where they clear the
// TF32 error bound, retaken in binary32 where they do not, and by the exact sequence at last.
#pragma once

#include "pkv_tcgen05.cuh"
#include "pkv_turbo_common.cuh"

namespace pkv_turbo {

// Counters of the certify-or-flag tiers since the last reset (pkv_stats_read): [0] pairs whose angle bucket
// went to the exact atan2f tier, [1] (vector, row) signs retaken by the binary32 dot, [2] list entries settled
// by turbo_encode_fix_kernel with the reference's own sequence.  One atomic per warp and tile at most.
static __device__ unsigned long long g_turbo_stats[4];

// Entries of the per-warp list of (vector, row) pairs awaiting the second tier (at most 64: the
// list and the 32 residual norms share the 256 bytes that held the vector offsets).
#ifndef PKV_QJL_LIST_CAP
#define PKV_QJL_LIST_CAP 64
#endif

template <int D>
struct TurboEnc {
  static constexpr int NWARPS = 4;  // one CTA = one 128-row tensor-core tile
  static constexpr int THREADS = 128, ROWS = 128, TV = 32, WS = 33, P = D / 2, LPV = D / 4;
  static constexpr int SLABS = D / 32;          // 128-byte column blocks per row
  static constexpr int X_SLAB = ROWS * 128;     // bytes per slab of the vector tile
  static constexpr int X_BYTES = SLABS * X_SLAB;
};

using pkv_tc::sw_piece;
using pkv_tc::tile_at;

// Replace angle index i in the shared angle words (LSB-first stream, bitpack.rs:135-143).
__device__ __forceinline__ void patch_angle(uint32_t* aw, int ws, int i, int pb, uint32_t idx) {
  const int pos = i * pb, wi = pos >> 5, sh = pos & 31;
  const uint32_t m = (1u << pb) - 1u;
  aw[wi * ws] = (aw[wi * ws] & ~(m << sh)) | (idx << sh);
  if (sh + pb > 32) {
    const int s2 = 32 - sh;
    aw[(wi + 1) * ws] = (aw[(wi + 1) * ws] & ~(m >> s2)) | (idx >> s2);
  }
}

// Angle index i of the shared angle words.
__device__ __forceinline__ uint32_t read_angle(const uint32_t* aw, int ws, int i, int pb) {
  const int pos = i * pb, wi = pos >> 5, sh = pos & 31;
  uint32_t idx = aw[wi * ws] >> sh;
  if (sh + pb > 32) idx |= aw[(wi + 1) * ws] << (32 - sh);
  return idx & ((1u << pb) - 1u);
}

// Exact angle buckets for the undecided pairs `unc` of ONE vector, computed by the whole warp
// (all 32 lanes call this together).  The rotated vector is rebuilt from the input row with
// D/32 elements per lane: the butterflies pair the same elements in the same order as
// fwht_normalized (in-lane for step < D/32, by lane-xor shuffles above), so every value is
// bit-identical to the owner thread's.  Lane l then holds pairs l*D/64 .. and each pending pair
// takes atan2f + the bucket expression of polar.rs:415-420; lane 0 patches the angle words.
// Returns (to every lane) whether an index differs from the one the shortcut had guessed.
template <int D>
__device__ __noinline__ bool fix_pairs_warp(const uint8_t* xt, int xrow, uint4 sign_mask, float scale,
                                            unsigned long long unc, uint32_t* aw, int ws, int pb,
                                            int lane) {
  constexpr int E = D / 32;  // elements per lane (2 or 4)
  float e[E];
#pragma unroll
  for (int k = 0; k < E; k++) {
    const int i = lane * E + k;
    const int wi = i >> 5;  // the mask travels by value: a pointer into the kernel parameters would
                            // force a per-thread copy of the whole parameter block
    const uint32_t mw = wi == 0 ? sign_mask.x : wi == 1 ? sign_mask.y : wi == 2 ? sign_mask.z : sign_mask.w;
    e[k] = __uint_as_float(__float_as_uint(*tile_at(xt, TurboEnc<D>::X_SLAB, xrow, i)) ^ (((mw >> (i & 31)) & 1u) << 31));
  }
#pragma unroll
  for (int step = 1; step < E; step <<= 1)
#pragma unroll
    for (int start = 0; start < E; start += 2 * step)
#pragma unroll
      for (int o = 0; o < step; o++) {
        const float a = e[start + o], b = e[start + o + step];
        e[start + o] = __fadd_rn(a, b);
        e[start + o + step] = __fsub_rn(a, b);
      }
#pragma unroll
  for (int step = E; step < D; step <<= 1) {
    const int lm = step / E;
    const bool upper = (lane & lm) != 0;
#pragma unroll
    for (int k = 0; k < E; k++) {
      const float p = __shfl_xor_sync(0xffffffffu, e[k], lm);
      e[k] = upper ? __fsub_rn(p, e[k]) : __fadd_rn(e[k], p);  // (a, b) -> (a + b, a - b)
    }
  }
  uint32_t mine[E / 2];
#pragma unroll
  for (int j = 0; j < E / 2; j++) {
    const int i = lane * (E / 2) + j;
    mine[j] = 0;
    if ((unc >> i) & 1ull)
      mine[j] = exact_bucket(__fmul_rn(e[2 * j + 1], scale), __fmul_rn(e[2 * j], scale), 1u << pb);
  }
  bool changed = false;
  while (unc) {
    const int i = __ffsll((long long)unc) - 1;
    unc &= unc - 1;
    uint32_t val = 0;
#pragma unroll
    for (int j = 0; j < E / 2; j++) {
      const uint32_t t = __shfl_sync(0xffffffffu, mine[j], i / (E / 2));
      if (j == i % (E / 2)) val = t;
    }
    if (lane == 0) {
      changed = changed || read_angle(aw, ws, i, pb) != val;
      patch_angle(aw, ws, i, pb, val);
    }
  }
  __syncwarp();
  return __shfl_sync(0xffffffffu, (int)changed, 0) != 0;
}

// Which of the two encode errors applies when some radius came out non-finite: a non-finite
// input value (turbo.rs:263, checked first by the reference) or an overflow in the butterflies
// (PolarCode::from_parts, polar.rs:127-133).
// The exact logarithm of the BlockLogU8 coder, kept out of line: four call sites, two of them rare.
// (with a table of the host libm's deviations: that libm's logf, bit for bit)
#define PKV_LOGF_TABLE_ARGS tp.logf_table.keys, tp.logf_table.dirs, tp.logf_table.bloom, tp.logf_table.n, tp.logf_table.bloom_log2
__device__ __noinline__ float exact_logf(float r, const uint32_t* keys, const uint32_t* dirs, const uint32_t* bloom,
                                         uint32_t n, uint32_t bloom_log2) {
  const float l = pkv_logf_portable(r);
  return keys == nullptr ? l : pkv_ulp_lookup(keys, dirs, bloom, n, bloom_log2, r, l);
}

__device__ __noinline__ int classify_bad_vector(const uint8_t* xt, int slab, int row, int dim) {
  for (int i = 0; i < dim; i++)
    if (!pkv_finite(*tile_at(xt, slab, row, i))) return PKV_VEC_NONFINITE_INPUT;
  return PKV_VEC_BAD_RADIUS;
}

// Dot of QJL row p with the residual in tile row `row`: binary32 fused in four chains (the second
// tier of the sign shortcut) and the reference's sequence (qjl.rs:214-217).
__device__ __noinline__ float fused_dot(const uint8_t* gt, int g_slab, int p, const uint8_t* xt, int x_slab,
                                        int row, int dim) {
  float d0 = 0.0f, d1 = 0.0f, d2 = 0.0f, d3 = 0.0f;
  for (int c = 0; c < dim / 4; c++) {
    const float4 g = *reinterpret_cast<const float4*>(gt + sw_piece(g_slab, p, c));
    const float4 x = *reinterpret_cast<const float4*>(xt + sw_piece(x_slab, row, c));
    d0 = fmaf(g.x, x.x, d0);
    d1 = fmaf(g.y, x.y, d1);
    d2 = fmaf(g.z, x.z, d2);
    d3 = fmaf(g.w, x.w, d3);
  }
  return (d0 + d1) + (d2 + d3);
}
__device__ __noinline__ float sequential_dot(const uint8_t* gt, int g_slab, int p, const uint8_t* xt,
                                             int x_slab, int row, int dim) {
  float dot = 0.0f;
  for (int c = 0; c < dim / 4; c++) {
    const float4 g = *reinterpret_cast<const float4*>(gt + sw_piece(g_slab, p, c));
    const float4 x = *reinterpret_cast<const float4*>(xt + sw_piece(x_slab, row, c));
    dot = __fadd_rn(dot, __fmul_rn(g.x, x.x));
    dot = __fadd_rn(dot, __fmul_rn(g.y, x.y));
    dot = __fadd_rn(dot, __fmul_rn(g.z, x.z));
    dot = __fadd_rn(dot, __fmul_rn(g.w, x.w));
  }
  return dot;
}

// The reference's own sequence for one vector, by one warp (all 32 lanes call this together), used by
// the rotated-domain sketch for what its shortcuts leave open: forward rotation and radii recomputed
// from the input row (bit-identical to the encoder thread's), polar.decode with the final angle indices
// read from the finished record (polar.rs:272-278,306-316), FastHadamardRotation::apply_inverse
// (rotation.rs:212-221), residual (turbo.rs:268-273) and QjlQuantizer::sketch's sequential dots
// (qjl.rs:214-217), lane t taking row c0 + t of the matrix `g` ([m][D], shared memory).  Lane t holds
// coordinates t E .. t E + E - 1 (E = D/32); the residual passes through `scratch` (D floats, shared).
// Returns the 32 sign bits; *bad is set for a residual that is not finite (qjl.rs:210).  A zero input
// has a zero residual: every dot is +0, every bit 1.
template <int D>
__device__ __forceinline__ uint32_t exact_signs_warp(const float* __restrict__ xrow, const uint32_t* aw, int pb,
                                                     uint4 sign_mask, float scale, const float* s_lut,
                                                     const float* g, int c0, float* scratch, int lane, int* bad) {
  constexpr int E = D / 32;
  float xv[E], e[E];
  bool zero_x = true;
#pragma unroll
  for (int k = 0; k < E; k++) {
    const int i = lane * E + k;
    const uint32_t mw = (i >> 5) == 0 ? sign_mask.x : (i >> 5) == 1 ? sign_mask.y : (i >> 5) == 2 ? sign_mask.z : sign_mask.w;
    xv[k] = __ldg(xrow + i);
    zero_x = zero_x && (__float_as_uint(xv[k]) & 0x7fffffffu) == 0u;
    e[k] = __uint_as_float(__float_as_uint(xv[k]) ^ (((mw >> (i & 31)) & 1u) << 31));
  }
  if (__all_sync(0xffffffffu, zero_x)) return 0xffffffffu;
  auto butterflies = [&]() {
#pragma unroll
    for (int step = 1; step < E; step <<= 1)
#pragma unroll
      for (int start = 0; start < E; start += 2 * step)
#pragma unroll
        for (int o = 0; o < step; o++) {
          const float a = e[start + o], b = e[start + o + step];
          e[start + o] = __fadd_rn(a, b);
          e[start + o + step] = __fsub_rn(a, b);
        }
#pragma unroll
    for (int step = E; step < D; step <<= 1) {
      const int lm = step / E;
      const bool upper = (lane & lm) != 0;
#pragma unroll
      for (int k = 0; k < E; k++) {
        const float p = __shfl_xor_sync(0xffffffffu, e[k], lm);
        e[k] = upper ? __fsub_rn(p, e[k]) : __fadd_rn(e[k], p);
      }
    }
  };
  butterflies();
#pragma unroll
  for (int j = 0; j < E / 2; j++) {  // encode_pair's radius, then the de-quantised pair
    const float a = __fmul_rn(e[2 * j], scale), b = __fmul_rn(e[2 * j + 1], scale);
    const float r = __fsqrt_rn(__fadd_rn(__fmul_rn(a, a), __fmul_rn(b, b)));
    const uint32_t idx = read_angle(aw, 1, lane * (E / 2) + j, pb);
    e[2 * j] = __fmul_rn(r, s_lut[2 * idx]);
    e[2 * j + 1] = __fmul_rn(r, s_lut[2 * idx + 1]);
  }
  butterflies();
  bool finite_res = true;
#pragma unroll
  for (int k = 0; k < E; k++) {
    const int i = lane * E + k;
    const uint32_t mw = (i >> 5) == 0 ? sign_mask.x : (i >> 5) == 1 ? sign_mask.y : (i >> 5) == 2 ? sign_mask.z : sign_mask.w;
    const float z = __fmul_rn(e[k], scale);
    const float rec = __uint_as_float(__float_as_uint(z) ^ (((mw >> (i & 31)) & 1u) << 31));
    const float res = __fsub_rn(xv[k], rec);
    finite_res = finite_res && pkv_finite(res);
    scratch[i] = res;
  }
  if (!__all_sync(0xffffffffu, finite_res)) *bad = PKV_VEC_NONFINITE_RESIDUAL;
  __syncwarp();
  // row c0 + lane of g, read with a rotation so that the 32 lanes hit 32 different banks
  const float* gr = g + (size_t)(c0 + lane) * (D + 1);
  float dot = 0.0f;
#pragma unroll 8
  for (int j = 0; j < D; j++) dot = __fadd_rn(dot, __fmul_rn(gr[j], scratch[j]));
  const uint32_t word = __ballot_sync(0xffffffffu, dot >= 0.0f);
  __syncwarp();
  return word;
}

// Second kernel of the rotated-domain sketch: the exact sequence for the (vector, block of 32
// projections) entries the encoder listed, one warp per entry, patching the sign bits named by the
// entry's mask in the finished record.  Entry: x = global vector index | block << 31, y = mask.
template <int D>
__global__ void __launch_bounds__(128)
turbo_encode_fix_kernel(PkvGeom g, TurboParams tp, const float* __restrict__ x, uint8_t* __restrict__ payload,
                        uint64_t* err, const uint32_t* __restrict__ count, const uint2* __restrict__ list) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int m = tp.projections;
  float* s_g = reinterpret_cast<float*>(smem);   // [m][D + 1]
  float* s_lut = s_g + m * (D + 1);              // (cos, sin)[levels]
  float* s_scr = s_lut + 2 * (1 << tp.polar_bits);  // [4][D]
  const uint32_t n = *count;
  if (blockIdx.x == 0 && threadIdx.x == 0 && n) atomicAdd(&g_turbo_stats[2], (unsigned long long)n);
  if ((uint32_t)blockIdx.x * 4u >= n) return;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int levels = 1 << tp.polar_bits;
  for (int i = threadIdx.x; i < m * D; i += 128) s_g[(i / D) * (D + 1) + (i % D)] = __ldg(tp.qjl + i);
  for (int i = threadIdx.x; i < levels; i += 128) {
    s_lut[2 * i] = __ldg(tp.lut + i);
    s_lut[2 * i + 1] = __ldg(tp.lut + levels + i);
  }
  __syncthreads();
  const uint4 smask = make_uint4(tp.sign_mask[0], tp.sign_mask[1], tp.sign_mask[2], tp.sign_mask[3]);
  const int sign_off = 4 * (D / 2) + 4 * tp.angle_words;
  for (uint32_t it = blockIdx.x * 4u + warp; it < n; it += gridDim.x * 4u) {
    const uint2 e = list[it];
    const int64_t gvec = (int64_t)(e.x & 0x7fffffffu);
    const int c0 = (int)(e.x >> 31) * 32;
    const int batch = (int)(gvec / g.vpb), v = (int)(gvec % g.vpb);
    uint8_t* rec = payload + (int64_t)batch * g.payload_batch_stride + (int64_t)v * g.rec_bytes;
    int bad = 0;
    const uint32_t word = exact_signs_warp<D>(x + pkv_vec_offset(g.L, batch, v),
                                              reinterpret_cast<const uint32_t*>(rec + 4 * (D / 2)), tp.polar_bits, smask,
                                              tp.scale, s_lut, s_g, c0, s_scr + warp * D, lane, &bad);
    if (lane == 0) {
      uint32_t* sw = reinterpret_cast<uint32_t*>(rec + sign_off) + (c0 >> 5);
      *sw = (*sw & ~e.y) | (word & e.y);
      if (bad) pkv_report(err, 0, gvec, bad);
    }
  }
}

template <int D>
struct TurboEncSmem {
  using K = TurboEnc<D>;
  // CTA-wide: vector tile, QJL matrix tile, cos/sin + ray tables; then one slice per warp
  static __host__ __device__ size_t table_bytes(int projections, int levels, int ray_count) {
    // 1024: the swizzled tiles start on a 1024-byte boundary found at run time
    const size_t n = 1024 + (size_t)K::X_BYTES + (size_t)K::SLABS * projections * 128 +
                     sizeof(float) * (2 * levels + 2 * ray_count + projections);
    return (n + 15) & ~(size_t)15;
  }
  static __host__ __device__ size_t warp_bytes(int tile_words, int lossy) {
    const size_t n = sizeof(int64_t) * K::TV + sizeof(uint32_t) * tile_words * K::WS;
    (void)lossy;
    return (n + 15) & ~(size_t)15;
  }
};

// f32 radii never pass through shared memory: they stay in the registers of their pairs and are
// stored by their thread into its own record; only the few angle / sign words sit in a small
// shared tile so that the cooperative fix-up can patch them.  DIRECT (record a multiple of 16
// bytes, angle + sign words a multiple of 4) stores 16-byte pieces, the other f32-radii shapes
// one word at a time (their records are only 4-byte aligned).  BlockLogU8 records are assembled
// whole in a word-transposed tile and written out by the warp.
//
// ROT (PolarWithQjl with f32 radii): the QJL sketch is taken in the rotated domain.  The reference
// signs g . res with res = x - rec, rec = S H~ p (p the de-quantised pairs, H~ = scale * H, S the signs).
// With y the rotated vector this is (g S H~) . (y - p) up to a modelling error bounded below, so the
// thread forms q = y - p pair by pair as it quantises, and the sketch is one TF32 product of the q
// tile with G'' = G S H~ (rows scaled to unit length, prepared on the host in binary64): no inverse
// butterflies and no residual in the common case.  A sign is accepted when |dot| clears the tier's
// bound; the rest are retaken in binary32 (fused dot of q with G''), and what is still open, or
// belongs to a vector the model does not cover (an index corrected after q was formed, radii beyond
// 1e30, norms lost to underflow), is listed for turbo_encode_fix_kernel, which runs the reference's own
// sequence for those vectors after this kernel (global vector indices below 2^31 fit the entries).
// Error of the model relative to |g|:  |G'' . q - g . res| / |g| <=
//   eta |y| + c_f (|x| + |p|) + u (|p| + |q|) + 2 u |q|,
// eta = |d scale^2 - 1| <= 4 u (scale = fl(1 / fl(sqrt d)); zero for d = 64), c_f = (log2 d + 1) u the
// 2-norm error of a rounded transform, u = 2^-24; the u terms are the roundings of r cos / r sin, of q,
// of G'' and of res.  With |p|, |x| <= |y| (1 + 1e-6) that is below 21 u |y| + 3 u |q| for d <= 128;
// the kernel adds PKV_QJL_MODEL_BOUND times an upper bound of |y| to both tiers' bounds.
// d = 64: eta = 0, c_f = 6 u (the scale 1/8 is exact): 13 u |y| = 7.8e-7 |y|;  d = 128: 21 u |y| = 1.25e-6 |y|.
// The second tier's bound is the rounding of the reference's sequential dot, (d + 1) u |g| |res|, plus
// the 3 u |q| above, plus the rounding of the tier's own dot: binary32, fused, four chains of d / 4 terms
// and two levels of additions, at most gamma_(d/4+2) sum |g_j q_j| <= (d / 4 + 3) u |q| (unit rows).
// A binary64 dot here (no rounding of its own) settled 0.02 % more vectors but cost two conversions
// per term on the quarter-rate conversion pipe: a fifth of the kernel's time.
#define PKV_QJL_MODEL_BOUND(D) ((D) == 64 ? 9.0e-7f : 1.45e-6f)
#define PKV_QJL_SEQ_BOUND(D) ((float)((D) + 4 + (D) / 4 + 3) * 5.9604645e-8f * 1.05f)
template <int D, int PB, bool DIRECT, bool ROT>
__global__ void __launch_bounds__(TurboEnc<D>::THREADS, D == 64 ? (DIRECT ? 4 : 3) : 2)
turbo_encode_kernel(PkvGeom g, TurboParams tp, const float* __restrict__ x,
                    uint8_t* __restrict__ payload, uint64_t* err, uint32_t* fix_count, uint2* fix_list) {
  using K = TurboEnc<D>;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t s_bar;  // completion of the tensor-core product
  __shared__ uint32_t s_tmem;              // base of the CTA's tensor-memory columns
  const int pb = PB ? PB : tp.polar_bits;
  const int levels = 1 << pb;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int m = tp.projections;  // 0 without the QJL stage
  const int g_slab = m * 128;
  uint8_t* s_xt = smem + ((1024u - (pkv_tc::smem_u32(smem) & 1023u)) & 1023u);  // vector tile, SLABS x [128 rows][128 B]
  uint8_t* s_gt = s_xt + K::X_BYTES;                                           // QJL matrix, SLABS x [m rows][128 B]
  float* s_lut = reinterpret_cast<float*>(s_gt + K::SLABS * g_slab);           // (cos, sin)[L], ray_cos, ray_sin
  const int lut_len = 2 * levels + 2 * tp.ray_count;
  float* s_thr = s_lut + lut_len;  // [m] binary32-tier thresholds of the sign shortcut
  const float* s_ray_cos = s_lut + 2 * levels;
  const float* s_ray_sin = s_ray_cos + tp.ray_count;
  // f32 radii never pass through shared memory (16-byte stores in the DIRECT kernel, 4-byte stores
  // otherwise); BlockLogU8 records are assembled whole in the tile
  const bool lossy = !DIRECT && !ROT && tp.lossy;
  const int rw = lossy ? tp.radii_words : 0;  // radii words present in the shared tile
  const int tile_words = lossy ? tp.rec_words : tp.angle_words + tp.sign_words;
  uint8_t* wbase = smem + TurboEncSmem<D>::table_bytes(m, levels, tp.ray_count) +
                   warp * TurboEncSmem<D>::warp_bytes(tile_words, tp.lossy);
  int64_t* s_off = reinterpret_cast<int64_t*>(wbase);                  // [TV]
  uint32_t* s_w = reinterpret_cast<uint32_t*>(s_off + K::TV);          // [tile_words][WS]

  const int64_t tile_id = (int64_t)blockIdx.x * K::NWARPS + warp;
  const bool active = tile_id < (int64_t)g.n_batches * g.tiles_per_batch;
  const int tile = active ? (int)(tile_id % g.tiles_per_batch) : 0;
  const int batch = active ? (int)(tile_id / g.tiles_per_batch) : 0;
  const int v0 = tile * K::TV;
  const int nv = active ? min(K::TV, g.vpb - v0) : 0;
  const int v = lane;
  const int row = warp * K::TV + v;  // this thread's row of the CTA tile
  const uint32_t tmem_cols = m > 32 ? 64u : 32u;

  if (m) {
    if (warp == 0) pkv_tc::tmem_alloc(&s_tmem, tmem_cols);
    if (threadIdx.x == 32) pkv_tc::mbar_init(&s_bar, 1);
  } else if (warp == 0) {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }

  // the warp's 32 vectors: 16 lanes x 16 bytes per vector, all copies in flight at once
  if (v < nv) s_off[v] = pkv_vec_offset(g.L, batch, v0 + v);
  __syncwarp();
#pragma unroll 4
  for (int i = lane; i < nv * K::LPV; i += 32) {
    const int vv = i / K::LPV, q = i % K::LPV;
    pkv_cp_async16(s_xt + sw_piece(K::X_SLAB, warp * K::TV + vv, q),
                   reinterpret_cast<const float4*>(x + s_off[vv]) + q);
  }
  for (int i = threadIdx.x; i < m * K::LPV; i += K::THREADS)
    pkv_cp_async16(s_gt + sw_piece(g_slab, i / K::LPV, i % K::LPV),
                   reinterpret_cast<const float4*>(ROT ? tp.qjl_rot : tp.qjl) + i);
  for (int i = threadIdx.x; i < m; i += K::THREADS) pkv_cp_async4(s_thr + i, tp.qjl + m * D + i);
  for (int i = threadIdx.x; i < lut_len; i += K::THREADS)  // cos / sin interleaved: one 8-byte read per pair
    pkv_cp_async4(s_lut + (i < levels ? 2 * i : i < 2 * levels ? 2 * (i - levels) + 1 : i), tp.lut + i);
  pkv_cp_async_wait_all();
  if (m) pkv_tc::fence_before_sync();
  __syncthreads();  // tables, barrier, tensor-memory base; the warp's own rows only need warp-level ordering until the product
  if (m) pkv_tc::fence_after_sync();

  // Every lane runs the per-vector code (lanes beyond nv work on their unused tile rows and
  // never report or get copied out), so the warp stays converged for the cooperative steps.
  const bool valid = v < nv;
  // piece c of this thread's vector sits at s_xt + (c >> 3) * X_SLAB + (xsw ^ ((c & 7) << 4))
  const uint32_t xsw = (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((row & 7) << 4));
  uint32_t* w = s_w + v;
  uint32_t* aw = w + rw * K::WS;
  uint8_t* my_rec = payload + (int64_t)batch * g.payload_batch_stride + (int64_t)(v0 + v) * g.rec_bytes;
  int code = 0;
  float y[D];
#pragma unroll
  for (int i = 0; i < D; i += 4) {
    const float4 t = *reinterpret_cast<const float4*>(s_xt + (i >> 5) * K::X_SLAB + (xsw ^ (((i >> 2) & 7) << 4)));
    y[i] = t.x; y[i + 1] = t.y; y[i + 2] = t.z; y[i + 3] = t.w;
  }
  // FastHadamardRotation::apply, rotation.rs:202-210.  A non-finite input makes every output of
  // the transform non-finite, so input finiteness is only looked at when a radius is bad.
  fwht_forward_signed<D>(y, tp.sgn, tp.scale);

  // Pass 1, encode_pair (polar.rs:413-421): radius exactly, bucket by the shortcut.  Radii stay in
  // the registers of their pairs; undecided pairs are noted in `unc`.
  constexpr int NW = PB ? K::P * PB / 32 : 1;
  unsigned long long unc = 0;
  [[maybe_unused]] float ysq = 0.0f;   // ROT: |y|^2 from the squared radii
  [[maybe_unused]] bool force = false;  // ROT: every sign of this vector comes from the exact sequence
  {
    uint32_t words[NW];
#pragma unroll
    for (int k = 0; k < NW; k++) words[k] = 0;
    uint64_t bitbuf = 0;
    int nbits = 0, wk = 0;
    uint32_t rmax = 0;  // radii are >= +0 or NaN: the largest bit pattern tells if any is not finite
    [[maybe_unused]] float rq[4];
#pragma unroll
    for (int i = 0; i < K::P; i++) {
      const float a = y[2 * i], b = y[2 * i + 1];
      float aa = a, bb = b;
      mul2(aa, bb, a, b);  // (a * a, b * b), each rounded on its own
      const float r2 = __fadd_rn(aa, bb);
      const float r = __fsqrt_rn(r2);
      int certain = 0;
      uint32_t idx = 0;
      if (tp.fast_bucket) idx = pkv_fast_bucket_any(a, b, pb, s_ray_cos, s_ray_sin, &certain);
      unc |= (unsigned long long)(certain ? 0u : 1u) << i;
      rmax = max(rmax, __float_as_uint(r));  // a square root is +x or NaN (either sign): unsigned order works
      if constexpr (ROT) {
        // the radius leaves for the record at once; the pair's registers take q = (a, b) - r (cos, sin)
        // of the guessed bucket (a vector whose guess is corrected later takes the exact sequence)
        ysq = __fadd_rn(ysq, r2);
        const float2 cs = *reinterpret_cast<const float2*>(s_lut + 2 * idx);
        y[2 * i] = __fmaf_rn(-r, cs.x, a);
        y[2 * i + 1] = __fmaf_rn(-r, cs.y, b);
        if constexpr (DIRECT) {
          rq[i & 3] = r;
          if ((i & 3) == 3 && valid) reinterpret_cast<float4*>(my_rec)[i >> 2] = make_float4(rq[0], rq[1], rq[2], rq[3]);
        } else {
          if (valid) reinterpret_cast<float*>(my_rec)[i] = r;
        }
      } else {
        y[2 * i] = r;  // a and b are spent: the pair's first register keeps r
      }
      if constexpr (PB != 0) {
        const int pos = i * PB, wi = pos >> 5, sh = pos & 31;
        words[wi] |= idx << sh;
        if (sh + PB > 32) words[wi + 1] |= idx >> (32 - sh);
      } else {
        bitbuf |= (uint64_t)idx << nbits;
        nbits += pb;
        if (nbits >= 32) {
          aw[wk * K::WS] = (uint32_t)bitbuf;
          wk++;
          bitbuf >>= 32;
          nbits -= 32;
        }
      }
    }
    if constexpr (PB != 0) {
#pragma unroll
      for (int k = 0; k < NW; k++) aw[k * K::WS] = words[k];
    } else if (nbits > 0) {
      aw[wk * K::WS] = (uint32_t)bitbuf;
    }
    if (rmax >= 0x7f800000u) code = classify_bad_vector(s_xt, K::X_SLAB, row, D);
    if constexpr (ROT) force = rmax >= 0x7149f2cau;  // radii beyond 1e30: the residual might overflow
  }
  if (!valid) unc = 0;
  {
    const unsigned n_unc = __reduce_add_sync(0xffffffffu, (unsigned)__popcll(unc));
    if (lane == 0 && n_unc) atomicAdd(&g_turbo_stats[0], (unsigned long long)n_unc);
  }
  for (unsigned pending = __ballot_sync(0xffffffffu, unc != 0); pending; pending &= pending - 1) {
    const int src = __ffs(pending) - 1;  // settle lane src's undecided pairs, all lanes helping
    const unsigned long long um =
        ((unsigned long long)__shfl_sync(0xffffffffu, (uint32_t)(unc >> 32), src) << 32) |
        __shfl_sync(0xffffffffu, (uint32_t)unc, src);
    const bool changed = fix_pairs_warp<D>(
        s_xt, warp * K::TV + src, make_uint4(tp.sign_mask[0], tp.sign_mask[1], tp.sign_mask[2], tp.sign_mask[3]),
        tp.scale, um, s_w + src + rw * K::WS, K::WS, pb, lane);
    if constexpr (ROT) force = force || (changed && lane == src);
  }
  if constexpr (ROT) {
    // radii already stored
  } else if constexpr (DIRECT) {
    if (valid) {
#pragma unroll
      for (int k = 0; k < K::P / 4; k++)
        reinterpret_cast<float4*>(my_rec)[k] = make_float4(y[8 * k], y[8 * k + 2], y[8 * k + 4], y[8 * k + 6]);
    }
  } else if (!lossy && valid) {  // records that are only 4-byte aligned: one word per store
#pragma unroll
    for (int i = 0; i < K::P; i++) reinterpret_cast<float*>(my_rec)[i] = y[2 * i];
  }
  if constexpr (!DIRECT && !ROT)  // direct stores and the rotated-domain sketch imply f32 radii
  if (tp.lossy) {
    // CompressedRadiiV1::compress, BlockLogU8 (radius.rs:58-77), min/max after the bytes (wire.rs:368-371),
    // straight from the radii in the registers (y[2i]; the reconstruction below still uses them).
    // The logarithm is monotone, so min / max of the logs are the logs of the smallest / largest
    // radius: two exact logarithms per vector (radii within 4e-5 of an extreme are taken exactly
    // too, in case the rounded logarithm is not monotone to the last bit there).  The 8-bit codes
    // come from the fast logarithm where that provably gives the reference's code
    // (pkv_fast_radius_code); the rare others are redone with the exact one from a copy of the
    // radii in local memory.
    float rmin = __int_as_float(0x7f800000), rmax = 0.0f;
#pragma unroll
    for (int i = 0; i < K::P; i++) {
      const float r = (code || !(y[2 * i] > PKV_FLT_MIN)) ? PKV_FLT_MIN : y[2 * i];
      rmin = fminf(rmin, r);
      rmax = fmaxf(rmax, r);
    }
    float mn = exact_logf(rmin, PKV_LOGF_TABLE_ARGS), mx = exact_logf(rmax, PKV_LOGF_TABLE_ARGS);
    const float near_min = __fmul_rn(rmin, 1.00004f), near_max = __fmul_rn(rmax, 0.99996f);
    bool ties = false;
#pragma unroll
    for (int i = 0; i < K::P; i++) {
      const float r = (code || !(y[2 * i] > PKV_FLT_MIN)) ? PKV_FLT_MIN : y[2 * i];
      ties = ties || (r != rmin && r <= near_min) || (r != rmax && r >= near_max);
    }
    float rl[K::P];  // local-memory copy, touched only on the rare paths
    if (ties) {
#pragma unroll
      for (int i = 0; i < K::P; i++) rl[i] = (code || !(y[2 * i] > PKV_FLT_MIN)) ? PKV_FLT_MIN : y[2 * i];
#pragma unroll 1
      for (int i = 0; i < K::P; i++) {
        const float r = rl[i];
        if (r <= near_min) mn = fminf(mn, exact_logf(r, PKV_LOGF_TABLE_ARGS));
        if (r >= near_max) mx = fmaxf(mx, exact_logf(r, PKV_LOGF_TABLE_ARGS));
      }
    }
    float span = __fsub_rn(mx, mn);
    if (!(span > PKV_FLT_EPS)) span = PKV_FLT_EPS;
    const float k = __fdiv_rn(255.0f, span);
    unsigned long long unsure = 0;
#pragma unroll
    for (int q = 0; q < K::P / 4; q++) {
      uint32_t q4 = 0;
#pragma unroll
      for (int b = 0; b < 4; b++) {
        const int i = 4 * q + b;
        const float r = (code || !(y[2 * i] > PKV_FLT_MIN)) ? PKV_FLT_MIN : y[2 * i];
        int certain;
        q4 |= pkv_fast_radius_code(__logf(r), mn, k, &certain) << (8 * b);
        unsure |= (unsigned long long)(certain ? 0u : 1u) << i;
      }
      w[q * K::WS] = q4;
    }
    if (unsure) {
#pragma unroll
      for (int i = 0; i < K::P; i++) rl[i] = (code || !(y[2 * i] > PKV_FLT_MIN)) ? PKV_FLT_MIN : y[2 * i];
      while (unsure) {
        const int i = __ffsll((long long)unsure) - 1;
        unsure &= unsure - 1;
        float nrm = __fdiv_rn(__fsub_rn(exact_logf(rl[i], PKV_LOGF_TABLE_ARGS), mn), span);
        nrm = nrm < 0.0f ? 0.0f : (nrm > 1.0f ? 1.0f : nrm);
        const uint32_t c8 = (uint32_t)roundf(__fmul_rn(nrm, 255.0f)) & 0xffu;
        const int sh = 8 * (i & 3);
        w[(i >> 2) * K::WS] = (w[(i >> 2) * K::WS] & ~(0xffu << sh)) | (c8 << sh);
      }
    }
    w[(K::P / 4) * K::WS] = __float_as_uint(mn);
    w[(K::P / 4 + 1) * K::WS] = __float_as_uint(mx);
  }

  if constexpr (ROT) {
   if (tp.mode == PKV_TURBO_POLAR_WITH_QJL) {
    // q replaces x in the tile: it is the A operand of the sketch
    float2 n2 = make_float2(0.0f, 0.0f);
#pragma unroll
    for (int i = 0; i < D; i += 4) {
      n2 = ffma2(make_float2(y[i], y[i + 1]), make_float2(y[i], y[i + 1]), n2);
      n2 = ffma2(make_float2(y[i + 2], y[i + 3]), make_float2(y[i + 2], y[i + 3]), n2);
      *reinterpret_cast<float4*>(s_xt + (i >> 5) * K::X_SLAB + (xsw ^ (((i >> 2) & 7) << 4))) =
          make_float4(y[i], y[i + 1], y[i + 2], y[i + 3]);
    }
    // upper bounds of |q| and |y|; sums under 1e-30 have lost squares to underflow and bound nothing
    // (this also catches the all-zero vector): such vectors take the exact sequence
    const float nsq = n2.x + n2.y;
    if (!(nsq >= 1.0e-30f) || !(ysq >= 1.0e-30f)) force = true;
    const float nq = __fmul_rn(__fsqrt_rn(nsq), 1.0001f);
    const float model = __fmul_rn(PKV_QJL_MODEL_BOUND(D), __fmul_rn(__fsqrt_rn(ysq), 1.0001f));
    const float tau1 = fmaf(PKV_QJL_TF32_BOUND, nq, model) + PKV_QJL_ABS_BOUND;
    const float tau2 = fmaf(PKV_QJL_SEQ_BOUND(D), nq, model) + PKV_QJL_ABS_BOUND;

    pkv_tc::fence_smem_to_async();
    __syncthreads();
    const uint32_t tmem_d = s_tmem;
    if (threadIdx.x == 0 && !tp.skip_issue) {
      pkv_tc::fence_after_sync();
      const uint32_t idesc = pkv_tc::idesc_tf32(K::ROWS, m > 32 ? 64 : 32);
      const uint32_t a0 = pkv_tc::smem_u32(s_xt), b0 = pkv_tc::smem_u32(s_gt);
      pkv_tc::mma_tf32_chain<D / 8>(tmem_d, a0, K::X_SLAB, b0, (uint32_t)g_slab, idesc, false);
      pkv_tc::mma_commit(&s_bar);
    }
    const bool done =
        __all_sync(0xffffffffu, pkv_tc::mbar_wait(&s_bar, 0, tp.skip_issue ? 256 : pkv_tc::kWaitPolls));
    pkv_tc::fence_after_sync();
    uint32_t* sw = w + (rw + tp.angle_words) * K::WS;
    float* s_bound = reinterpret_cast<float*>(s_off);                      // [32] (the offsets are spent)
    uint16_t* s_items = reinterpret_cast<uint16_t*>(s_bound + K::TV);      // [PKV_QJL_LIST_CAP]
    const bool settle = valid && !code;  // this vector's signs matter
    if (done) {
#pragma unroll
      for (int c = 0; c < 64; c += 32) {
        if (c >= m) break;
        float dots[32];
        pkv_tc::tmem_load32(tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)c, dots);
        uint32_t bits = 0, flagged = 0;
#pragma unroll
        for (int p = 0; p < 32; p++) {  // rows of G'' have unit length: one bound for all of them
          flagged |= (fabsf(dots[p]) > tau1 ? 0u : 1u) << p;
          bits |= (dots[p] >= 0.0f ? 1u : 0u) << p;
        }
        if (!settle || force) flagged = 0;
        // Second tier (binary32 fused dot) for the flagged (vector, row) pairs of the whole warp, spread over the lanes
        // through a prefix-summed list; pairs beyond the list's capacity are taken by their owner.
        // What this tier leaves open is noted in `open`.
        uint32_t open = 0;
        const uint32_t cnt = __popc(flagged);
        uint32_t incl = cnt;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
          if (lane >= d) incl += t;
        }
        const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
        if (total) {
          if (lane == 0) atomicAdd(&g_turbo_stats[1], (unsigned long long)total);
          constexpr uint32_t CAP = PKV_QJL_LIST_CAP;
          s_bound[v] = tau2;
          uint32_t pos = incl - cnt;
          for (uint32_t f = flagged; f; f &= f - 1, pos++)
            if (pos < CAP) s_items[pos] = (uint16_t)((v << 5) | (__ffs(f) - 1));
          __syncwarp();
          const uint32_t n_list = min(total, CAP);
          for (uint32_t e = lane; e < n_list; e += 32) {
            const uint32_t it = s_items[e];
            const float dot = fused_dot(s_gt, g_slab, c + (int)(it & 31u), s_xt, K::X_SLAB,
                                        warp * K::TV + (int)(it >> 5), D);
            const uint32_t res = !(fabsf(dot) > s_bound[it >> 5]) ? 0x4000u : (dot >= 0.0f ? 0x8000u : 0u);
            s_items[e] = (uint16_t)(it | res);
          }
          __syncwarp();
          pos = incl - cnt;
          for (uint32_t f = flagged; f; f &= f - 1, pos++) {
            const int p = __ffs(f) - 1;
            uint32_t res;
            if (pos < CAP) {
              res = s_items[pos];
            } else {
              const float dot = fused_dot(s_gt, g_slab, c + p, s_xt, K::X_SLAB, row, D);
              res = !(fabsf(dot) > tau2) ? 0x4000u : (dot >= 0.0f ? 0x8000u : 0u);
            }
            if (res & 0x4000u) open |= 1u << p;
            else bits = (res & 0x8000u) ? (bits | (1u << p)) : (bits & ~(1u << p));
          }
          __syncwarp();
        }
        // What is still open goes on the list of turbo_encode_fix_kernel, which runs the reference's
        // own sequence for the vector and patches these bits of the record.
        if (settle && (force || open != 0)) {
          const uint32_t gvec = (uint32_t)((int64_t)batch * g.vpb + v0 + v);
          fix_list[atomicAdd(fix_count, 1u)] = make_uint2(gvec | ((uint32_t)(c >> 5) << 31), force ? 0xffffffffu : open);
        }
        sw[(c >> 5) * K::WS] = bits;
      }
    } else if (threadIdx.x == 0) {
      pkv_report(err, 0, 0, PKV_VEC_DEVICE_WAIT);
    }
   }
  } else if (tp.mode == PKV_TURBO_POLAR_WITH_QJL) {
    // polar.decode (polar.rs:272-278,306-316): de-quantised pairs from the final indices
    {
      const uint32_t mask = (uint32_t)levels - 1u;
      uint32_t words[NW];
      uint64_t bitbuf = 0;
      int nbits = 0, wk = 0;
      if constexpr (PB != 0) {
#pragma unroll
        for (int k = 0; k < NW; k++) words[k] = aw[k * K::WS];
      }
#pragma unroll
      for (int i = 0; i < K::P; i++) {
        uint32_t idx;
        if constexpr (PB != 0) {
          const int pos = i * PB, wi = pos >> 5, sh = pos & 31;
          idx = words[wi] >> sh;
          if (sh + PB > 32) idx |= words[wi + 1] << (32 - sh);
          idx &= mask;
        } else {
          if (nbits < pb) {
            bitbuf |= (uint64_t)aw[wk * K::WS] << nbits;
            wk++;
            nbits += 32;
          }
          idx = (uint32_t)bitbuf & mask;
          bitbuf >>= pb;
          nbits -= pb;
        }
        const float r = y[2 * i];
        const float2 cs = *reinterpret_cast<const float2*>(s_lut + 2 * idx);
        y[2 * i] = cs.x;
        y[2 * i + 1] = cs.y;
        mul2(y[2 * i], y[2 * i + 1], r, r);  // (r cos, r sin)
      }
    }
    // inverse rotation (rotation.rs:212-221), residual = vector - reconstruction (turbo.rs:268-273)
    fwht_inverse_signed<D>(y, tp.sgn_scale);
    float2 n2 = make_float2(0.0f, 0.0f);
    uint32_t res_any = 0;  // OR of the residual's magnitude bits: zero only for an all-zero residual
#pragma unroll
    for (int i = 0; i < D; i += 4) {
      float4* piece = reinterpret_cast<float4*>(s_xt + (i >> 5) * K::X_SLAB + (xsw ^ (((i >> 2) & 7) << 4)));
      const float4 t = *piece;
      // scalar subtractions on purpose: a packed subtraction right after the packed multiply by the
      // signed scale gets contracted into a fused multiply-add by the assembler (one rounding
      // instead of two), which moves residual elements by an ulp and, once in ~1e8 dots, a sign
      y[i] = __fsub_rn(t.x, y[i]);
      y[i + 1] = __fsub_rn(t.y, y[i + 1]);
      y[i + 2] = __fsub_rn(t.z, y[i + 2]);
      y[i + 3] = __fsub_rn(t.w, y[i + 3]);
      n2 = ffma2(make_float2(y[i], y[i + 1]), make_float2(y[i], y[i + 1]), n2);
      n2 = ffma2(make_float2(y[i + 2], y[i + 3]), make_float2(y[i + 2], y[i + 3]), n2);
      res_any |= (__float_as_uint(y[i]) | __float_as_uint(y[i + 1]) | __float_as_uint(y[i + 2]) |
                  __float_as_uint(y[i + 3])) & 0x7fffffffu;
      // the residual replaces x in the tile: it is the A operand of the QJL product
      *piece = make_float4(y[i], y[i + 1], y[i + 2], y[i + 3]);
    }
    // a non-finite residual element makes the squared norm non-finite (qjl.rs:210)
    const float nsq = n2.x + n2.y;
    if (!code && !pkv_finite(nsq)) {
      bool res_ok = true;
      for (int i = 0; i < D; i++) res_ok = res_ok && pkv_finite(*tile_at(s_xt, K::X_SLAB, row, i));
      if (!res_ok) code = PKV_VEC_NONFINITE_RESIDUAL;
    }
    // |residual| rounded up, the yardstick of both sign shortcuts.  Squares of elements below ~1e-19
    // underflow, so a sum under 1e-30 says nothing about the norm: such a vector is treated as
    // having an unbounded one (no shortcut certifies, every sign comes from the exact sequence).
    // Above that, underflowed squares change the sum by less than 1e-6 of it (the 1.0001 covers it).
    const float rnorm = nsq < 1.0e-30f ? __int_as_float(0x7f800000) : __fmul_rn(__fsqrt_rn(nsq), 1.0001f);

    // QjlQuantizer::sketch, qjl.rs:214-217: sign of the sequential f32 dot per projection row.
    // All 128 x m dots come from one TF32 product on the tensor cores: A = the CTA's residual
    // tile, B = the matrix tile, D in tensor memory with row r in lane r.
    pkv_tc::fence_smem_to_async();
    __syncthreads();
    const uint32_t tmem_d = s_tmem;
    if (threadIdx.x == 0 && !tp.skip_issue) {
      pkv_tc::fence_after_sync();
      const uint32_t idesc = pkv_tc::idesc_tf32(K::ROWS, m > 32 ? 64 : 32);
      const uint32_t a0 = pkv_tc::smem_u32(s_xt), b0 = pkv_tc::smem_u32(s_gt);
      // 8 columns = 32 bytes further along the rows; four steps per slab
      pkv_tc::mma_tf32_chain<D / 8>(tmem_d, a0, K::X_SLAB, b0, (uint32_t)g_slab, idesc, false);
      pkv_tc::mma_commit(&s_bar);
    }
    const bool done =
        __all_sync(0xffffffffu, pkv_tc::mbar_wait(&s_bar, 0, tp.skip_issue ? 256 : pkv_tc::kWaitPolls));
    pkv_tc::fence_after_sync();
    uint32_t* sw = w + (rw + tp.angle_words) * K::WS;
    if (done) {
#pragma unroll
      for (int c = 0; c < 64; c += 32) {  // unrolled: the thresholds below are read at fixed parameter offsets
        if (c >= m) break;
        float dots[32];
        pkv_tc::tmem_load32(tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)c, dots);
        uint32_t bits = 0, flagged = 0;
#pragma unroll
        for (int p = 0; p < 32; p++) {
          const float tau = fmaf(tp.qjl_thr_tf32[c + p], rnorm, PKV_QJL_ABS_BOUND);
          flagged |= (fabsf(dots[p]) > tau ? 0u : 1u) << p;
          bits |= (dots[p] >= 0.0f ? 1u : 0u) << p;
        }
        // an all-zero residual gives +-0 for every dot: sign bit 1 without further tests.  The test
        // is on the bits: a squared norm that merely underflowed to zero (elements below ~1e-23)
        // stays flagged, falls under the absolute bound and takes the exact sequence.
        if (!valid || res_any == 0u) flagged = 0;
        // Second tier (binary32 fused dot) and third (the reference's own sequence) for the flagged
        // (vector, row) pairs of the whole warp, spread over the lanes: each lane lists its pairs
        // at the position a prefix sum gives it, lane j settles list entry j, the owner reads the
        // sign back.  Pairs beyond the list's capacity are settled by their owner.
        const uint32_t cnt = __popc(flagged);
        uint32_t incl = cnt;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
          if (lane >= d) incl += t;
        }
        const uint32_t total = __shfl_sync(0xffffffffu, incl, 31);
        if (total) {
          if (lane == 0) atomicAdd(&g_turbo_stats[1], (unsigned long long)total);
          constexpr uint32_t CAP = PKV_QJL_LIST_CAP;
          float* s_rn = reinterpret_cast<float*>(s_off);                   // [32] (the offsets are spent)
          uint16_t* list = reinterpret_cast<uint16_t*>(s_rn + K::TV);      // [CAP]
          s_rn[v] = rnorm;
          uint32_t pos = incl - cnt;
          for (uint32_t f = flagged; f; f &= f - 1, pos++)
            if (pos < CAP) list[pos] = (uint16_t)((v << 5) | (__ffs(f) - 1));
          __syncwarp();
          const uint32_t n_list = min(total, CAP);
          for (uint32_t e = lane; e < n_list; e += 32) {
            const uint32_t it = list[e];
            const int r = warp * K::TV + (int)(it >> 5), p = c + (int)(it & 31u);
            float dot = fused_dot(s_gt, g_slab, p, s_xt, K::X_SLAB, r, D);
            const float tau = fmaf(s_thr[p], s_rn[it >> 5], PKV_QJL_ABS_BOUND);
            if (!(fabsf(dot) > tau)) {  // third tier, in the kernel for this variant: counted with the list entries
              dot = sequential_dot(s_gt, g_slab, p, s_xt, K::X_SLAB, r, D);
              atomicAdd(&g_turbo_stats[2], 1ull);
            }
            list[e] = (uint16_t)(it | (dot >= 0.0f ? 0x8000u : 0u));
          }
          __syncwarp();
          pos = incl - cnt;
          for (uint32_t f = flagged; f; f &= f - 1, pos++) {
            const int p = __ffs(f) - 1;
            bool plus;
            if (pos < CAP) {
              plus = (list[pos] & 0x8000u) != 0;
            } else {
              float dot = fused_dot(s_gt, g_slab, c + p, s_xt, K::X_SLAB, row, D);
              const float tau = fmaf(s_thr[c + p], rnorm, PKV_QJL_ABS_BOUND);
              if (!(fabsf(dot) > tau)) dot = sequential_dot(s_gt, g_slab, c + p, s_xt, K::X_SLAB, row, D);
              plus = dot >= 0.0f;
            }
            bits = plus ? (bits | (1u << p)) : (bits & ~(1u << p));
          }
          __syncwarp();
        }
        sw[(c >> 5) * K::WS] = bits;
      }
    } else if (threadIdx.x == 0) {
      pkv_report(err, 0, 0, PKV_VEC_DEVICE_WAIT);
    }
  }
  if (valid && code) pkv_report(err, 0, (int64_t)batch * g.vpb + v0 + v, code);
  if constexpr (DIRECT) {
    if (valid) {  // angle and sign words (patched in place by the fix-ups) follow the radii
      for (int k = 0; k < tile_words; k += 4)
        *reinterpret_cast<uint4*>(my_rec + 4 * (K::P + k)) =
            make_uint4(w[k * K::WS], w[(k + 1) * K::WS], w[(k + 2) * K::WS], w[(k + 3) * K::WS]);
    }
  } else if (!lossy) {
    if (valid)
      for (int k = 0; k < tile_words; k++) reinterpret_cast<uint32_t*>(my_rec)[K::P + k] = w[k * K::WS];
  } else {
    __syncwarp();
    stage_records<D, false>(
        s_w, reinterpret_cast<uint32_t*>(payload + (int64_t)batch * g.payload_batch_stride +
                                         (int64_t)v0 * g.rec_bytes),
        nv, tp.rec_words, lane);
  }
  if (m) {  // every warp has read its accumulator rows: the columns can go back
    pkv_tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) pkv_tc::tmem_free(s_tmem, tmem_cols);
  }
}

inline bool turbo_encode_direct(const TurboParams& tp) {
  return !tp.lossy && (tp.rec_words % 4) == 0 && ((tp.angle_words + tp.sign_words) % 4) == 0;
}

template <int D>
size_t turbo_encode_smem(const TurboParams& tp) {
  const int tile_words = tp.lossy ? tp.rec_words : tp.angle_words + tp.sign_words;
  return TurboEncSmem<D>::table_bytes(tp.projections, 1 << tp.polar_bits, tp.ray_count) +
         TurboEnc<D>::NWARPS * TurboEncSmem<D>::warp_bytes(tile_words, tp.lossy);
}

}  // namespace pkv_turbo
