// fib-quant encode for the cold-tier default (d = 64, fp16 norm, 5-bit indices): the dense
// rotation on the tensor cores.  Included by pkv_fib.cu inside its unnamed namespace.
//
// One thread per vector, one warp per tile of 32 vectors, one CTA = 4 warps = one 128-row
// tensor-core tile.  Per vector: exact f64 norm and certified normalisation as in
// pkv_fib_encode_fast.cuh; the normalised vector n is split into n_hi (11 significant bits, what a
// TF32 operand keeps) and the exact remainder n_lo, the f32 matrix likewise into M_hi + M_lo (split
// once on the host), and
//   y~ = n_lo M_hi^T + n_hi M_hi^T + n_hi M_lo^T        (three 128 x 64 x 64 TF32 products)
// accumulates in tensor memory (pkv_fast_paths.h gives the error bound PKV_FIB_ROT_ERR_TC).  The
// thread reads its row back and runs the certified nearest-codeword search on its 16 blocks.
// Blocks the bound cannot settle are redone by the whole warp in binary64 (fib_exact_block), which
// reproduces the reference's value unless it rounds within 2e-14 of a binary32 boundary; those few go
// on the list of fib_encode_fix_kernel, which redoes them with the reference's exact f64 sequence.
#pragma once

#include "pkv_tcgen05.cuh"

// The reference's nearest codeword of one block whose rotated values s0..s3 are exact: lane c evaluates
// the distance to codeword c in the reference's operation order (simd_nearest.rs:24-39,62-92) and the
// warp takes the smallest, lowest index first, which is what the strict-less-than scan returns.
__device__ __forceinline__ int fib_block_nearest_warp(float s0, float s1, float s2, float s3, const float4* s_cb,
                                                      int n_codewords, int order, int lane) {
  const float4 w = s_cb[lane];
  const int paired = order == PKV_ARGMIN_PAIRWISE ? (n_codewords & ~1) : 0;
  float dist;
  if (lane < paired) {
    const float d0 = __fsub_rn(w.x, s0), d1 = __fsub_rn(w.y, s1);
    const float d2 = __fsub_rn(w.z, s2), d3 = __fsub_rn(w.w, s3);
    dist = __fadd_rn(__fadd_rn(__fmul_rn(d0, d0), __fmul_rn(d1, d1)), __fadd_rn(__fmul_rn(d2, d2), __fmul_rn(d3, d3)));
  } else {
    const float d0 = __fsub_rn(s0, w.x), d1 = __fsub_rn(s1, w.y);
    const float d2 = __fsub_rn(s2, w.z), d3 = __fsub_rn(s3, w.w);
    dist = __fadd_rn(__fadd_rn(__fadd_rn(__fmul_rn(d0, d0), __fmul_rn(d1, d1)), __fmul_rn(d2, d2)), __fmul_rn(d3, d3));
  }
  // distances are sums of squares: non-negative, so their bit patterns order like the values
  const uint32_t key = lane < n_codewords ? __float_as_uint(dist) : 0xffffffffu;
  const uint32_t least = __reduce_min_sync(0xffffffffu, key);
  return __ffs(__ballot_sync(0xffffffffu, key == least)) - 1;
}

// Exact tier shared by the tensor-core encoders.  For one block of one vector whose normalised form
// (exact binary32, the reference's n) is row `trow` of the swizzled tile: the warp evaluates the four
// rotated values in binary64 from the f64 matrix (lane l takes columns l, l + 32, .., then a
// butterfly sum, bitwise the same in every lane), which differs from the reference's sequential
// binary64 sum (rotation.rs:104-115) by at most
//   (D + 1) 2^-53 + (D / 32 + 6) 2^-53  <  1.6e-14      (sum |M_rj n_j| <= |M_r| |n| = 1 to 1e-6),
// so the reference's (f32) rounding is known unless the value lies within PKV_FIB_F64_SUM_ERR of a
// binary32 rounding boundary.  With the exact block, lane c evaluates the reference's distance to
// codeword c in its operation order (simd_nearest.rs:24-39,62-92) and the warp takes the smallest,
// lowest index first, which is what the strict-less-than scan returns.  Result: the index, or -1
// when a rounding was not certain (the block then stays on the list of the fix-up kernel).
#define PKV_FIB_F64_SUM_ERR 2.0e-14
template <int D, int X_SLAB>
__device__ __forceinline__ int fib_exact_block(const uint8_t* s_xt, int trow, int gb, const double* __restrict__ rot,
                                               const float4* s_cb, int n_codewords, int order, int lane) {
  double part[4];
#pragma unroll
  for (int rr = 0; rr < 4; rr++) {
    const double* mrow = rot + (size_t)(4 * gb + rr) * D;
    double a = 0.0;
#pragma unroll
    for (int k = 0; k < D / 32; k++) {
      const int j = lane + 32 * k;
      a = __dadd_rn(a, __dmul_rn(__ldg(mrow + j), (double)*pkv_tc::tile_at(s_xt, X_SLAB, trow, j)));
    }
    part[rr] = a;
  }
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1)
#pragma unroll
    for (int rr = 0; rr < 4; rr++) part[rr] = __dadd_rn(part[rr], __shfl_xor_sync(0xffffffffu, part[rr], o));
  float s[4];
  bool sure = true;
#pragma unroll
  for (int rr = 0; rr < 4; rr++) {
    s[rr] = __double2float_rn(part[rr]);
    sure = sure && __double2float_rn(__dadd_rn(part[rr], PKV_FIB_F64_SUM_ERR)) ==
                       __double2float_rn(__dsub_rn(part[rr], PKV_FIB_F64_SUM_ERR));
  }
  const int idx = fib_block_nearest_warp(s[0], s[1], s[2], s[3], s_cb, n_codewords, order, lane);
  return sure ? idx : -1;
}

struct FibTc {
  static constexpr int D = 64, B = 16, THREADS = 128, NWARPS = 4, TV = 32, ROWS = 128;
  static constexpr int X_SLAB = ROWS * 128, X_BYTES = 2 * X_SLAB;  // vector tile: 2 slabs of [128 rows][128 B]
  static constexpr int M_SLAB = D * 128, M_BYTES = 2 * M_SLAB;     // matrix tile: 2 slabs of [64 rows][128 B]
  static constexpr int WARP_BYTES = TV * (int)sizeof(int64_t);
  static constexpr size_t SMEM = 1024 + X_BYTES + 2 * M_BYTES + 32 * sizeof(float4) + 32 * sizeof(float) +
                                 NWARPS * WARP_BYTES;
};

__global__ void __launch_bounds__(FibTc::THREADS, 3)
fib_encode_tc_kernel(PkvGeom g, const float* __restrict__ x, const float* __restrict__ rot_hi,
                     const float* __restrict__ rot_lo, const float* __restrict__ codebook,
                     const float* __restrict__ half_norm, int n_codewords, const double* __restrict__ rot,
                     int argmin_order, float score_abs, uint8_t* __restrict__ payload, uint64_t* err, uint32_t* flag_count,
                     uint32_t* flag_list, int skip_issue, float* __restrict__ y_capture) {
  using K = FibTc;
  using pkv_tc::sw_piece;
  using pkv_tc::tile_at;
  constexpr int D = K::D;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ uint32_t s_tmem;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint8_t* s_xt = smem + ((1024u - (pkv_tc::smem_u32(smem) & 1023u)) & 1023u);  // x, then n_lo, then n
  uint8_t* s_mh = s_xt + K::X_BYTES;                                           // M_hi [r][j]
  uint8_t* s_ml = s_mh + K::M_BYTES;                                           // M_lo [r][j]
  float4* s_cb = reinterpret_cast<float4*>(s_ml + K::M_BYTES);                 // [32] codewords
  float* s_hn = reinterpret_cast<float*>(s_cb + 32);                           // [32] |c|^2 / 2
  uint8_t* wbase = reinterpret_cast<uint8_t*>(s_hn + 32) + warp * K::WARP_BYTES;
  int64_t* s_off = reinterpret_cast<int64_t*>(wbase);                          // [TV]

  if (warp == 0) pkv_tc::tmem_alloc(&s_tmem, 64);
  if (threadIdx.x == 32) pkv_tc::mbar_init(&s_bar, 1);
  for (int i = threadIdx.x; i < D * 16; i += K::THREADS) {
    pkv_cp_async16(s_mh + sw_piece(K::M_SLAB, i >> 4, i & 15), reinterpret_cast<const float4*>(rot_hi) + i);
    pkv_cp_async16(s_ml + sw_piece(K::M_SLAB, i >> 4, i & 15), reinterpret_cast<const float4*>(rot_lo) + i);
  }
  if (threadIdx.x < 32) {
    s_cb[threadIdx.x] = __ldg(reinterpret_cast<const float4*>(codebook) + threadIdx.x);
    // entries past the codebook score higher than any real one
    s_hn[threadIdx.x] = (int)threadIdx.x < n_codewords ? __ldg(half_norm + threadIdx.x) : 3.0e38f;
  }
  const int v = lane, row = warp * K::TV + v;
  // piece c of this thread's row sits at s_xt + (c >> 3) * X_SLAB + (xsw ^ ((c & 7) << 4))
  const uint32_t xsw = (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((row & 7) << 4));
  const uint32_t idesc = pkv_tc::idesc_tf32(K::ROWS, D);
  const uint32_t a0 = pkv_tc::smem_u32(s_xt), bh = pkv_tc::smem_u32(s_mh), bl = pkv_tc::smem_u32(s_ml);
  const int64_t n_tiles = (int64_t)g.n_batches * g.tiles_per_batch;
  // skip_issue (test hook): the products are never issued, so the first wait runs out after a
  // short limit and the kernel takes its failure exit with nothing outstanding
  const int wait_limit = skip_issue ? 256 : pkv_tc::kWaitPolls;
  bool failed = false;
  uint32_t pending_parity = 0;  // phase the CTA was waiting for when it gave up

  // The CTA walks over groups of four tiles (one per warp); the matrix tiles, the codebook and the
  // tensor-memory columns are set up once.  Each round completes the barrier twice, so the phase
  // parities repeat from round to round.
  for (int64_t quad = blockIdx.x; quad * K::NWARPS < n_tiles; quad += gridDim.x) {
  const int64_t tile_id = quad * K::NWARPS + warp;
  const bool active = tile_id < n_tiles;
  const int tile = active ? (int)(tile_id % g.tiles_per_batch) : 0;
  const int batch = active ? (int)(tile_id / g.tiles_per_batch) : 0;
  const int v0 = tile * K::TV;
  const int nv = active ? min(K::TV, g.vpb - v0) : 0;
  const bool valid = v < nv;

  s_off[v] = valid ? pkv_vec_offset(g.L, batch, v0 + v) : 0;
  __syncwarp();
#pragma unroll 4
  for (int i = lane; i < nv * 16; i += 32) {
    const int vv = i >> 4, q = i & 15;
    pkv_cp_async16(s_xt + sw_piece(K::X_SLAB, warp * K::TV + vv, q),
                   reinterpret_cast<const float4*>(x + s_off[vv]) + q);
  }
  pkv_cp_async_wait_all();
  pkv_tc::fence_before_sync();
  __syncthreads();  // first round: tables, barrier, tensor-memory base; every round: the previous
                    // round's accumulator rows have been read by all warps
  pkv_tc::fence_after_sync();

  float n[D];
#pragma unroll
  for (int i = 0; i < D; i += 4) {
    const float4 t = valid ? *reinterpret_cast<const float4*>(s_xt + (i >> 5) * K::X_SLAB + (xsw ^ (((i >> 2) & 7) << 4)))
                           : make_float4(0.f, 0.f, 0.f, 0.f);
    n[i] = t.x; n[i + 1] = t.y; n[i + 2] = t.z; n[i + 3] = t.w;
  }

  // exact norm (codec.rs:1049-1057; the square of a binary32 value is exact in binary64, so the
  // fused form rounds exactly like the reference's multiply-then-add; a non-finite element makes the
  // sum non-finite), certified normalisation by the pair form, the division where that is unsure
  double acc = 0.0;
  uint32_t min_key = 0xffffffffu;
#pragma unroll
  for (int i = 0; i < D; i++) {
    const double t = (double)n[i];
    acc = fma(t, t, acc);
    min_key = min(min_key, pkv_fib_mag_key(n[i]));
  }
  const bool finite = acc < __longlong_as_double(0x7ff0000000000000ll);
  double norm = __dsqrt_rn(acc);
  int bad = 0;
  if (valid) {
    if (!finite) bad = PKV_VEC_NONFINITE_INPUT;
    else if (norm == 0.0) bad = PKV_VEC_ZERO_NORM;
    if (bad) pkv_report(err, 0, (int64_t)batch * g.vpb + v0 + v, bad);
  }
  const bool skip = bad || !valid;
  if (skip) norm = 1.0;
  {
    const double inv = __ddiv_rn(1.0, norm);
    const float invh = __double2float_rn(inv), invl = __double2float_rn(__dsub_rn(inv, (double)invh));
    uint32_t unsure = pkv_fib_fast_norm_ok(norm, min_key) ? 0u : 1u;
#pragma unroll
    for (int i = 0; i < D; i++) n[i] = pkv_fib_norm_quotient(n[i], invh, invl, &unsure);
    if (unsure || skip) {
      // rare: the reference's division element by element, through the tile (x is still there)
#pragma unroll 1
      for (int c = 0; c < D / 4; c++) {
        float4* cell = reinterpret_cast<float4*>(s_xt + (c >> 3) * K::X_SLAB + (xsw ^ ((c & 7) << 4)));
        float4 t = *cell;
        t.x = skip ? 0.0f : __double2float_rn(__ddiv_rn((double)t.x, norm));
        t.y = skip ? 0.0f : __double2float_rn(__ddiv_rn((double)t.y, norm));
        t.z = skip ? 0.0f : __double2float_rn(__ddiv_rn((double)t.z, norm));
        t.w = skip ? 0.0f : __double2float_rn(__ddiv_rn((double)t.w, norm));
        *cell = t;
      }
#pragma unroll
      for (int i = 0; i < D; i += 4) {
        const float4 t = *reinterpret_cast<const float4*>(s_xt + (i >> 5) * K::X_SLAB + (xsw ^ (((i >> 2) & 7) << 4)));
        n[i] = t.x; n[i + 1] = t.y; n[i + 2] = t.z; n[i + 3] = t.w;
      }
    }
  }

  // first operand: the exact remainder n_lo = n - n_hi (n_hi = n with its 13 low bits cleared);
  // one product (M_hi)
#pragma unroll
  for (int i = 0; i < D; i += 4) {
    float lo[4];
#pragma unroll
    for (int k = 0; k < 4; k++)
      lo[k] = __fsub_rn(n[i + k], __uint_as_float(__float_as_uint(n[i + k]) & 0xffffe000u));
    *reinterpret_cast<float4*>(s_xt + (i >> 5) * K::X_SLAB + (xsw ^ (((i >> 2) & 7) << 4))) =
        make_float4(lo[0], lo[1], lo[2], lo[3]);
  }
  pkv_tc::fence_smem_to_async();
  __syncthreads();
  if (threadIdx.x == 0 && !skip_issue) {
    pkv_tc::fence_after_sync();
    pkv_tc::mma_tf32_chain<D / 8>(s_tmem, a0, K::X_SLAB, bh, K::M_SLAB, idesc, false);
    pkv_tc::mma_commit(&s_bar);
  }
  // The outcome of a wait is made uniform over the CTA: when it ran out for any thread, every
  // warp leaves the loop together, no further product is issued and no accumulator is read.
  if (!__syncthreads_and(pkv_tc::mbar_wait(&s_bar, 0, wait_limit))) {
    failed = true;
    pending_parity = 0;
    break;
  }
  pkv_tc::fence_after_sync();
  // second operand: n itself -- the unit reads only its 11 leading bits, i.e. n_hi, and the full
  // value stays in the tile for the second tier; two products (M_hi, M_lo)
#pragma unroll
  for (int i = 0; i < D; i += 4)
    *reinterpret_cast<float4*>(s_xt + (i >> 5) * K::X_SLAB + (xsw ^ (((i >> 2) & 7) << 4))) =
        make_float4(n[i], n[i + 1], n[i + 2], n[i + 3]);
  pkv_tc::fence_smem_to_async();
  pkv_tc::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0) {
    pkv_tc::fence_after_sync();
    pkv_tc::mma_tf32_chain<D / 8>(s_tmem, a0, K::X_SLAB, bh, K::M_SLAB, idesc, true);
    pkv_tc::mma_tf32_chain<D / 8>(s_tmem, a0, K::X_SLAB, bl, K::M_SLAB, idesc, true);
    pkv_tc::mma_commit(&s_bar);
  }
  if (!__syncthreads_and(pkv_tc::mbar_wait(&s_bar, 1, wait_limit))) {
    failed = true;
    pending_parity = 1;
    break;
  }
  pkv_tc::fence_after_sync();

  uint32_t idx4[4] = {0, 0, 0, 0};  // four 8-bit indices per word
  uint32_t flagged = 0;             // blocks whose nearest codeword is not settled yet
  {
    float y[D];
    {
      float h0[32], h1[32];
      const uint32_t taddr = s_tmem + ((uint32_t)(warp * 32) << 16);
      pkv_tc::tmem_load32(taddr, h0);
      pkv_tc::tmem_load32(taddr + 32, h1);
#pragma unroll
      for (int i = 0; i < 32; i++) {
        y[i] = h0[i];
        y[32 + i] = h1[i];
      }
    }
    if (y_capture != nullptr && valid) {  // test hook: the rotated values as the tensor cores delivered them
      float4* dst = reinterpret_cast<float4*>(y_capture + ((int64_t)batch * g.vpb + v0 + v) * D);
#pragma unroll
      for (int i = 0; i < D; i += 4) dst[i >> 2] = make_float4(y[i], y[i + 1], y[i + 2], y[i + 3]);
    }
    // certified nearest codeword of the 16 blocks (pkv_fast_paths.h)
    float best[K::B], second[K::B];
#pragma unroll
    for (int b = 0; b < K::B; b++) best[b] = second[b] = __int_as_float(0x7f800000);
    // two codewords per step (the tables hold 32 entries; those past n_codewords never win)
#pragma unroll 1
    for (int c = 0; c < n_codewords; c += 2) {
      const float4 w0 = s_cb[c], w1 = s_cb[c + 1];
      const float hn0 = s_hn[c], hn1 = s_hn[c + 1];
#pragma unroll
      for (int b = 0; b < K::B; b++)
        pkv_fib_top2_pair(&best[b], &second[b],
                          pkv_fib_key(y[4 * b], y[4 * b + 1], y[4 * b + 2], y[4 * b + 3], w0.x, w0.y, w0.z, w0.w,
                                      hn0, (uint32_t)c),
                          pkv_fib_key(y[4 * b], y[4 * b + 1], y[4 * b + 2], y[4 * b + 3], w1.x, w1.y, w1.z, w1.w,
                                      hn1, (uint32_t)c + 1u));
    }
#pragma unroll
    for (int b = 0; b < K::B; b++) {
      idx4[b >> 2] |= (__float_as_uint(best[b]) & 31u) << (8 * (b & 3));
      if (!pkv_fib_certify_eta(best[b], second[b], y[4 * b], y[4 * b + 1], y[4 * b + 2], y[4 * b + 3],
                               PKV_FIB_ROT_ERR_TC, score_abs))
        flagged |= 1u << b;
    }
    if (skip) flagged = 0;
  }

  fib_count_flagged(flagged, lane);
  // Second tier: the flagged blocks of one vector at a time, the whole warp on each, exactly
  // (fib_exact_block); the owner keeps the result.
  for (unsigned pending = __ballot_sync(0xffffffffu, flagged != 0); pending; pending &= pending - 1) {
    const int src = __ffs(pending) - 1;
    uint32_t todo = __shfl_sync(0xffffffffu, flagged, src);
    while (todo) {
      const int b = __ffs(todo) - 1;
      todo &= todo - 1;
      const int idx = fib_exact_block<D, K::X_SLAB>(s_xt, warp * K::TV + src, b, rot, s_cb, n_codewords,
                                                    argmin_order, lane);
      if (lane == src && idx >= 0) {
        const int wi = b >> 2, sh = 8 * (b & 3);
#pragma unroll
        for (int k = 0; k < 4; k++)
          if (k == wi) idx4[k] = (idx4[k] & ~(0xffu << sh)) | ((uint32_t)idx << sh);
        flagged &= ~(1u << b);
      }
    }
  }

  // encode_norm (codec.rs:994-1020), pack_indices (bitpack.rs:4-44): the record is three words
  if (valid) {
    uint32_t rec0 = 0, rec1 = 0, rec2 = 0;
    if (!bad) {
      const float nf = __double2float_rn(norm);
      const uint32_t h = pkv_f32_to_f16_bits(nf);
      if ((h & 0x7fffu) < 0x7c00u && (h & 0x7fffu) != 0) {
        unsigned long long lo = 0;  // stream bits 0..63
        uint32_t hi = 0;            // stream bits 64..79
#pragma unroll
        for (int b = 0; b < K::B; b++) {
          const unsigned long long iv = (idx4[b >> 2] >> (8 * (b & 3))) & 31u;
          const int pos = 5 * b;
          if (pos < 64) lo |= iv << pos;
          if (pos + 5 > 64) hi |= (uint32_t)(iv >> (pos < 64 ? 64 - pos : 0)) << (pos < 64 ? 0 : pos - 64);
        }
        rec0 = h | ((uint32_t)lo << 16);
        rec1 = (uint32_t)(lo >> 16);
        rec2 = (uint32_t)(lo >> 48) | (hi << 16);
        if (flagged) {
          const uint32_t which = (flagged & (flagged - 1)) ? PKV_FIB_ENTRY_ALL
                                                                       : (uint32_t)(__ffs(flagged) - 1);
          const uint32_t gvec = (uint32_t)((int64_t)batch * g.vpb + v0 + v);
          flag_list[atomicAdd(flag_count, 1u)] = (gvec << 5) | which;
        }
      } else {
        pkv_report(err, 1, (int64_t)batch * g.vpb + v0 + v, PKV_VEC_NORM_RANGE);
      }
    }
    uint32_t* dst = reinterpret_cast<uint32_t*>(payload + (int64_t)batch * g.payload_batch_stride +
                                                (int64_t)(v0 + v) * 12);
    dst[0] = rec0;
    dst[1] = rec1;
    dst[2] = rec2;
  }
  }  // rounds
  if (failed) {
    // the launch's payload is declared invalid; give products that may still be in flight one
    // more bounded wait before the columns go back
    if (threadIdx.x == 0) pkv_report(err, 0, 0, PKV_VEC_DEVICE_WAIT);
    if (!skip_issue) pkv_tc::mbar_wait(&s_bar, pending_parity, wait_limit);
  }
  pkv_tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) pkv_tc::tmem_free(s_tmem, 64);
}
