// fib-quant encode with the rotation the reference's `gpu` build applies in encode_batch: an f32
// Walsh-Hadamard transform instead of the stored dense matrix (fib-quant/src/codec.rs:612-656 calls
// gpu_backend::hadamard_batch, whose arithmetic gpu-backend/src/fallback.rs:12-62 defines: butterflies
// (a, b) -> (a + b, a - b) for step = 1, 2, 4, .., then x sign_i, then x 1/sqrt(dim), all binary32).
// Included by pkv_fib.cu inside its unnamed namespace.
//
// Every operation of that transform is a correctly rounded binary32 operation on a fixed dataflow, so
// the kernel reproduces the rotated vector bit for bit without a second tier: one thread per vector,
// the vector in registers, the butterflies as packed two-lane adds and subtracts, the sign and the
// scale as one multiply by +-scale (RN(v s) for s = +-1 is exact, so RN(RN(v s) scale) = RN(v (s scale))).
// The nearest-codeword search is the certified top-2 search of the dense encoders with a rotation error
// of zero; a block whose two best scores are closer than the rounding of the reference's own distance
// arithmetic is settled by the warp with that arithmetic (fib_block_nearest_warp).  Nothing is left for
// a fix-up kernel.
#pragma once

struct FibWhtParams {
  float sgn_scale[128];  // sign_i / sqrt(dim) as the reference's f32 values multiply out
};

template <int D>
struct FibWht {
  static constexpr int B = D / 4, THREADS = 128, TV = 128;
  static constexpr int HB = 16;                       // blocks searched at a time
  static constexpr int X_SLAB = TV * 128, X_BYTES = (D / 32) * X_SLAB;  // D/32 slabs of [128 rows][128 B]
  static size_t smem(int rec) {
    return 1024 + X_BYTES + 32 * sizeof(float4) + sizeof(FibSearchTab) + TV * sizeof(int64_t) + (size_t)TV * rec + 16;
  }
};

template <int D>
__global__ void __launch_bounds__(FibWht<D>::THREADS, D == 128 ? 2 : 4)
fib_encode_wht_kernel(PkvGeom g, const float* __restrict__ x, const __grid_constant__ FibWhtParams prm,
                      const float* __restrict__ codebook, const float* __restrict__ half_norm, int n_codewords,
                      int idx_bits, int norm_len, int argmin_order, FibSearchBias bias, uint8_t* __restrict__ payload,
                      uint64_t* err) {
  using K = FibWht<D>;
  using pkv_tc::sw_piece;
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31;
  uint8_t* s_xt = smem + ((1024u - (pkv_tc::smem_u32(smem) & 1023u)) & 1023u);  // x, later y
  float4* s_cb = reinterpret_cast<float4*>(s_xt + K::X_BYTES);                  // [32] codewords
  FibSearchTab* s_tab = reinterpret_cast<FibSearchTab*>(s_cb + 32);
  int64_t* s_off = reinterpret_cast<int64_t*>(s_tab + 1);                       // [TV]
  uint8_t* s_rec = reinterpret_cast<uint8_t*>(s_off + K::TV);                   // [TV][rec]
  s_rec += (16 - (reinterpret_cast<uintptr_t>(s_rec) & 15)) & 15;

  const int tile = blockIdx.x % g.tiles_per_batch;
  const int batch = blockIdx.x / g.tiles_per_batch;
  const int v0 = tile * K::TV;
  const int nv = min(K::TV, g.vpb - v0);
  const int rec = g.rec_bytes;
  const bool valid = tid < nv;

  s_off[tid] = valid ? pkv_vec_offset(g.L, batch, v0 + tid) : 0;
  if (tid < 32) {
    s_cb[tid] = __ldg(reinterpret_cast<const float4*>(codebook) + tid);
    fib_search_fill(s_tab, codebook, half_norm, n_codewords, bias.off, tid);
  }
  __syncthreads();
#pragma unroll 4
  for (int i = tid; i < nv * (D / 4); i += K::THREADS) {
    const int vv = i / (D / 4), q = i % (D / 4);
    pkv_cp_async16(s_xt + sw_piece(K::X_SLAB, vv, q), reinterpret_cast<const float4*>(x + s_off[vv]) + q);
  }
  pkv_cp_async_wait_all();
  __syncthreads();

  // piece c of this thread's row sits at s_xt + (c >> 3) * X_SLAB + (xsw ^ ((c & 7) << 4))
  const uint32_t xsw = (uint32_t)((tid >> 3) * 1024 + (tid & 7) * 128 + ((tid & 7) << 4));
  float n[D];
#pragma unroll
  for (int i = 0; i < D; i += 4) {
    const float4 t = valid ? *reinterpret_cast<const float4*>(s_xt + (i >> 5) * K::X_SLAB + (xsw ^ (((i >> 2) & 7) << 4)))
                           : make_float4(0.f, 0.f, 0.f, 0.f);
    n[i] = t.x; n[i + 1] = t.y; n[i + 2] = t.z; n[i + 3] = t.w;
  }

  // exact norm (codec.rs:1049-1057; the square of a binary32 value is exact in binary64, so the fused
  // form rounds exactly like the reference's multiply-then-add; a non-finite element makes the sum
  // non-finite), certified normalisation by the pair form, the division where that is unsure
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
    if (bad) pkv_report(err, 0, (int64_t)batch * g.vpb + v0 + tid, bad);
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
      // rare: the reference's division element by element, from the tile (x is still there)
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

  // the transform (fallback.rs:34-56); the rotated row goes back to the tile for the exact tier
  pkv_turbo::fwht_inverse_signed<D>(n, prm.sgn_scale);
#pragma unroll
  for (int i = 0; i < D; i += 4)
    *reinterpret_cast<float4*>(s_xt + (i >> 5) * K::X_SLAB + (xsw ^ (((i >> 2) & 7) << 4))) =
        make_float4(n[i], n[i + 1], n[i + 2], n[i + 3]);

  // certified nearest codeword (pkv_fib_search.cuh, rotation error 0), HB blocks at a time
  uint32_t idx4[K::B / 4];  // four 8-bit indices per word
#pragma unroll
  for (int i = 0; i < K::B / 4; i++) idx4[i] = 0;
  uint32_t flagged = 0;
  unsigned long long yp[K::B / 2][4];  // the rotated row, two blocks per operand; n is not used again
  fib_search_pack<D, 0, K::B>(n, yp);
#pragma unroll
  for (int h = 0; h < K::B / K::HB; h++) {
    uint32_t best[K::HB], second[K::HB];
    if (h == 0) fib_search_keys<K::B, 0, K::HB>(yp, s_tab, n_codewords, bias.mult, best, second);
    if constexpr (K::B > K::HB)  // d = 128: the second half of the blocks
      if (h == 1) fib_search_keys<K::B, K::HB, K::HB>(yp, s_tab, n_codewords, bias.mult, best, second);
#pragma unroll
    for (int b = 0; b < K::HB; b++) {
      const int gb = K::HB * h + b;
      idx4[gb >> 2] |= (best[b] & 31u) << (8 * (gb & 3));
      // Quick test on the keys themselves: a gap of the two best scores above a constant derived on the
      // host from the codebook (pkv_fast_paths.h (3b)) certifies without looking at the block.
      if ((second[b] >> 5) - (best[b] >> 5) > bias.quick_gap) continue;
      float sb[4];
      fib_search_block<K::B>(yp, gb, sb);
      if (!pkv_fib_certify_abs(fib_search_score(best[b], bias.off), fib_search_score(second[b], bias.off), sb[0],
                               sb[1], sb[2], sb[3], 0.0f, bias.e_f))
        flagged |= 1u << gb;
    }
  }
  if (skip) flagged = 0;
  __syncwarp();  // the warp's rows of y are in the tile

  fib_count_flagged(flagged, lane);
  // exact tier: the flagged blocks of one vector at a time, lane c on codeword c
  for (unsigned pending = __ballot_sync(0xffffffffu, flagged != 0); pending; pending &= pending - 1) {
    const int src = __ffs(pending) - 1;
    uint32_t todo = __shfl_sync(0xffffffffu, flagged, src);
    const int srow = (tid & ~31) + src;
    while (todo) {
      const int b = __ffs(todo) - 1;
      todo &= todo - 1;
      const float4 s = *reinterpret_cast<const float4*>(s_xt + sw_piece(K::X_SLAB, srow, b));
      const int idx = fib_block_nearest_warp(s.x, s.y, s.z, s.w, s_cb, n_codewords, argmin_order, lane);
      if (lane == src) {
        const int wi = b >> 2, sh = 8 * (b & 3);
#pragma unroll
        for (int k = 0; k < K::B / 4; k++)
          if (k == wi) idx4[k] = (idx4[k] & ~(0xffu << sh)) | ((uint32_t)idx << sh);
      }
    }
  }

  // encode_norm (codec.rs:994-1020) + pack_indices (bitpack.rs:4-44)
  if (valid) {
    uint8_t* r = s_rec + tid * rec;
    for (int i = 0; i < rec; i++) r[i] = 0;
    if (!bad) {
      const float nf = __double2float_rn(norm);
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
        pkv_report(err, 1, (int64_t)batch * g.vpb + v0 + tid, PKV_VEC_NORM_RANGE);
        for (int i = 0; i < norm_len; i++) r[i] = 0;
      } else {
#pragma unroll
        for (int b = 0; b < K::B; b++) {
          const int pos = b * idx_bits;
          const uint32_t val = ((idx4[b >> 2] >> (8 * (b & 3))) & 31u) << (pos & 7);
          r[norm_len + (pos >> 3)] |= (uint8_t)val;
          if (val >> 8) r[norm_len + (pos >> 3) + 1] |= (uint8_t)(val >> 8);
        }
      }
    }
  }
  __syncthreads();
  stage_out(payload + (int64_t)batch * g.payload_batch_stride + (int64_t)v0 * rec, s_rec, nv * rec);
}
