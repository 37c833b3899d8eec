// fib-quant encode for d = 128 (fp16 norm, 5-bit indices): the dense rotation on the tensor cores.
// Included by pkv_fib.cu inside its unnamed namespace, after pkv_fib_encode_tc.cuh.
//
// The three operand tiles of the split product (n, M_hi, M_lo: 64 KB each) fill most of an SM's
// shared memory, so one persistent CTA runs per SM and PARTS threads share a vector:
// thread (row, part) normalises elements EPT part .. EPT part + EPT - 1 of vector `row`, and after the
//   y~ = n_lo M_hi^T + n_hi M_hi^T + n_hi M_lo^T        (three 128 x 128 x 128 TF32 products)
// reads accumulator columns EPT part .. (blocks HB part .. HB part + HB - 1) of its row from tensor
// memory -- warps w, w + 4, .. all own lanes 32 (w % 4) .. of it -- and runs the certified search on
// them.  Every thread of a vector runs the whole f64 norm chain (its order is the reference's).
// Tiers as for d = 64: tensor-core value with PKV_FIB_ROT_ERR_TC128, then the warp in binary64
// (fib_exact_block), then the list of fib_encode_fix_kernel<128>.
#pragma once

struct FibTc128 {
  static constexpr int D = 128, PARTS = 2, ROWS = 128, REC = 22;
  static constexpr int THREADS = ROWS * PARTS, NWARPS = THREADS / 32;
  static constexpr int EPT = D / PARTS;   // elements normalised / accumulator columns read per thread
  static constexpr int PPT = EPT / 4;     // 16-byte pieces of the row per thread
  static constexpr int HB = EPT / 4;      // blocks searched per thread
  static constexpr int X_SLAB = ROWS * 128, X_BYTES = 4 * X_SLAB;  // vector tile: 4 slabs of [128 rows][128 B]
  static constexpr int M_SLAB = D * 128, M_BYTES = 4 * M_SLAB;     // matrix tile: 4 slabs of [128 rows][128 B]
  static constexpr size_t SMEM = 1024 + X_BYTES + 2 * M_BYTES + 32 * sizeof(float4) + 32 * sizeof(float) +
                                 ROWS * (sizeof(int64_t) + sizeof(double) + 2 * sizeof(uint32_t)) + ROWS * REC + 16;
  static_assert(PARTS == 2 || PARTS == 4, "threads per vector");
};

__global__ void __launch_bounds__(FibTc128::THREADS, 1)
fib_encode_tc128_kernel(PkvGeom g, const float* __restrict__ x, const float* __restrict__ rot_hi,
                        const float* __restrict__ rot_lo, const float* __restrict__ codebook,
                        const float* __restrict__ half_norm, int n_codewords, const double* __restrict__ rot,
                        int argmin_order, float score_abs, uint8_t* __restrict__ payload, uint64_t* err, uint32_t* flag_count,
                        uint32_t* flag_list, int skip_issue, float* __restrict__ y_capture) {
  using K = FibTc128;
  using pkv_tc::sw_piece;
  constexpr int D = K::D;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ uint32_t s_tmem;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = threadIdx.x & 127, part = threadIdx.x >> 7;
  uint8_t* s_xt = smem + ((1024u - (pkv_tc::smem_u32(smem) & 1023u)) & 1023u);  // x, then n_lo, then n
  uint8_t* s_mh = s_xt + K::X_BYTES;                                           // M_hi [r][j]
  uint8_t* s_ml = s_mh + K::M_BYTES;                                           // M_lo [r][j]
  float4* s_cb = reinterpret_cast<float4*>(s_ml + K::M_BYTES);                 // [32] codewords
  float* s_hn = reinterpret_cast<float*>(s_cb + 32);                           // [32] |c|^2 / 2
  int64_t* s_off = reinterpret_cast<int64_t*>(s_hn + 32);                      // [ROWS]
  double* s_sq = reinterpret_cast<double*>(s_off + K::ROWS);                   // [ROWS] squared norms
  uint32_t* s_key = reinterpret_cast<uint32_t*>(s_sq + K::ROWS);               // [ROWS] smallest nonzero magnitude keys
  uint32_t* s_flag = s_key + K::ROWS;                                          // [ROWS] undecided blocks
  uint8_t* s_rec = reinterpret_cast<uint8_t*>(s_flag + K::ROWS);               // [ROWS][22]
  s_rec += (16 - (pkv_tc::smem_u32(s_rec) & 15u)) & 15u;

  if (warp == 0) pkv_tc::tmem_alloc(&s_tmem, 128);
  if (threadIdx.x == 32) pkv_tc::mbar_init(&s_bar, 1);
  for (int i = threadIdx.x; i < D * 32; i += K::THREADS) {
    pkv_cp_async16(s_mh + sw_piece(K::M_SLAB, i >> 5, i & 31), reinterpret_cast<const float4*>(rot_hi) + i);
    pkv_cp_async16(s_ml + sw_piece(K::M_SLAB, i >> 5, i & 31), reinterpret_cast<const float4*>(rot_lo) + i);
  }
  if (threadIdx.x < 32) {
    s_cb[threadIdx.x] = __ldg(reinterpret_cast<const float4*>(codebook) + threadIdx.x);
    // entries past the codebook score higher than any real one
    s_hn[threadIdx.x] = (int)threadIdx.x < n_codewords ? __ldg(half_norm + threadIdx.x) : 3.0e38f;
  }
  // piece c of this thread's row sits at s_xt + (c >> 3) * X_SLAB + (xsw ^ ((c & 7) << 4))
  const uint32_t xsw = (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((row & 7) << 4));
  const uint32_t idesc = pkv_tc::idesc_tf32(K::ROWS, D);
  const uint32_t a0 = pkv_tc::smem_u32(s_xt), bh = pkv_tc::smem_u32(s_mh), bl = pkv_tc::smem_u32(s_ml);
  const int64_t n_tiles = (int64_t)g.n_batches * g.tiles_per_batch;
  const int wait_limit = skip_issue ? 256 : pkv_tc::kWaitPolls;  // test hook: see fib_encode_tc_kernel
  bool failed = false;
  uint32_t pending_parity = 0;

  // element offset of this thread's row in tile `id` (threads with part == 0 only; 0 past the batch's end)
  auto row_offset = [&](int64_t id) -> int64_t {
    if (id >= n_tiles) return 0;
    const int t = (int)(id % g.tiles_per_batch), b = (int)(id / g.tiles_per_batch);
    return t * K::ROWS + row < g.vpb ? pkv_vec_offset(g.L, b, t * K::ROWS + row) : 0;
  };
  int64_t off_next = part == 0 ? row_offset(blockIdx.x) : 0;  // computed one round ahead, where the row is prefetched

  for (int64_t tile_id = blockIdx.x; tile_id < n_tiles; tile_id += gridDim.x) {
  const int tile = (int)(tile_id % g.tiles_per_batch);
  const int batch = (int)(tile_id / g.tiles_per_batch);
  const int v0 = tile * K::ROWS;
  const int nv = min(K::ROWS, g.vpb - v0);
  const bool valid = row < nv;

  if (part == 0) {
    s_off[row] = off_next;
    s_flag[row] = 0;
  }
  __syncthreads();  // also: the previous round's records have been copied out
#pragma unroll 4
  for (int i = threadIdx.x; i < nv * 32; i += K::THREADS) {
    const int vv = i >> 5, q = i & 31;
    pkv_cp_async16(s_xt + sw_piece(K::X_SLAB, vv, q), reinterpret_cast<const float4*>(x + s_off[vv]) + q);
  }
  pkv_cp_async_wait_all();
  pkv_tc::fence_before_sync();
  __syncthreads();  // first round: tables, barrier, tensor-memory base; every round: the previous
                    // round's accumulator rows have been read by all warps
  pkv_tc::fence_after_sync();

  // exact norm over the whole row in the reference's order (codec.rs:1049-1057; see
  // fib_encode_tc_kernel): one thread per vector runs the chain (the conversions to binary64 are what
  // it costs, so it is not repeated by the other threads of the vector) and shares the sum
  float n[K::EPT];
  if (part == 0) {
    double sq = 0.0;
    uint32_t key = 0xffffffffu;
#pragma unroll 8
    for (int c = 0; c < D / 4; c++) {
      const float4 t = valid ? *reinterpret_cast<const float4*>(s_xt + (c >> 3) * K::X_SLAB + (xsw ^ ((c & 7) << 4)))
                             : make_float4(0.f, 0.f, 0.f, 0.f);
      sq = fma((double)t.x, (double)t.x, sq);
      sq = fma((double)t.y, (double)t.y, sq);
      sq = fma((double)t.z, (double)t.z, sq);
      sq = fma((double)t.w, (double)t.w, sq);
      key = min(min(key, min(pkv_fib_mag_key(t.x), pkv_fib_mag_key(t.y))),
                min(pkv_fib_mag_key(t.z), pkv_fib_mag_key(t.w)));
    }
    s_sq[row] = sq;
    s_key[row] = key;
  }
#pragma unroll
  for (int i = 0; i < K::EPT; i += 4) {
    const int c = part * K::PPT + (i >> 2);
    const float4 t = valid ? *reinterpret_cast<const float4*>(s_xt + (c >> 3) * K::X_SLAB + (xsw ^ ((c & 7) << 4)))
                           : make_float4(0.f, 0.f, 0.f, 0.f);
    n[i] = t.x; n[i + 1] = t.y; n[i + 2] = t.z; n[i + 3] = t.w;
  }
  __syncthreads();  // the sums are there, and every chain has read the tile: parts may now be rewritten in place
  const double acc = s_sq[row];
  const uint32_t min_key = s_key[row];
  const bool finite = acc < __longlong_as_double(0x7ff0000000000000ll);
  double norm = __dsqrt_rn(acc);
  int bad = 0;
  if (valid) {
    if (!finite) bad = PKV_VEC_NONFINITE_INPUT;
    else if (norm == 0.0) bad = PKV_VEC_ZERO_NORM;
    if (bad && part == 0) pkv_report(err, 0, (int64_t)batch * g.vpb + v0 + row, bad);
  }
  const bool skip = bad || !valid;
  if (skip) norm = 1.0;
  {
    const double inv = __ddiv_rn(1.0, norm);
    const float invh = __double2float_rn(inv), invl = __double2float_rn(__dsub_rn(inv, (double)invh));
    uint32_t unsure = pkv_fib_fast_norm_ok(norm, min_key) ? 0u : 1u;
#pragma unroll
    for (int i = 0; i < K::EPT; i++) n[i] = pkv_fib_norm_quotient(n[i], invh, invl, &unsure);
    if (unsure || skip) {
      // rare: the reference's division element by element, through the tile (x is still there)
#pragma unroll 1
      for (int c = part * K::PPT; c < (part + 1) * K::PPT; c++) {
        float4* cell = reinterpret_cast<float4*>(s_xt + (c >> 3) * K::X_SLAB + (xsw ^ ((c & 7) << 4)));
        float4 t = *cell;
        t.x = skip ? 0.0f : __double2float_rn(__ddiv_rn((double)t.x, norm));
        t.y = skip ? 0.0f : __double2float_rn(__ddiv_rn((double)t.y, norm));
        t.z = skip ? 0.0f : __double2float_rn(__ddiv_rn((double)t.z, norm));
        t.w = skip ? 0.0f : __double2float_rn(__ddiv_rn((double)t.w, norm));
        *cell = t;
      }
#pragma unroll
      for (int i = 0; i < K::EPT; i += 4) {
        const int c = part * K::PPT + (i >> 2);
        const float4 t = *reinterpret_cast<const float4*>(s_xt + (c >> 3) * K::X_SLAB + (xsw ^ ((c & 7) << 4)));
        n[i] = t.x; n[i + 1] = t.y; n[i + 2] = t.z; n[i + 3] = t.w;
      }
    }
  }

  // first operand: the exact remainder n_lo = n - n_hi; one product (M_hi)
#pragma unroll
  for (int i = 0; i < K::EPT; i += 4) {
    const int c = part * K::PPT + (i >> 2);
    float lo[4];
#pragma unroll
    for (int k = 0; k < 4; k++)
      lo[k] = __fsub_rn(n[i + k], __uint_as_float(__float_as_uint(n[i + k]) & 0xffffe000u));
    *reinterpret_cast<float4*>(s_xt + (c >> 3) * K::X_SLAB + (xsw ^ ((c & 7) << 4))) =
        make_float4(lo[0], lo[1], lo[2], lo[3]);
  }
  pkv_tc::fence_smem_to_async();
  __syncthreads();
  if (threadIdx.x == 0 && !skip_issue) {
    pkv_tc::fence_after_sync();
    pkv_tc::mma_tf32_chain<D / 8>(s_tmem, a0, K::X_SLAB, bh, K::M_SLAB, idesc, false);
    pkv_tc::mma_commit(&s_bar);
  }
  if (!__syncthreads_and(pkv_tc::mbar_wait(&s_bar, 0, wait_limit))) {
    failed = true;
    pending_parity = 0;
    break;
  }
  pkv_tc::fence_after_sync();
  // second operand: n itself (the unit reads n_hi); two products (M_hi, M_lo)
#pragma unroll
  for (int i = 0; i < K::EPT; i += 4) {
    const int c = part * K::PPT + (i >> 2);
    *reinterpret_cast<float4*>(s_xt + (c >> 3) * K::X_SLAB + (xsw ^ ((c & 7) << 4))) =
        make_float4(n[i], n[i + 1], n[i + 2], n[i + 3]);
  }
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

  // the next tile's rows on their way into L2 while this one is searched (four 128-byte lines per row)
  if (part == 0) {
    const int64_t next_id = tile_id + gridDim.x;
    off_next = row_offset(next_id);
    if (next_id < n_tiles && (int)(next_id % g.tiles_per_batch) * K::ROWS + row < g.vpb) {
#pragma unroll
      for (int q = 0; q < D / 32; q++) asm volatile("prefetch.global.L2 [%0];" ::"l"(x + off_next + 32 * q));
    }
  }
  uint32_t idx4[K::HB / 4] = {};  // four 8-bit indices per word: this thread's blocks
  uint32_t flagged = 0;             // those whose nearest codeword is not settled yet
  {
    float y[K::EPT];
    {
      const uint32_t taddr = s_tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(part * K::EPT);
#pragma unroll
      for (int h = 0; h < K::EPT / 32; h++) {
        float part32[32];
        pkv_tc::tmem_load32(taddr + 32 * h, part32);
#pragma unroll
        for (int i = 0; i < 32; i++) y[32 * h + i] = part32[i];
      }
    }
    if (y_capture != nullptr && valid) {  // test hook: the rotated values as the tensor cores delivered them
      float4* dst = reinterpret_cast<float4*>(y_capture + ((int64_t)batch * g.vpb + v0 + row) * D + part * K::EPT);
#pragma unroll
      for (int i = 0; i < K::EPT; i += 4) dst[i >> 2] = make_float4(y[i], y[i + 1], y[i + 2], y[i + 3]);
    }
    float best[K::HB], second[K::HB];
#pragma unroll
    for (int b = 0; b < K::HB; b++) best[b] = second[b] = __int_as_float(0x7f800000);
    // two codewords per step (the tables hold 32 entries; those past n_codewords never win)
#pragma unroll 1
    for (int c = 0; c < n_codewords; c += 2) {
      const float4 w0 = s_cb[c], w1 = s_cb[c + 1];
      const float hn0 = s_hn[c], hn1 = s_hn[c + 1];
#pragma unroll
      for (int b = 0; b < K::HB; b++)
        pkv_fib_top2_pair(&best[b], &second[b],
                          pkv_fib_key(y[4 * b], y[4 * b + 1], y[4 * b + 2], y[4 * b + 3], w0.x, w0.y, w0.z, w0.w,
                                      hn0, (uint32_t)c),
                          pkv_fib_key(y[4 * b], y[4 * b + 1], y[4 * b + 2], y[4 * b + 3], w1.x, w1.y, w1.z, w1.w,
                                      hn1, (uint32_t)c + 1u));
    }
#pragma unroll
    for (int b = 0; b < K::HB; b++) {
      idx4[b >> 2] |= (__float_as_uint(best[b]) & 31u) << (8 * (b & 3));
      if (!pkv_fib_certify_eta(best[b], second[b], y[4 * b], y[4 * b + 1], y[4 * b + 2], y[4 * b + 3],
                               PKV_FIB_ROT_ERR_TC128, score_abs))
        flagged |= 1u << b;
    }
    if (skip) flagged = 0;
  }

  fib_count_flagged(flagged, lane);
  // Second tier: the flagged blocks of one thread at a time, the whole warp on each, exactly
  // (fib_exact_block); the owner keeps the result.
  for (unsigned pending = __ballot_sync(0xffffffffu, flagged != 0); pending; pending &= pending - 1) {
    const int src = __ffs(pending) - 1;
    uint32_t todo = __shfl_sync(0xffffffffu, flagged, src);
    while (todo) {
      const int b = __ffs(todo) - 1;
      todo &= todo - 1;
      const int idx = fib_exact_block<D, K::X_SLAB>(s_xt, (warp & 3) * 32 + src, part * K::HB + b, rot, s_cb,
                                                    n_codewords, argmin_order, lane);
      if (lane == src && idx >= 0) {
        const int wi = b >> 2, sh = 8 * (b & 3);
#pragma unroll
        for (int k = 0; k < K::HB / 4; k++)
          if (k == wi) idx4[k] = (idx4[k] & ~(0xffu << sh)) | ((uint32_t)idx << sh);
        flagged &= ~(1u << b);
      }
    }
  }

  // encode_norm (codec.rs:994-1020), pack_indices (bitpack.rs:4-44): the record is the fp16 norm and
  // 160 index bits, 5 HB of them (a whole number of bytes) from each thread of the vector
  {
    const float nf = __double2float_rn(norm);
    const uint32_t h = pkv_f32_to_f16_bits(nf);
    const bool norm_ok = (h & 0x7fffu) < 0x7c00u && (h & 0x7fffu) != 0;
    unsigned long long lo = 0;  // stream bits 0..63 of this part
    uint32_t hi = 0;            // stream bits 64..79 (HB = 16 only)
    if (!bad && norm_ok) {
#pragma unroll
      for (int b = 0; b < K::HB; b++) {
        const unsigned long long iv = (idx4[b >> 2] >> (8 * (b & 3))) & 31u;
        const int pos = 5 * b;
        if (pos < 64) lo |= iv << pos;
        if (pos + 5 > 64) hi |= (uint32_t)(iv >> (pos < 64 ? 64 - pos : 0)) << (pos < 64 ? 0 : pos - 64);
      }
    } else {
      flagged = 0;
    }
    uint8_t* r8 = s_rec + row * K::REC;
    if (part == 0) *reinterpret_cast<uint16_t*>(r8) = (!bad && norm_ok) ? (uint16_t)h : (uint16_t)0;
    uint8_t* mine = r8 + 2 + (5 * K::HB / 8) * part;
#pragma unroll
    for (int k = 0; k < 5 * K::HB / 8; k++) mine[k] = k < 8 ? (uint8_t)(lo >> (8 * k)) : (uint8_t)(hi >> (8 * (k - 8)));
    if (flagged) atomicOr(&s_flag[row], flagged << (K::HB * part));
    if (valid && !bad && !norm_ok && part == 0)
      pkv_report(err, 1, (int64_t)batch * g.vpb + v0 + row, PKV_VEC_NORM_RANGE);
  }
  __syncthreads();
  if (part == 0 && valid) {
    const uint32_t fl = s_flag[row];
    if (fl) {
      const uint32_t which = (fl & (fl - 1)) ? PKV_FIB_ENTRY_ALL : (uint32_t)(__ffs(fl) - 1);
      const uint32_t gvec = (uint32_t)((int64_t)batch * g.vpb + v0 + row);
      flag_list[atomicAdd(flag_count, 1u)] = (gvec << 5) | which;
    }
  }
  stage_out(payload + (int64_t)batch * g.payload_batch_stride + (int64_t)v0 * K::REC, s_rec, nv * K::REC);
  }  // rounds
  if (failed) {
    // the launch's payload is declared invalid; give products that may still be in flight one
    // more bounded wait before the columns go back
    if (threadIdx.x == 0) pkv_report(err, 0, 0, PKV_VEC_DEVICE_WAIT);
    if (!skip_issue) pkv_tc::mbar_wait(&s_bar, pending_parity, wait_limit);
  }
  pkv_tc::fence_before_sync();
  __syncthreads();
  if (warp == 0) pkv_tc::tmem_free(s_tmem, 128);
}
