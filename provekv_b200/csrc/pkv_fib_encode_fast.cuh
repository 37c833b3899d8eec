// fib-quant encode, two kernels (included by pkv_fib.cu inside its unnamed namespace).
//
// fib_encode_fast_kernel: every vector through certified shortcuts (pkv_fast_paths.h): exact f64
// norm, certified normalisation, binary32 fused rotation as a register-tiled product with the
// f32 copy of the matrix, certified nearest-codeword per 4-block, 5-bit packing.  Blocks (or whole
// vectors) whose decision could not be certified are appended to a list in global scratch memory.
// fib_encode_fix_kernel: one warp per list entry redoes the entry with the reference's exact
// operation sequence (fib-quant/src/codec.rs:594-729, rotation.rs:104-115,
// gpu-backend/src/simd_nearest.rs:24-94) and patches the record.
// Together they emit the same bytes as fib_encode_kernel; the exact f64 work shrinks from
// 2*dim*dim operations per vector to a few per mille of the blocks.
#pragma once

// list entry: (global vector index << 5) | block, block 31 = every block of the vector
#define PKV_FIB_ENTRY_ALL 31u

template <int D>
struct FibFast {
  static constexpr int B = D / 4;
  static constexpr int THREADS = 128;
  static constexpr int VPT = 8;  // vectors per thread in the product
  static constexpr int RG = D / 8;              // threads along the rows (2 blocks each)
  static constexpr int VG = THREADS / RG;       // threads along the vectors (VPT vectors each)
  static constexpr int TV = VG * VPT;           // 128 vectors (D = 64), 64 (D = 128)
  static constexpr int SPLIT = THREADS / TV;    // threads sharing one vector's normalisation
  static constexpr int EPT = D / SPLIT;         // elements each of them normalises
  static constexpr int XS = D + 4;              // row stride of the staged input tile
  static constexpr size_t tile_floats = (size_t)TV * XS > (size_t)D * TV ? (size_t)TV * XS : (size_t)D * TV;
};

template <int D>
__global__ void __launch_bounds__(FibFast<D>::THREADS, D == 128 ? 2 : 3)
fib_encode_fast_kernel(PkvGeom g, const float* __restrict__ x, const float* __restrict__ rot32_t,
                       const float* __restrict__ codebook, const float* __restrict__ half_norm,
                       int n_codewords, int idx_bits, int norm_len, float score_abs, uint8_t* __restrict__ payload,
                       uint64_t* err, uint32_t* flag_count, uint32_t* flag_list) {
  using K = FibFast<D>;
  extern __shared__ __align__(128) uint8_t smem[];
  float* s_m = reinterpret_cast<float*>(smem);                     // [j][r] = (f32) M[r][j]
  float* s_t = s_m + D * D;                                        // input tile [TV][XS], then n~ [j][TV]
  float4* s_cb = reinterpret_cast<float4*>(s_t + K::tile_floats);  // [32]
  float* s_hn = reinterpret_cast<float*>(s_cb + 32);               // [32]
  double* s_norm = reinterpret_cast<double*>(s_hn + 32);           // [TV]
  int64_t* s_off = reinterpret_cast<int64_t*>(s_norm + K::TV);     // [TV]
  uint32_t* s_flag = reinterpret_cast<uint32_t*>(s_off + K::TV);   // [TV] undecided-block masks
  uint8_t* s_bad = reinterpret_cast<uint8_t*>(s_flag + K::TV);     // [TV]
  uint8_t* s_idx = s_bad + K::TV;                                  // [TV][B]
  uint8_t* s_rec = s_idx + K::TV * K::B;                           // [TV][rec], 16-aligned below
  s_rec += (16 - (reinterpret_cast<uintptr_t>(s_rec) & 15)) & 15;

  const int tile = blockIdx.x % g.tiles_per_batch;
  const int batch = blockIdx.x / g.tiles_per_batch;
  const int v0 = tile * K::TV;
  const int nv = min(K::TV, g.vpb - v0);
  const int rec = g.rec_bytes;
  const int tid = threadIdx.x;

  for (int v = tid; v < K::TV; v += K::THREADS) {
    s_off[v] = v < nv ? pkv_vec_offset(g.L, batch, v0 + v) : 0;
    s_flag[v] = 0;
  }
  for (int i = tid; i < D * D / 4; i += K::THREADS)
    pkv_cp_async16(reinterpret_cast<float4*>(s_m) + i, reinterpret_cast<const float4*>(rot32_t) + i);
  if (tid < 32) {
    s_cb[tid] = __ldg(reinterpret_cast<const float4*>(codebook) + tid);
    s_hn[tid] = tid < n_codewords ? __ldg(half_norm + tid) : 3.0e38f;  // padding scores above any real entry
  }
  __syncthreads();
  for (int i = tid; i < nv * (D / 4); i += K::THREADS) {
    const int v = i / (D / 4), q = i % (D / 4);
    pkv_cp_async16(s_t + v * K::XS + 4 * q, reinterpret_cast<const float4*>(x + s_off[v]) + q);
  }
  pkv_cp_async_wait_all();
  __syncthreads();

  // (A) exact norm (codec.rs:1049-1057; the square of a binary32 value is exact in binary64, so
  // the fused form rounds exactly like the reference's multiply-then-add), then the certified
  // normalised vector written transposed, n~[j][v], over the input tile.  SPLIT threads share a
  // vector: each runs the whole norm chain from the tile and normalises its own EPT elements.
  {
    const int v = tid % K::TV, part = tid / K::TV;
    const float* row = s_t + v * K::XS;
    double acc = 0.0;  // a non-finite element makes the sum non-finite
    uint32_t min_key = 0xffffffffu;
#pragma unroll 8
    for (int i = 0; i < D; i += 4) {
      const float4 t = v < nv ? *reinterpret_cast<const float4*>(row + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      acc = fma((double)t.x, (double)t.x, acc);
      acc = fma((double)t.y, (double)t.y, acc);
      acc = fma((double)t.z, (double)t.z, acc);
      acc = fma((double)t.w, (double)t.w, acc);
      min_key = min(min(min_key, min(pkv_fib_mag_key(t.x), pkv_fib_mag_key(t.y))),
                    min(pkv_fib_mag_key(t.z), pkv_fib_mag_key(t.w)));
    }
    const bool finite = acc < __longlong_as_double(0x7ff0000000000000ll);
    float xr[K::EPT];
#pragma unroll
    for (int i = 0; i < K::EPT; i += 4) {
      const float4 t = v < nv ? *reinterpret_cast<const float4*>(row + part * K::EPT + i)
                              : make_float4(0.f, 0.f, 0.f, 0.f);
      xr[i] = t.x; xr[i + 1] = t.y; xr[i + 2] = t.z; xr[i + 3] = t.w;
    }
    __syncthreads();  // every row has been read: the tile may now be overwritten
    double norm = __dsqrt_rn(acc);
    int bad = 0;
    if (v < nv) {
      if (!finite) bad = PKV_VEC_NONFINITE_INPUT;
      else if (norm == 0.0) bad = PKV_VEC_ZERO_NORM;
      if (bad && part == 0) pkv_report(err, 0, (int64_t)batch * g.vpb + v0 + v, bad);
    }
    const bool skip = bad || v >= nv;
    if (skip) norm = 1.0;
    if (part == 0) {
      s_norm[v] = norm;
      s_bad[v] = (uint8_t)skip;
    }
    const double inv = __ddiv_rn(1.0, norm);
    const float invh = __double2float_rn(inv), invl = __double2float_rn(__dsub_rn(inv, (double)invh));
    uint32_t unsure = pkv_fib_fast_norm_ok(norm, min_key) ? 0u : 1u;
    float q[K::EPT];
#pragma unroll
    for (int i = 0; i < K::EPT; i++) q[i] = pkv_fib_norm_quotient(xr[i], invh, invl, &unsure);
    if (unsure && !skip) {  // rare: the reference's division
#pragma unroll
      for (int i = 0; i < K::EPT; i++) q[i] = __double2float_rn(__ddiv_rn((double)xr[i], norm));
    }
#pragma unroll
    for (int i = 0; i < K::EPT; i++) s_t[(part * K::EPT + i) * K::TV + v] = skip ? 0.0f : q[i];
  }
  __syncthreads();

  // (B) y~ = M32 n~ as a register-tiled product: thread (rg, vg) owns the blocks rg and B/2 + rg
  // (rows 4rg..4rg+3 and D/2+4rg..: a warp's matrix reads are then contiguous, free of bank
  // conflicts) of vectors VPT*vg.. and accumulates over j with fused multiply-adds.
  const int rg = tid % K::RG, vg = tid / K::RG;
  constexpr int VPT = K::VPT;
  float acc[VPT][8];
#pragma unroll
  for (int i = 0; i < VPT; i++)
#pragma unroll
    for (int r = 0; r < 8; r++) acc[i][r] = 0.0f;
#pragma unroll 2
  for (int j = 0; j < D; j++) {
    const float4 m0 = *reinterpret_cast<const float4*>(s_m + j * D + 4 * rg);
    const float4 m1 = *reinterpret_cast<const float4*>(s_m + j * D + D / 2 + 4 * rg);
    const float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float nn[VPT];
#pragma unroll
    for (int i = 0; i < VPT; i += 4) {
      const float4 t = *reinterpret_cast<const float4*>(s_t + j * K::TV + VPT * vg + i);
      nn[i] = t.x; nn[i + 1] = t.y; nn[i + 2] = t.z; nn[i + 3] = t.w;
    }
#pragma unroll
    for (int i = 0; i < VPT; i++)
#pragma unroll
      for (int r = 0; r < 8; r++) acc[i][r] = fmaf(mm[r], nn[i], acc[i][r]);
  }

  // (C) certified nearest codeword of the 2 * VPT (vector, block) pairs this thread holds
  {
    float best[2 * VPT], second[2 * VPT];
#pragma unroll
    for (int k = 0; k < 2 * VPT; k++) best[k] = second[k] = __int_as_float(0x7f800000);
    // two codewords per step (the tables hold 32 entries; those past n_codewords never win)
#pragma unroll 1
    for (int c = 0; c < n_codewords; c += 2) {
      const float4 w0 = s_cb[c], w1 = s_cb[c + 1];
      const float hn0 = s_hn[c], hn1 = s_hn[c + 1];
#pragma unroll
      for (int i = 0; i < VPT; i++)
#pragma unroll
        for (int h = 0; h < 2; h++)
          pkv_fib_top2_pair(&best[2 * i + h], &second[2 * i + h],
                            pkv_fib_key(acc[i][4 * h], acc[i][4 * h + 1], acc[i][4 * h + 2], acc[i][4 * h + 3],
                                        w0.x, w0.y, w0.z, w0.w, hn0, (uint32_t)c),
                            pkv_fib_key(acc[i][4 * h], acc[i][4 * h + 1], acc[i][4 * h + 2], acc[i][4 * h + 3],
                                        w1.x, w1.y, w1.z, w1.w, hn1, (uint32_t)c + 1u));
    }
#pragma unroll
    for (int i = 0; i < VPT; i++)
#pragma unroll
      for (int h = 0; h < 2; h++) {
        const int v = VPT * vg + i, b = h * (K::B / 2) + rg;
        s_idx[v * K::B + b] = (uint8_t)(__float_as_uint(best[2 * i + h]) & 31u);
        if (!pkv_fib_certify_eta(best[2 * i + h], second[2 * i + h], acc[i][4 * h], acc[i][4 * h + 1],
                                 acc[i][4 * h + 2], acc[i][4 * h + 3], PKV_FIB_ROT_ERR_D(D), score_abs))
          atomicOr(&s_flag[v], 1u << b);
      }
  }
  __syncthreads();

  // (D) encode_norm (:994-1020) + pack_indices (bitpack.rs:4-44); undecided work goes to the list
  for (int v = tid; v < nv; v += K::THREADS) {
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
    const uint32_t fl = s_flag[v];
    if (fl) {
      const uint32_t blocks = fl & 0x7fffffffu;
      const uint32_t which = ((fl >> 31) || (blocks & (blocks - 1))) ? PKV_FIB_ENTRY_ALL
                                                                      : (uint32_t)(__ffs(blocks) - 1);
      const uint32_t gvec = (uint32_t)((int64_t)batch * g.vpb + v0 + v);
      flag_list[atomicAdd(flag_count, 1u)] = (gvec << 5) | which;
    }
  }
  __syncthreads();
  stage_out(payload + (int64_t)batch * g.payload_batch_stride + (int64_t)v0 * rec, s_rec, nv * rec);
}

template <int D>
size_t fib_encode_fast_smem(int rec) {
  using K = FibFast<D>;
  return sizeof(float) * D * D + sizeof(float) * K::tile_floats + sizeof(float4) * 32 + sizeof(float) * 32 +
         sizeof(double) * K::TV + sizeof(int64_t) * K::TV + sizeof(uint32_t) * K::TV + K::TV +
         K::TV * K::B + (size_t)K::TV * rec + 32;
}

// The reference's exact sequence (batch numerics: normalised vector rounded to binary32,
// codec.rs:607-609) for the listed entries.  rot is the f64 matrix row-major, M[r][j].
// Phase A: single-block entries, four lanes per entry (one per row of the block), eight entries
// per warp.  Phase B: whole-vector entries, one warp per entry.
template <int D>
__global__ void __launch_bounds__(kThreads)
fib_encode_fix_kernel(PkvGeom g, const float* __restrict__ x, const double* __restrict__ rot,
                      const float* __restrict__ codebook, int n_codewords, int idx_bits, int norm_len,
                      int argmin_order, uint8_t* __restrict__ payload, const uint32_t* flag_count,
                      const uint32_t* flag_list) {
  constexpr int E = D / 32;   // elements of the vector each lane loads
  constexpr int RPL = D / 32; // rows per lane when the whole vector is redone
  constexpr int B = D / 4;
  constexpr int Q = D / 4;    // phase A: elements of the vector each of an entry's four lanes normalises
  __shared__ float s_x[kThreads / 32][D];
  __shared__ double s_n[kThreads / 32][D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nw = (gridDim.x * blockDim.x) >> 5;
  const float4* cb4 = reinterpret_cast<const float4*>(codebook);
  const uint32_t count = *flag_count;
  if (blockIdx.x == 0 && threadIdx.x == 0 && count) atomicAdd(&g_fib_stats[1], (unsigned long long)count);

  for (uint32_t base = (uint32_t)gw * 8u; base < count; base += (uint32_t)nw * 8u) {
    const int r = lane & 3;
    const uint32_t e = base + (uint32_t)(lane >> 2);
    const uint32_t ent = e < count ? flag_list[e] : PKV_FIB_ENTRY_ALL;
    const uint32_t blk = ent & 31u, gvec = ent >> 5;
    const bool act = blk != PKV_FIB_ENTRY_ALL;  // idle groups run along on vector 0, block 0, and write nothing
    const int batch = (int)(gvec / (uint32_t)g.vpb), v = (int)(gvec % (uint32_t)g.vpb);
    const float4* xv4 = reinterpret_cast<const float4*>(x + pkv_vec_offset(g.L, batch, v));
    // l2_norm: sequential over j (codec.rs:1049-1057), every lane of the group the same chain
    double acc = 0.0;
#pragma unroll 4
    for (int i = 0; i < D / 4; i++) {
      const float4 t = __ldg(xv4 + i);
      acc = __dadd_rn(acc, __dmul_rn((double)t.x, (double)t.x));
      acc = __dadd_rn(acc, __dmul_rn((double)t.y, (double)t.y));
      acc = __dadd_rn(acc, __dmul_rn((double)t.z, (double)t.z));
      acc = __dadd_rn(acc, __dmul_rn((double)t.w, (double)t.w));
    }
    double norm = __dsqrt_rn(acc);
    if (!(norm > 0.0)) norm = 1.0;  // only an idle group's stand-in vector can get here
    // lane r normalises elements Q r .. Q r + Q - 1
    float q[Q];
#pragma unroll
    for (int k4 = 0; k4 < Q / 4; k4++) {
      const float4 t = __ldg(xv4 + (Q / 4) * r + k4);
      q[4 * k4] = __double2float_rn(__ddiv_rn((double)t.x, norm));
      q[4 * k4 + 1] = __double2float_rn(__ddiv_rn((double)t.y, norm));
      q[4 * k4 + 2] = __double2float_rn(__ddiv_rn((double)t.z, norm));
      q[4 * k4 + 3] = __double2float_rn(__ddiv_rn((double)t.w, norm));
    }
    // StoredRotation::apply (rotation.rs:104-115): lane r takes row 4 blk + r, j ascending; n_j comes
    // from the lane of the group that normalised it
    const double* mrow = rot + (size_t)(4 * (act ? blk : 0u) + (uint32_t)r) * D;
    double s = 0.0;
#pragma unroll
    for (int o = 0; o < 4; o++)
#pragma unroll
      for (int k = 0; k < Q; k++) {
        const float nj = __shfl_sync(0xffffffffu, q[k], o, 4);
        s = __dadd_rn(s, __dmul_rn(__ldg(mrow + Q * o + k), (double)nj));
      }
    const float yv = __double2float_rn(s);
    const float s0 = __shfl_sync(0xffffffffu, yv, 0, 4), s1 = __shfl_sync(0xffffffffu, yv, 1, 4);
    const float s2 = __shfl_sync(0xffffffffu, yv, 2, 4), s3 = __shfl_sync(0xffffffffu, yv, 3, 4);
    if (act && r == 0) {
      const uint32_t idx = (uint32_t)nearest_codeword(cb4, n_codewords, argmin_order, s0, s1, s2, s3);
      uint8_t* rec = payload + (int64_t)batch * g.payload_batch_stride + (int64_t)v * g.rec_bytes + norm_len;
      const int pos = (int)blk * idx_bits;
      const uint32_t m = ((1u << idx_bits) - 1u) << (pos & 7), val = idx << (pos & 7);
      rec[pos >> 3] = (uint8_t)((rec[pos >> 3] & ~m) | val);
      if (m >> 8) rec[(pos >> 3) + 1] = (uint8_t)((rec[(pos >> 3) + 1] & ~(m >> 8)) | (val >> 8));
    }
  }

  for (uint32_t e = gw; e < count; e += nw) {
    const uint32_t ent = flag_list[e], blk = ent & 31u, gvec = ent >> 5;
    if (blk != PKV_FIB_ENTRY_ALL) continue;  // settled in phase A
    const int batch = (int)(gvec / (uint32_t)g.vpb), v = (int)(gvec % (uint32_t)g.vpb);
    const float* xv = x + pkv_vec_offset(g.L, batch, v);
    // the vector, then its normalised form, are shared through a per-warp slice of shared memory
    float* sx = s_x[warp];
    double* sn = s_n[warp];
    __syncwarp();
#pragma unroll
    for (int k = 0; k < E; k++) sx[lane * E + k] = xv[lane * E + k];
    __syncwarp();
    // l2_norm: sequential over j (codec.rs:1049-1057); every lane runs the same chain
    double acc = 0.0;
#pragma unroll 8
    for (int j = 0; j < D; j++) {
      const double t = (double)sx[j];
      acc = __dadd_rn(acc, __dmul_rn(t, t));
    }
    const double norm = __dsqrt_rn(acc);
#pragma unroll
    for (int k = 0; k < E; k++)
      sn[lane * E + k] = (double)__double2float_rn(__ddiv_rn((double)sx[lane * E + k], norm));
    __syncwarp();
    // StoredRotation::apply (rotation.rs:104-115): lane l takes rows l, l + 32, .., j ascending
    float yv[RPL];
#pragma unroll
    for (int rr = 0; rr < RPL; rr++) {
      const double* mrow = rot + (size_t)(lane + 32 * rr) * D;
      double s = 0.0;
#pragma unroll 8
      for (int j = 0; j < D; j++) s = __dadd_rn(s, __dmul_rn(__ldg(mrow + j), sn[j]));
      yv[rr] = __double2float_rn(s);
    }
    // nearest codeword per block, reference order; lanes with lane % 4 == 0 own a block
    uint32_t idx[RPL];
#pragma unroll
    for (int rr = 0; rr < RPL; rr++) {
      const float s1 = __shfl_down_sync(0xffffffffu, yv[rr], 1);
      const float s2 = __shfl_down_sync(0xffffffffu, yv[rr], 2);
      const float s3 = __shfl_down_sync(0xffffffffu, yv[rr], 3);
      idx[rr] = (uint32_t)nearest_codeword(cb4, n_codewords, argmin_order, yv[rr], s1, s2, s3);
    }
    uint8_t* rec = payload + (int64_t)batch * g.payload_batch_stride + (int64_t)v * g.rec_bytes + norm_len;
    {
      // block b sits in lane 4 * (b % 8), slot b / 8; lane 0 rebuilds the whole index stream
      uint8_t bytes[(B * 5 + 7) / 8 + 1];
      for (int i = 0; i < (B * idx_bits + 7) / 8; i++) bytes[i] = 0;
      for (int b = 0; b < B; b++) {
        uint32_t val = 0;
#pragma unroll
        for (int rr = 0; rr < RPL; rr++) {
          const uint32_t t = __shfl_sync(0xffffffffu, idx[rr], 4 * (b % 8));
          if (rr == b / 8) val = t;
        }
        const int pos = b * idx_bits;
        val <<= (pos & 7);
        bytes[pos >> 3] |= (uint8_t)val;
        if (val >> 8) bytes[(pos >> 3) + 1] |= (uint8_t)(val >> 8);
      }
      if (lane == 0)
        for (int i = 0; i < (B * idx_bits + 7) / 8; i++) rec[i] = bytes[i];
    }
    __syncwarp();
  }
}
