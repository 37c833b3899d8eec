// turbo-quant encode: one thread per vector, one warp per tile of 32 vectors.
//  turbo-quant/src/turbo.rs:256-288, polar.rs:246-266,413-421, rotation.rs:202-221,379-398,
//  qjl.rs:203-220, radius.rs:58-77, bitpack.rs:21-62, wire.rs:350-396
//
// The per-pair and per-projection work is written as straight-line unrolled passes without
// calls or data-dependent branches, so the compiler can interleave independent pairs; the
// decisions a shortcut could not certify are collected in bit masks and settled afterwards
// by out-of-line routines that run the exact operation sequence.
#pragma once

#include "pkv_turbo_common.cuh"

namespace pkv_turbo {

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

// Exact angle buckets for the undecided pairs `unc` of ONE vector, computed by the whole warp
// (all 32 lanes call this together).  The rotated vector is rebuilt from the input row with
// D/32 elements per lane: the butterflies pair the same elements in the same order as
// fwht_normalized (in-lane for step < D/32, by lane-xor shuffles above), so every value is
// bit-identical to the owner thread's.  Lane l then holds pairs l*D/64 .. and each pending pair
// takes atan2f + the bucket expression of polar.rs:415-420; lane 0 patches the angle words.
template <int D>
__device__ __noinline__ void fix_pairs_warp(const float* xrow, uint4 sign_mask, float scale,
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
    e[k] = __uint_as_float(__float_as_uint(xrow[i]) ^ (((mw >> (i & 31)) & 1u) << 31));
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
  while (unc) {
    const int i = __ffsll((long long)unc) - 1;
    unc &= unc - 1;
    uint32_t val = 0;
#pragma unroll
    for (int j = 0; j < E / 2; j++) {
      const uint32_t t = __shfl_sync(0xffffffffu, mine[j], i / (E / 2));
      if (j == i % (E / 2)) val = t;
    }
    if (lane == 0) patch_angle(aw, ws, i, pb, val);
  }
  __syncwarp();
}

// Which of the two encode errors applies when some radius came out non-finite: a non-finite
// input value (turbo.rs:263, checked first by the reference) or an overflow in the butterflies
// (PolarCode::from_parts, polar.rs:127-133).
__device__ __noinline__ int classify_bad_vector(const float* xrow, int dim) {
  for (int i = 0; i < dim; i++)
    if (!pkv_finite(xrow[i])) return PKV_VEC_NONFINITE_INPUT;
  return PKV_VEC_BAD_RADIUS;
}

template <int D>
struct TurboEncSmem {
  using K = Turbo<D>;
  static __host__ __device__ size_t warp_bytes(int rec_words, int lossy) {
    const size_t n = sizeof(float) * K::TV * K::XS + sizeof(int64_t) * K::TV +
                     sizeof(uint32_t) * rec_words * K::WS + (lossy ? sizeof(float) * K::P * K::WS : 0);
    return (n + 15) & ~(size_t)15;
  }
  static __host__ __device__ size_t table_bytes(int projections, int levels, int ray_count) {
    const size_t n = sizeof(float) * (projections * (K::XS + 1) + 2 * levels + 2 * ray_count);
    return (n + 15) & ~(size_t)15;
  }
};

// DIRECT (f32 radii, record a multiple of 16 bytes, angle + sign words a multiple of 4): the
// record never passes through shared memory.  Radii stay in the registers of their pairs and are
// stored by their thread as 16-byte pieces of its own record; only the few angle / sign words
// sit in a small shared tile so that the cooperative fix-up can patch them.  The staged variant
// handles every other record shape through a word-transposed tile.
template <int D, int PB, bool DIRECT>
__global__ void __launch_bounds__(Turbo<D>::THREADS, (D == 64 && DIRECT) ? 4 : 1)
turbo_encode_kernel(PkvGeom g, TurboParams tp, const float* __restrict__ x,
                    uint8_t* __restrict__ payload, uint64_t* err) {
  using K = Turbo<D>;
  extern __shared__ __align__(16) uint8_t smem[];
  const int pb = PB ? PB : tp.polar_bits;
  const int levels = 1 << pb;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* s_g = reinterpret_cast<float*>(smem);                 // [m][XS] (padded rows)
  float* s_lut = s_g + tp.projections * K::XS;                 // (cos, sin)[L], ray_cos, ray_sin
  const int lut_len = 2 * levels + 2 * tp.ray_count;
  float* s_thr = s_lut + lut_len;                              // [m] sign-shortcut thresholds
  const float* s_ray_cos = s_lut + 2 * levels;
  const float* s_ray_sin = s_ray_cos + tp.ray_count;
  const int rw = DIRECT ? 0 : tp.radii_words;  // radii words present in the shared tile
  const int tile_words = DIRECT ? tp.angle_words + tp.sign_words : tp.rec_words;
  uint8_t* wbase = smem + TurboEncSmem<D>::table_bytes(tp.projections, levels, tp.ray_count) +
                   warp * TurboEncSmem<D>::warp_bytes(tile_words, tp.lossy);
  float* s_x = reinterpret_cast<float*>(wbase);                        // [TV][XS]
  int64_t* s_off = reinterpret_cast<int64_t*>(s_x + K::TV * K::XS);    // [TV]
  uint32_t* s_w = reinterpret_cast<uint32_t*>(s_off + K::TV);          // [tile_words][WS]
  float* s_rad = reinterpret_cast<float*>(s_w + tile_words * K::WS);   // [P][WS], lossy only

  const int64_t tile_id = (int64_t)blockIdx.x * K::NWARPS + warp;
  const bool active = tile_id < (int64_t)g.n_batches * g.tiles_per_batch;
  const int tile = active ? (int)(tile_id % g.tiles_per_batch) : 0;
  const int batch = active ? (int)(tile_id / g.tiles_per_batch) : 0;
  const int v0 = tile * K::TV;
  const int nv = active ? min(K::TV, g.vpb - v0) : 0;
  const int v = lane;

  // the warp's 32 vectors: 16 lanes x 16 bytes per vector, all copies in flight at once
  if (v < nv) s_off[v] = pkv_vec_offset(g.L, batch, v0 + v);
  __syncwarp();
#pragma unroll 4
  for (int i = lane; i < nv * K::LPV; i += 32) {
    const int vv = i / K::LPV, q = i % K::LPV;
    pkv_cp_async16(s_x + vv * K::XS + 4 * q, reinterpret_cast<const float4*>(x + s_off[vv]) + q);
  }
  for (int i = threadIdx.x; i < tp.projections * K::LPV; i += K::THREADS)
    pkv_cp_async16(s_g + (i / K::LPV) * K::XS + 4 * (i % K::LPV), reinterpret_cast<const float4*>(tp.qjl) + i);
  for (int i = threadIdx.x; i < tp.projections; i += K::THREADS)
    pkv_cp_async4(s_thr + i, tp.qjl + tp.projections * D + i);
  for (int i = threadIdx.x; i < lut_len; i += K::THREADS)  // cos / sin interleaved: one 8-byte read per pair
    pkv_cp_async4(s_lut + (i < levels ? 2 * i : i < 2 * levels ? 2 * (i - levels) + 1 : i), tp.lut + i);
  pkv_cp_async_wait_all();
  __syncthreads();  // tables; the warp's own tile only needs warp-level ordering from here on

  // Every lane runs the per-vector code (lanes beyond nv work on their unused tile rows and
  // never report or get copied out), so the warp stays converged for the cooperative fix-up.
  const bool valid = v < nv;
  {
    float* row = s_x + v * K::XS;
    uint32_t* w = s_w + v;
    uint32_t* aw = w + rw * K::WS;
    uint8_t* my_rec = payload + (int64_t)batch * g.payload_batch_stride + (int64_t)(v0 + v) * g.rec_bytes;
    int code = 0;
    float y[D];
#pragma unroll
    for (int i = 0; i < D; i += 4) {
      const float4 t = *reinterpret_cast<const float4*>(row + i);
      y[i] = t.x; y[i + 1] = t.y; y[i + 2] = t.z; y[i + 3] = t.w;
    }
    // FastHadamardRotation::apply, rotation.rs:202-210.  A non-finite input makes every output of
    // the transform non-finite, so input finiteness is only looked at when a radius is bad.
    fwht_forward_signed<D>(y, tp.sgn, tp.scale);

    // Pass 1, encode_pair (polar.rs:413-421): radius exactly, bucket by the shortcut.  Radii go
    // to the record (f32 codec) or to s_rad (BlockLogU8); undecided pairs are noted in `unc`.
    float* radp = tp.lossy ? (s_rad + v) : reinterpret_cast<float*>(w);
    constexpr int NW = PB ? K::P * PB / 32 : 1;
    unsigned long long unc = 0;
    {
      uint32_t words[NW];
#pragma unroll
      for (int k = 0; k < NW; k++) words[k] = 0;
      uint64_t bitbuf = 0;
      int nbits = 0, wk = 0;
      uint32_t rmax = 0;  // radii are >= 0 or NaN: the largest bit pattern tells if any is not finite
#pragma unroll
      for (int i = 0; i < K::P; i++) {
        const float a = y[2 * i], b = y[2 * i + 1];
        const float r = __fsqrt_rn(__fadd_rn(__fmul_rn(a, a), __fmul_rn(b, b)));
        int certain = 0;
        uint32_t idx = 0;
        if (tp.fast_bucket) idx = pkv_fast_bucket_any(a, b, pb, s_ray_cos, s_ray_sin, &certain);
        unc |= (unsigned long long)(certain ? 0u : 1u) << i;
        rmax = max(rmax, __float_as_uint(r) & 0x7fffffffu);
        if constexpr (DIRECT) y[2 * i] = r;  // a and b are spent: the pair's first register keeps r
        else radp[i * K::WS] = r;
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
      if (rmax >= 0x7f800000u) code = classify_bad_vector(row, D);
    }
    if (!valid) unc = 0;
    for (unsigned pending = __ballot_sync(0xffffffffu, unc != 0); pending; pending &= pending - 1) {
      const int src = __ffs(pending) - 1;  // settle lane src's undecided pairs, all lanes helping
      const unsigned long long m =
          ((unsigned long long)__shfl_sync(0xffffffffu, (uint32_t)(unc >> 32), src) << 32) |
          __shfl_sync(0xffffffffu, (uint32_t)unc, src);
      fix_pairs_warp<D>(s_x + src * K::XS,
                        make_uint4(tp.sign_mask[0], tp.sign_mask[1], tp.sign_mask[2], tp.sign_mask[3]), tp.scale, m,
                        s_w + src + rw * K::WS, K::WS, pb, lane);
    }
    if constexpr (DIRECT) {
      if (valid) {
#pragma unroll
        for (int k = 0; k < K::P / 4; k++)
          reinterpret_cast<float4*>(my_rec)[k] = make_float4(y[8 * k], y[8 * k + 2], y[8 * k + 4], y[8 * k + 6]);
      }
    }

    if (tp.mode == PKV_TURBO_POLAR_WITH_QJL) {
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
          const float r = DIRECT ? y[2 * i] : radp[i * K::WS];
          const float2 cs = *reinterpret_cast<const float2*>(s_lut + 2 * idx);
          y[2 * i] = __fmul_rn(r, cs.x);
          y[2 * i + 1] = __fmul_rn(r, cs.y);
        }
      }
      // inverse rotation (rotation.rs:212-221), residual = vector - reconstruction (turbo.rs:268-273)
      fwht_inverse_signed<D>(y, tp.sgn_scale);
      float2 n2 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int i = 0; i < D; i += 4) {
        const float4 t = *reinterpret_cast<const float4*>(row + i);
        y[i] = __fsub_rn(t.x, y[i]);
        y[i + 1] = __fsub_rn(t.y, y[i + 1]);
        y[i + 2] = __fsub_rn(t.z, y[i + 2]);
        y[i + 3] = __fsub_rn(t.w, y[i + 3]);
        n2 = ffma2(make_float2(y[i], y[i + 1]), make_float2(y[i], y[i + 1]), n2);
        n2 = ffma2(make_float2(y[i + 2], y[i + 3]), make_float2(y[i + 2], y[i + 3]), n2);
        // the residual replaces x in the tile: the exact dot of an undecided row reads it there
        *reinterpret_cast<float4*>(row + i) = make_float4(y[i], y[i + 1], y[i + 2], y[i + 3]);
      }
      // a non-finite residual element makes the squared norm non-finite (qjl.rs:210)
      const float nsq = n2.x + n2.y;
      if (!code && !pkv_finite(nsq)) {
        bool res_ok = true;
        for (int i = 0; i < D; i++) res_ok = res_ok && pkv_finite(row[i]);
        if (!res_ok) code = PKV_VEC_NONFINITE_RESIDUAL;
      }
      // QjlQuantizer::sketch, qjl.rs:214-217: sign of the sequential f32 dot per projection row.
      // The residual rows now sit in the warp's tile, and the 32 x m dots are taken as a small
      // register-tiled product from shared memory: lane (vg, pg) owns vectors 4vg..4vg+3 and, per
      // chunk of 32 projections, rows pg, pg+4, .., pg+28 (rows 4 apart sit in different banks),
      // with packed fused multiply-adds over even / odd columns.  The sign of such a dot is the
      // reference's whenever |dot| clears the rounding bound (pkv_fast_paths.h); otherwise the
      // lane takes the exact sequential dot for that (vector, row).
      float* s_rn = reinterpret_cast<float*>(s_off);  // the vector offsets are spent
      s_rn[v] = __fmul_rn(__fsqrt_rn(nsq), 1.0001f);
      __syncwarp();
      {
        const int vg = lane >> 2, pg = lane & 3;
        const float* xr = s_x + (4 * vg) * K::XS;
        const float4 rn4 = *reinterpret_cast<const float4*>(s_rn + 4 * vg);
        const float rn[4] = {rn4.x, rn4.y, rn4.z, rn4.w};
        uint32_t* sw = s_w + (rw + tp.angle_words) * K::WS;
        for (int c = 0; c < tp.projections; c += 32) {
          const float* gr = s_g + (c + pg) * K::XS;
          float2 acc[4][8];
#pragma unroll
          for (int i = 0; i < 4; i++)
#pragma unroll
            for (int k = 0; k < 8; k++) acc[i][k] = make_float2(0.0f, 0.0f);
#pragma unroll 2
          for (int j = 0; j < D; j += 4) {
            float4 r[4];
#pragma unroll
            for (int i = 0; i < 4; i++) r[i] = *reinterpret_cast<const float4*>(xr + i * K::XS + j);
#pragma unroll
            for (int k = 0; k < 8; k++) {
              const float4 gk = *reinterpret_cast<const float4*>(gr + 4 * k * K::XS + j);
#pragma unroll
              for (int i = 0; i < 4; i++) {
                acc[i][k] = ffma2(make_float2(gk.x, gk.y), make_float2(r[i].x, r[i].y), acc[i][k]);
                acc[i][k] = ffma2(make_float2(gk.z, gk.w), make_float2(r[i].z, r[i].w), acc[i][k]);
              }
            }
          }
          uint32_t word[4];
#pragma unroll
          for (int i = 0; i < 4; i++) {
            word[i] = 0;
            uint32_t unc8 = 0;  // rows k whose sign the bound does not settle
#pragma unroll
            for (int k = 0; k < 8; k++) {
              const float dot = acc[i][k].x + acc[i][k].y;
              const float tau = fmaf(s_thr[c + pg + 4 * k], rn[i], PKV_QJL_ABS_BOUND);
              unc8 |= (fabsf(dot) > tau ? 0u : 1u) << k;
              word[i] |= (dot >= 0.0f ? 1u : 0u) << (pg + 4 * k);
            }
            if (4 * vg + i >= nv) unc8 = 0;
            while (unc8) {
              const int k = __ffs(unc8) - 1;
              unc8 &= unc8 - 1;
              const float dot = exact_dot(s_g + (c + pg + 4 * k) * K::XS, xr + i * K::XS, D);
              const uint32_t bit = 1u << (pg + 4 * k);
              word[i] = dot >= 0.0f ? (word[i] | bit) : (word[i] & ~bit);
            }
            word[i] |= __shfl_xor_sync(0xffffffffu, word[i], 1);
            word[i] |= __shfl_xor_sync(0xffffffffu, word[i], 2);
          }
          sw[(c >> 5) * K::WS + 4 * vg + pg] = pg == 0 ? word[0] : pg == 1 ? word[1] : pg == 2 ? word[2] : word[3];
        }
      }
      __syncwarp();
    }
    if (tp.lossy) {
      // CompressedRadiiV1::compress, BlockLogU8 (radius.rs:58-77), min/max after the bytes (wire.rs:368-371)
      float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
#pragma unroll 4
      for (int i = 0; i < K::P; i++) {
        float r = s_rad[i * K::WS + v];
        r = (code || !(r > PKV_FLT_MIN)) ? PKV_FLT_MIN : r;
        const float l = pkv_logf_portable(r);
        s_rad[i * K::WS + v] = l;
        mn = l < mn ? l : mn;
        mx = l > mx ? l : mx;
      }
      float span = __fsub_rn(mx, mn);
      if (!(span > PKV_FLT_EPS)) span = PKV_FLT_EPS;
#pragma unroll 2
      for (int k = 0; k < K::P / 4; k++) {
        uint32_t q4 = 0;
#pragma unroll
        for (int b = 0; b < 4; b++) {
          float nrm = __fdiv_rn(__fsub_rn(s_rad[(4 * k + b) * K::WS + v], mn), span);
          nrm = nrm < 0.0f ? 0.0f : (nrm > 1.0f ? 1.0f : nrm);
          q4 |= ((uint32_t)roundf(__fmul_rn(nrm, 255.0f)) & 0xffu) << (8 * b);
        }
        w[k * K::WS] = q4;
      }
      w[(K::P / 4) * K::WS] = __float_as_uint(mn);
      w[(K::P / 4 + 1) * K::WS] = __float_as_uint(mx);
    }
    if (valid && code) pkv_report(err, 0, (int64_t)batch * g.vpb + v0 + v, code);
    if constexpr (DIRECT) {
      if (valid) {  // angle and sign words (patched in place by the fix-ups) follow the radii
        for (int k = 0; k < tile_words; k += 4)
          *reinterpret_cast<uint4*>(my_rec + 4 * (K::P + k)) =
              make_uint4(w[k * K::WS], w[(k + 1) * K::WS], w[(k + 2) * K::WS], w[(k + 3) * K::WS]);
      }
    }
  }
  if constexpr (!DIRECT) {
    __syncwarp();
    stage_records<D, false>(
        s_w, reinterpret_cast<uint32_t*>(payload + (int64_t)batch * g.payload_batch_stride +
                                         (int64_t)v0 * g.rec_bytes),
        nv, tp.rec_words, lane);
  }
}

inline bool turbo_encode_direct(const TurboParams& tp) {
  return !tp.lossy && (tp.rec_words % 4) == 0 && ((tp.angle_words + tp.sign_words) % 4) == 0;
}

template <int D>
size_t turbo_encode_smem(const TurboParams& tp) {
  const int tile_words = turbo_encode_direct(tp) ? tp.angle_words + tp.sign_words : tp.rec_words;
  return TurboEncSmem<D>::table_bytes(tp.projections, 1 << tp.polar_bits, tp.ray_count) +
         Turbo<D>::NWARPS * TurboEncSmem<D>::warp_bytes(tile_words, tp.lossy);
}

}  // namespace pkv_turbo
