// turbo-quant decode fused with the write into the KV cache.
//  turbo-quant/src/wire.rs:497-565 (per-vector record), radius.rs:81-147,
//  polar.rs:286-316 (dequantise angle, r cos / r sin), rotation.rs:170-194 (inverse FWHT, signs)
#pragma once

#include "pkv_turbo_common.cuh"

namespace pkv_turbo {

template <int D>
struct TurboDecSmem {  // per-warp slices follow the CTA-wide tables
  using K = Turbo<D>;
  static __host__ __device__ size_t warp_bytes(int rec_words) {
    // the f32 output tile reuses the record tile's space (records are in registers by then)
    const size_t tile = sizeof(float) * K::TV * K::XS, recs = sizeof(uint32_t) * rec_words * K::WS;
    const size_t n = (tile > recs ? tile : recs) + sizeof(int64_t) * K::TV;
    return (n + 15) & ~(size_t)15;  // the next warp's f32 tile stays 16-byte aligned
  }
  static __host__ __device__ size_t table_bytes(int levels) { return sizeof(float) * (256 + 2 * levels); }
};

// RAW != 0 (f32 radii, fixed angle width): the warp's run of records is copied as it lies with 16-byte
// copies.  RAW == 1 (records a multiple of 16 bytes): every lane reads its own record with 16-byte
// loads into registers (consecutive 144-byte records start 9 sixteen-byte units apart: the lanes of a
// quarter-warp hit distinct bank groups).  RAW == 2 (an odd number of words per record, e.g. 71): the
// lane reads its words one by one, conflict-free because the record stride is odd.  RAW == 0: the
// records go through a word-transposed tile, 4 bytes per copy.
template <int D, int PB, int DST, int RAW>
__global__ void __launch_bounds__(Turbo<D>::THREADS)
turbo_decode_patch_kernel(PkvGeom g, TurboParams tp, const uint8_t* __restrict__ payload,
                          typename PkvDst<DST>::type* __restrict__ cache, uint64_t* err) {
  using K = Turbo<D>;
  extern __shared__ __align__(128) uint8_t smem[];
  const int pb = PB ? PB : tp.polar_bits;
  const int levels = 1 << pb;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* s_q255 = reinterpret_cast<float*>(smem);  // [256]
  float* s_lut = s_q255 + 256;                     // (cos, sin)[L]
  uint8_t* wbase = smem + TurboDecSmem<D>::table_bytes(levels) + warp * TurboDecSmem<D>::warp_bytes(tp.rec_words);
  int64_t* s_off = reinterpret_cast<int64_t*>(wbase);                 // [TV]
  uint32_t* s_w = reinterpret_cast<uint32_t*>(s_off + K::TV);         // [rec_words][WS]
  float* s_x = reinterpret_cast<float*>(s_w);                         // [TV][XS], after the records are consumed

  const int64_t tile_id = (int64_t)blockIdx.x * K::NWARPS + warp;
  const bool active = tile_id < (int64_t)g.n_batches * g.tiles_per_batch;
  const int tile = active ? (int)(tile_id % g.tiles_per_batch) : 0;
  const int batch = active ? (int)(tile_id / g.tiles_per_batch) : 0;
  const int v0 = tile * K::TV;
  const int nv = active ? min(K::TV, g.vpb - v0) : 0;
  const int v = lane;

  const uint8_t* src = payload + (int64_t)batch * g.payload_batch_stride + (int64_t)v0 * g.rec_bytes;
  // RAW: the warp's run of records is contiguous and starts on a 16-byte boundary (32 records are a
  // multiple of 16 bytes): one bulk copy signalling the warp's mbarrier when the run is a multiple of
  // 16 bytes long, 16- and 4-byte copies for the ragged last run otherwise
  __shared__ __align__(8) uint64_t s_bar[Turbo<D>::NWARPS];
  bool bulk = false;
  if constexpr (RAW != 0) {
    const int nw = nv * tp.rec_words, n16 = nw / 4;
    bulk = nv > 0 && (nw & 3) == 0;
    if (bulk) {
      if (lane == 0) {
        pkv_mbar_init(&s_bar[warp], 1);
        pkv_mbar_expect_tx(&s_bar[warp], (uint32_t)nw * 4u);
        pkv_bulk_load(s_w, src, (uint32_t)nw * 4u, &s_bar[warp]);
      }
    } else {
      for (int i = lane; i < n16; i += 32)
        pkv_cp_async16(reinterpret_cast<uint4*>(s_w) + i, reinterpret_cast<const uint4*>(src) + i);
      for (int i = 4 * n16 + lane; i < nw; i += 32) pkv_cp_async4(s_w + i, reinterpret_cast<const uint32_t*>(src) + i);
    }
  } else {
    stage_records<D, true>(s_w, reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(src)), nv, tp.rec_words, lane);
  }
  for (int i = threadIdx.x; i < 2 * levels; i += K::THREADS)  // interleaved: one 8-byte read per pair
    pkv_cp_async4(s_lut + (i < levels ? 2 * i : 2 * (i - levels) + 1), tp.lut + i);
  if (tp.lossy)  // `*value as f32 / u8::MAX as f32`, radius.rs:143
    for (int i = threadIdx.x; i < 256; i += K::THREADS) s_q255[i] = __fdiv_rn((float)i, 255.0f);
  if (v < nv) s_off[v] = pkv_dst_offset(g, batch, v0 + v, DST == PKV_DST_F32 ? 4 : 8, err);
  pkv_cp_async_wait_all();
  __syncthreads();  // tables; the warp's own tile only needs warp-level ordering from here on
  if (bulk) {
    __syncwarp();
    if (!__all_sync(0xffffffffu, pkv_mbar_wait(&s_bar[warp], 0))) {  // never completed: nothing is decoded
      if (lane == 0) pkv_report(err, 0, (int64_t)batch * g.vpb + v0, PKV_VEC_DEVICE_WAIT);
      return;
    }
  }

  float y[D];
  if (v < nv) {
    // word k of this lane's record (k is a compile-time constant wherever RAW is used)
    constexpr int RW = RAW == 1 ? ((K::P + K::P * (PB ? PB : 1) / 32 + 3) & ~3) : 4;
    uint32_t rw[RW];
    if constexpr (RAW == 1) {
      const uint4* w4 = reinterpret_cast<const uint4*>(s_w + v * tp.rec_words);
#pragma unroll
      for (int k = 0; k < RW / 4; k++) {
        const uint4 u = w4[k];  // the last piece may reach into the sign words, which decode ignores
        rw[4 * k] = u.x; rw[4 * k + 1] = u.y; rw[4 * k + 2] = u.z; rw[4 * k + 3] = u.w;
      }
    }
    const uint32_t* wt = s_w + v;
    const uint32_t* wr = s_w + v * tp.rec_words;
    auto w = [&](int k) -> uint32_t {
      if constexpr (RAW == 1) return rw[k];
      else if constexpr (RAW == 2) return wr[k];
      else return wt[k * K::WS];
    };
    int code = 0;
    // radii -> y[2i] (temporarily)
    if (!tp.lossy) {
      uint32_t bad = 0;
#pragma unroll
      for (int i = 0; i < K::P; i++) {
        const uint32_t u = w(i);
        // finite and non-negative (radius.rs:98-103): sign clear and exponent not all ones
        bad |= (u >> 31) | (uint32_t)((u & 0x7f800000u) == 0x7f800000u);
        y[2 * i] = __uint_as_float(u);
      }
      // -0.0 has the sign bit set but passes `value < 0.0`; re-check exactly when flagged
      if (bad) {
#pragma unroll
        for (int i = 0; i < K::P; i++) {
          const float r = __uint_as_float(w(i));
          if (!code && (!pkv_finite(r) || r < 0.0f)) code = PKV_VEC_BAD_RADIUS;
        }
      }
    } else {
      const float mn = __uint_as_float(wt[(K::P / 4) * K::WS]);
      const float mx = __uint_as_float(wt[(K::P / 4 + 1) * K::WS]);
      if (!pkv_finite(mn) || !pkv_finite(mx) || mn > mx) code = PKV_VEC_BAD_RADIUS_RANGE;
      const float span = __fsub_rn(mx, mn);
#pragma unroll
      for (int k = 0; k < K::P / 4; k++) {
        const uint32_t q4 = wt[k * K::WS];
#pragma unroll
        for (int b = 0; b < 4; b++) {
          const float t = __fadd_rn(mn, __fmul_rn(span, s_q255[(q4 >> (8 * b)) & 0xffu]));
          const float r = code ? 0.0f : pkv_ulp_adjust(tp.expf_table, t, pkv_expf_portable(t));
          if (!code && !pkv_finite(r)) code = PKV_VEC_BAD_RADIUS;  // polar.rs:127-133
          y[2 * (4 * k + b)] = r;
        }
      }
    }
    // angle indices (LSB-first stream, bitpack.rs:135-153) and the polar -> cartesian step
    const uint32_t* aw = wt + tp.radii_words * K::WS;
    const uint32_t mask = (uint32_t)levels - 1u;
    if constexpr (PB != 0) {
      constexpr int NW = K::P * PB / 32;
      uint32_t words[NW];
#pragma unroll
      for (int k = 0; k < NW; k++) words[k] = RAW != 0 ? w(K::P + k) : aw[k * K::WS];
#pragma unroll
      for (int i = 0; i < K::P; i++) {
        const int pos = i * PB, wi = pos >> 5, sh = pos & 31;
        uint32_t idx = words[wi] >> sh;
        if (sh + PB > 32) idx |= words[wi + 1] << (32 - sh);
        idx &= mask;
        const float r = y[2 * i];
        const float2 cs = *reinterpret_cast<const float2*>(s_lut + 2 * idx);
        y[2 * i] = cs.x;
        y[2 * i + 1] = cs.y;
        mul2(y[2 * i], y[2 * i + 1], r, r);  // (r * theta.cos(), r * theta.sin()), polar.rs:312-313
      }
    } else {
      uint64_t bitbuf = 0;
      int nbits = 0, wk = 0;
#pragma unroll
      for (int i = 0; i < K::P; i++) {
        if (nbits < pb) {
          bitbuf |= (uint64_t)aw[wk * K::WS] << nbits;
          wk++;
          nbits += 32;
        }
        const uint32_t idx = (uint32_t)bitbuf & mask;
        bitbuf >>= pb;
        nbits -= pb;
        const float r = y[2 * i];
        const float2 cs = *reinterpret_cast<const float2*>(s_lut + 2 * idx);
        y[2 * i] = cs.x;
        y[2 * i + 1] = cs.y;
        mul2(y[2 * i], y[2 * i + 1], r, r);
      }
    }
    if (code) pkv_report(err, 0, (int64_t)batch * g.vpb + v0 + v, code);
    // FastHadamardRotation::apply_inverse, rotation.rs:212-221
    fwht_inverse_signed<D>(y, tp.sgn_scale);
  }
  __syncwarp();  // every lane has consumed its record: the tile may now hold the f32 rows
  if (v < nv) {
    float* row = s_x + v * K::XS;
#pragma unroll
    for (int i = 0; i < D; i += 4)
      *reinterpret_cast<float4*>(row + i) = make_float4(y[i], y[i + 1], y[i + 2], y[i + 3]);
  }
  __syncwarp();

  if constexpr (DST == PKV_DST_F32) {
    // coalesced write-out: D/4 lanes per vector, one float4 each, every replica
#pragma unroll 4
    for (int i = lane; i < nv * K::LPV; i += 32) {
      const int vv = i / K::LPV, q = i % K::LPV;
      if (s_off[vv] == PKV_SKIP_DST) continue;
      const float4 val = *reinterpret_cast<const float4*>(s_x + vv * K::XS + 4 * q);
      float* dst = cache + s_off[vv] + 4 * q;
      for (int r = 0; r < g.L.n_replicas; r++) {
        *reinterpret_cast<float4*>(dst) = val;
        dst += g.L.replica_stride;
      }
    }
  } else {
    // 16-bit cache: D/8 lanes per vector, eight values rounded to nearest-even and stored as 16 bytes
    constexpr int LPH = D / 8;
#pragma unroll 4
    for (int i = lane; i < nv * LPH; i += 32) {
      const int vv = i / LPH, q = i % LPH;
      if (s_off[vv] == PKV_SKIP_DST) continue;
      const float4 a = *reinterpret_cast<const float4*>(s_x + vv * K::XS + 8 * q);
      const float4 b = *reinterpret_cast<const float4*>(s_x + vv * K::XS + 8 * q + 4);
      const uint4 val = make_uint4(pkv_pack2<DST>(a.x, a.y), pkv_pack2<DST>(a.z, a.w),
                                   pkv_pack2<DST>(b.x, b.y), pkv_pack2<DST>(b.z, b.w));
      typename PkvDst<DST>::type* dst = cache + s_off[vv] + 8 * q;
      for (int r = 0; r < g.L.n_replicas; r++) {
        *reinterpret_cast<uint4*>(dst) = val;
        dst += g.L.replica_stride;
      }
    }
  }
}

inline int turbo_decode_raw(const TurboParams& tp, int pb_template) {
  if (pb_template == 0 || tp.lossy) return 0;
  return (tp.rec_words % 4) == 0 ? 1 : (tp.rec_words & 1) ? 2 : 0;
}

template <int D>
size_t turbo_decode_smem(const TurboParams& tp) {
  return TurboDecSmem<D>::table_bytes(1 << tp.polar_bits) +
         Turbo<D>::NWARPS * TurboDecSmem<D>::warp_bytes(tp.rec_words);
}

}  // namespace pkv_turbo
