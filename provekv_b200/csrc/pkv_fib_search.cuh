// Certified nearest-codeword search of the fib-quant encoders on biased scores.
//
// Score of codeword c for the rotated block s:  F_c = |c|^2 / 2 - s . c   (|s - c|^2 = 2 F_c + |s|^2).
// The kernels keep F_c + off, with off = 1.5 * 2^k chosen on the host so that every possible score lies
// in the one binade [2^k, 2^(k+1)): |F_c| <= max_c |c|^2 / 2 + max_c |c| * |s| and |s| <= 1 for a block of
// a normalised vector, so 2^(k-1) >= 1.001 (max |c|^2 / 2 + 1.001 max |c|) suffices (fib_search_bias in
// pkv_host.cu).  Inside one binade the bit patterns of binary32 numbers differ only in their 23
// significand bits and order like the values, so
//     key = bits(F_c + off) * 32 + c   (mod 2^32)
// keeps the whole significand, carries the codeword index in its five low bits and orders, as an
// unsigned integer, first by score and then by index.  The index is merged by one integer multiply-add
// (FMA pipe) where the float keys of pkv_fib_key need a logic operation, and the four fused multiply-adds
// of a score run as packed two-lane operations on two blocks at a time: 6.1 instructions per (block,
// codeword) pair instead of 9.0, measured on the bare loop.  Used by the Hadamard encoder, whose 128
// registers per thread (four CTAs per SM) it makes possible.  The tensor-core encoders keep the float keys:
// with this form they measured slower (d = 64: 0.59 against 0.55 ms on 1.5 M vectors).
//
// Error of a kept score against the exact F_c: the start value |c|^2 / 2 + off and the four fused
// operations each round to the binade's grid, ulp_b = 2^(k-23): at most 2.5 ulp_b =: e_f.
#pragma once

struct FibSearchBias {
  float off, e_f;  // 1.5 * 2^k and 2.5 * 2^(k-23)
  // 32, handed over as a kernel argument: with the literal the compiler turns the multiply-add into a shift
  // and an add on the integer pipe, which is the pipe this form of the key is meant to relieve
  uint32_t mult;
  // exact-rotation encoders: a gap between the two best scores, in units of the binade's grid, above which
  // the best codeword is certain whatever the block (derivation beside its use)
  uint32_t quick_gap;
};

struct FibSearchTab {
  unsigned long long cbn[32][4];  // (-c_j, -c_j)
  unsigned long long hn2[32];     // (|c|^2 / 2 + off) in both lanes; past the codebook: the top of the binade
};

__device__ __forceinline__ unsigned long long pkv_pack2(float a, float b) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ unsigned long long pkv_fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ void pkv_unpack2(unsigned long long v, uint32_t& lo, uint32_t& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
}
__device__ __forceinline__ uint32_t pkv_mad_u32(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
// Keep the two smallest keys of {best, second, a, b}: the second smallest is the least of second,
// max(a, b) and max(best, min(a, b)).
__device__ __forceinline__ void pkv_top2_pair_u32(uint32_t& best, uint32_t& second, uint32_t a, uint32_t b) {
  const uint32_t lo = min(a, b), hi = max(a, b);
  const uint32_t t = max(best, lo);
  second = __vimin3_u32(second, hi, t);
  best = min(best, lo);
}

// Threads 0..31 of a CTA fill the table (entry = thread).
__device__ __forceinline__ void fib_search_fill(FibSearchTab* tab, const float* __restrict__ codebook,
                                                const float* __restrict__ half_norm, int n_codewords, float off, int c) {
  const float4 w = __ldg(reinterpret_cast<const float4*>(codebook) + c);
  const bool real = c < n_codewords;
  tab->cbn[c][0] = real ? pkv_pack2(-w.x, -w.x) : 0ull;
  tab->cbn[c][1] = real ? pkv_pack2(-w.y, -w.y) : 0ull;
  tab->cbn[c][2] = real ? pkv_pack2(-w.z, -w.z) : 0ull;
  tab->cbn[c][3] = real ? pkv_pack2(-w.w, -w.w) : 0ull;
  // off = 1.5 * 2^k: the largest number of its binade has all significand bits set
  const float top = __uint_as_float(__float_as_uint(off) | 0x007fffffu);
  const float h = real ? __fadd_rn(__ldg(half_norm + c), off) : top;
  tab->hn2[c] = pkv_pack2(h, h);
}

// The rotated values of NB consecutive blocks (NB even) starting at y[E0], as two-lane operands: lane 0
// holds block 2q, lane 1 block 2q + 1.  Callers keep only this form alive during the search (the scalar
// copy beside it would cost 4 NB more registers, which the compiler recovers by re-packing inside the loop).
template <int D, int E0, int NB>
__device__ __forceinline__ void fib_search_pack(const float (&y)[D], unsigned long long (&yp)[NB / 2][4]) {
#pragma unroll
  for (int q = 0; q < NB / 2; q++)
#pragma unroll
    for (int j = 0; j < 4; j++) yp[q][j] = pkv_pack2(y[E0 + 8 * q + j], y[E0 + 8 * q + 4 + j]);
}
// The four values of block b.
template <int NB>
__device__ __forceinline__ void fib_search_block(const unsigned long long (&yp)[NB / 2][4], int b, float (&s)[4]) {
#pragma unroll
  for (int j = 0; j < 4; j++) {
    uint32_t lo, hi;
    pkv_unpack2(yp[b >> 1][j], lo, hi);
    s[j] = __uint_as_float((b & 1) ? hi : lo);
  }
}

// Best and second-best key of the NB blocks from block B0 on (both even) of a packed row of NBT blocks.
template <int NBT, int B0, int NB>
__device__ __forceinline__ void fib_search_keys(const unsigned long long (&ypt)[NBT / 2][4], const FibSearchTab* tab,
                                                int n_codewords, uint32_t mult, uint32_t (&best)[NB],
                                                uint32_t (&second)[NB]) {
  const unsigned long long (*yp)[4] = &ypt[B0 / 2];
#pragma unroll
  for (int b = 0; b < NB; b++) best[b] = second[b] = 0xffffffffu;
  // two codewords per step (the table holds 32 entries; those past n_codewords never win)
#pragma unroll 1
  for (int c = 0; c < n_codewords; c += 2) {
    const unsigned long long a0 = tab->cbn[c][0], a1 = tab->cbn[c][1], a2 = tab->cbn[c][2], a3 = tab->cbn[c][3];
    const unsigned long long b0 = tab->cbn[c + 1][0], b1 = tab->cbn[c + 1][1], b2 = tab->cbn[c + 1][2],
                             b3 = tab->cbn[c + 1][3];
    const unsigned long long ha = tab->hn2[c], hb = tab->hn2[c + 1];
#pragma unroll
    for (int q = 0; q < NB / 2; q++) {
      const unsigned long long fa = pkv_fma2(yp[q][3], a3, pkv_fma2(yp[q][2], a2, pkv_fma2(yp[q][1], a1, pkv_fma2(yp[q][0], a0, ha))));
      const unsigned long long fb = pkv_fma2(yp[q][3], b3, pkv_fma2(yp[q][2], b2, pkv_fma2(yp[q][1], b1, pkv_fma2(yp[q][0], b0, hb))));
      uint32_t fa0, fa1, fb0, fb1;
      pkv_unpack2(fa, fa0, fa1);
      pkv_unpack2(fb, fb0, fb1);
      pkv_top2_pair_u32(best[2 * q], second[2 * q], pkv_mad_u32(fa0, mult, (uint32_t)c),
                        pkv_mad_u32(fb0, mult, (uint32_t)c + 1u));
      pkv_top2_pair_u32(best[2 * q + 1], second[2 * q + 1], pkv_mad_u32(fa1, mult, (uint32_t)c),
                        pkv_mad_u32(fb1, mult, (uint32_t)c + 1u));
    }
  }
}

// The score a key was made from.
__device__ __forceinline__ float fib_search_score(uint32_t key, float off) { return pkv_fib_key_score(key, off); }
