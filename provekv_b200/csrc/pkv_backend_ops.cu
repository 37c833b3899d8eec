// The two operators of the reference's gpu-backend crate that sit on the fib encode path, as stand-alone
// device calls at that crate's own boundary (gpu-backend/src/lib.rs:66-90, 196-239):
//
//   hadamard_batch(data, n, dim, seed)           in-place f32 Walsh-Hadamard transform, LCG signs, 1/sqrt(dim)
//   codebook_lookup_batch(input, codebook, ...)  nearest codeword of every k-block, f32, strict less-than scan
//
// Their arithmetic is defined by the crate's CPU code (gpu-backend/src/fallback.rs:12-62 and :254-305),
// which both kernels reproduce bit for bit.  (The crate's own .cu files are not the reference here: the
// Hadamard kernel races on its butterfly and the lookup kernel breaks ties differently from the CPU scan.)
//
// The transform is the one fib encoder that is bound by HBM and nothing else: a warp owns a vector, a lane
// dim/32 of its elements, the butterflies run in registers and across lanes by shuffles, every element is
// read once and written once.
#include <string.h>

#include "pkv_common.cuh"
#include "pkv_fast_paths.h"

namespace {

struct WhtSigns {
  uint32_t neg[32];  // bit i set: sign_i = -1 (i < padded dim <= 1024)
};

// Element i of the padded vector lives in lane (i / V) % 32, slot (i / V / 32) * V + i % V, with V =
// min(E, 4) consecutive elements per lane and load: 16-byte (8-byte for E = 2) coalesced accesses.
// A butterfly stage pairs i with i + step (bit `step` of i clear -> a + b, set -> a - b, a the element
// with the bit clear): inside a lane's V-group for step < V, across lanes (shuffle) for step < 32 V,
// across the lane's groups beyond that.  fallback.rs:34-46 runs the stages in the same order.
template <int E>
__global__ void __launch_bounds__(256, E >= 16 ? 3 : 8)
hadamard_batch_kernel(float* __restrict__ data, int64_t n, int dim, WhtSigns sg, float scale, int vec_ok) {
  constexpr int V = E < 4 ? E : 4, G = E / V;  // elements per group, groups per lane
  __shared__ uint32_t s_neg[32];
  if (threadIdx.x < 32) s_neg[threadIdx.x] = sg.neg[threadIdx.x];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t v = warp0; v < n; v += nwarps) {
    float* row = data + v * dim;
    float x[E];
#pragma unroll
    for (int gidx = 0; gidx < G; gidx++) {
      const int i0 = (gidx * 32 + lane) * V;
      if (vec_ok && i0 + V <= dim) {
        if constexpr (V == 4) {
          const float4 t = *reinterpret_cast<const float4*>(row + i0);
          x[gidx * V] = t.x; x[gidx * V + 1] = t.y; x[gidx * V + 2] = t.z; x[gidx * V + 3] = t.w;
        } else if constexpr (V == 2) {
          const float2 t = *reinterpret_cast<const float2*>(row + i0);
          x[gidx * V] = t.x; x[gidx * V + 1] = t.y;
        } else {
          x[gidx * V] = row[i0];
        }
      } else {
#pragma unroll
        for (int t = 0; t < V; t++) x[gidx * V + t] = i0 + t < dim ? row[i0 + t] : 0.0f;  // zero padding, :29-31
      }
    }
    // stages inside a group
#pragma unroll
    for (int step = 1; step < V; step <<= 1)
#pragma unroll
      for (int s = 0; s < E; s++)
        if ((s & step) == 0) {
          const float a = x[s], b = x[s + step];
          x[s] = __fadd_rn(a, b);
          x[s + step] = __fsub_rn(a, b);
        }
    // stages across lanes: the partner's element sits in the same slot of lane ^ (step / V)
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
      const bool upper = (lane & m) != 0;
#pragma unroll
      for (int s = 0; s < E; s++) {
        const float other = __shfl_xor_sync(0xffffffffu, x[s], m);
        x[s] = upper ? __fsub_rn(other, x[s]) : __fadd_rn(x[s], other);
      }
    }
    // stages across the lane's groups
#pragma unroll
    for (int gs = 1; gs < G; gs <<= 1)
#pragma unroll
      for (int gidx = 0; gidx < G; gidx++)
        if ((gidx & gs) == 0)
#pragma unroll
          for (int t = 0; t < V; t++) {
            const float a = x[gidx * V + t], b = x[(gidx + gs) * V + t];
            x[gidx * V + t] = __fadd_rn(a, b);
            x[(gidx + gs) * V + t] = __fsub_rn(a, b);
          }
    // x sign, x scale (:49-56): RN(RN(v s) scale) = s RN(v scale) for s = +-1
#pragma unroll
    for (int gidx = 0; gidx < G; gidx++) {
      const int i0 = (gidx * 32 + lane) * V;
      const uint32_t bits = s_neg[i0 >> 5] >> (i0 & 31);  // V <= 4 consecutive bits never straddle a word
#pragma unroll
      for (int t = 0; t < V; t++)
        x[gidx * V + t] = __uint_as_float(__float_as_uint(__fmul_rn(x[gidx * V + t], scale)) ^ (((bits >> t) & 1u) << 31));
      if (vec_ok && i0 + V <= dim) {
        if constexpr (V == 4)
          *reinterpret_cast<float4*>(row + i0) = make_float4(x[gidx * V], x[gidx * V + 1], x[gidx * V + 2], x[gidx * V + 3]);
        else if constexpr (V == 2)
          *reinterpret_cast<float2*>(row + i0) = make_float2(x[gidx * V], x[gidx * V + 1]);
        else
          row[i0] = x[gidx * V];
      } else {
#pragma unroll
        for (int t = 0; t < V; t++)
          if (i0 + t < dim) row[i0 + t] = x[gidx * V + t];  // truncated back to dim, :59
      }
    }
  }
}

// Padded dims 32 and 64 with 16-byte-aligned rows: LPV = dim / 4 lanes per vector, one float4 each, so a warp
// carries 32 / LPV vectors and the stages across lanes stop at LPV (half the shuffles of the layout above
// and 16-byte accesses).
template <int LPV>
__global__ void __launch_bounds__(256)
hadamard_batch_narrow_kernel(float* __restrict__ data, int64_t n, int dim, WhtSigns sg, float scale) {
  constexpr int VPW = 32 / LPV;  // vectors per warp and pass
  constexpr int U = 4;           // passes whose loads are in flight together (256 B per warp and pass alone
                                 // leaves the memory system short of requests)
  const int lane = threadIdx.x & 31, sub = lane / LPV, l = lane % LPV;
  const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const uint32_t bits = sg.neg[(4 * l) >> 5] >> ((4 * l) & 31);
  for (int64_t v0 = warp0 * (VPW * U); v0 < n; v0 += nwarps * (VPW * U)) {
    float x[U][4];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
      const int64_t v = v0 + u * VPW + sub;
      live[u] = v < n && 4 * l + 4 <= dim;  // dim is a multiple of 4 here; lanes past it hold the zero padding
      float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
      if (live[u]) t = *reinterpret_cast<const float4*>(data + v * dim + 4 * l);
      x[u][0] = t.x; x[u][1] = t.y; x[u][2] = t.z; x[u][3] = t.w;
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
      {
        const float a0 = x[u][0], b0 = x[u][1], a1 = x[u][2], b1 = x[u][3];  // step 1
        x[u][0] = __fadd_rn(a0, b0); x[u][1] = __fsub_rn(a0, b0); x[u][2] = __fadd_rn(a1, b1); x[u][3] = __fsub_rn(a1, b1);
      }
      {
        const float a0 = x[u][0], a1 = x[u][1], b0 = x[u][2], b1 = x[u][3];  // step 2
        x[u][0] = __fadd_rn(a0, b0); x[u][1] = __fadd_rn(a1, b1); x[u][2] = __fsub_rn(a0, b0); x[u][3] = __fsub_rn(a1, b1);
      }
#pragma unroll
      for (int m = 1; m < LPV; m <<= 1) {
        const bool upper = (l & m) != 0;
#pragma unroll
        for (int k = 0; k < 4; k++) {
          const float other = __shfl_xor_sync(0xffffffffu, x[u][k], m);
          x[u][k] = upper ? __fsub_rn(other, x[u][k]) : __fadd_rn(x[u][k], other);
        }
      }
#pragma unroll
      for (int k = 0; k < 4; k++)
        x[u][k] = __uint_as_float(__float_as_uint(__fmul_rn(x[u][k], scale)) ^ (((bits >> k) & 1u) << 31));
      if (live[u])
        *reinterpret_cast<float4*>(data + (v0 + u * VPW + sub) * dim + 4 * l) = make_float4(x[u][0], x[u][1], x[u][2], x[u][3]);
    }
  }
}

// Padded dims below 32: one thread per vector, the vector in local memory (not a throughput path).
__global__ void hadamard_batch_small_kernel(float* __restrict__ data, int64_t n, int dim, int pd, WhtSigns sg,
                                            float scale) {
  const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= n) return;
  float x[16];
  for (int i = 0; i < pd; i++) x[i] = i < dim ? data[v * dim + i] : 0.0f;
  for (int step = 1; step < pd; step <<= 1)
    for (int i = 0; i < pd; i += 2 * step)
      for (int j = 0; j < step; j++) {
        const float a = x[i + j], b = x[i + j + step];
        x[i + j] = __fadd_rn(a, b);
        x[i + j + step] = __fsub_rn(a, b);
      }
  for (int i = 0; i < dim; i++)
    data[v * dim + i] = __uint_as_float(__float_as_uint(__fmul_rn(x[i], scale)) ^ (((sg.neg[0] >> i) & 1u) << 31));
}

// codebook_lookup_cpu (fallback.rs:254-305) for k = 4 and at most 32 codewords: per block the squared
// distances summed in coordinate order, strict less-than scan from index 0.  One thread per 16 blocks
// (64 consecutive floats): certified top-2 search on fused scores (pkv_fast_paths.h (3), rotation error
// 0: the bounds are relative, so the input need not be normalised), and for a block the bound cannot settle
// -- or one that is not finite -- the warp evaluates the reference's own distances, lane c for codeword c.
// A distance that is not below +inf never wins the reference's scan, which then keeps index 0.
__global__ void __launch_bounds__(128, 3)
codebook_lookup_kernel(const float* __restrict__ input, int64_t n_groups, int64_t n_blocks,
                       const float* __restrict__ codebook, int n_codewords, uint32_t* __restrict__ out) {
  __shared__ float4 s_cb[32];
  __shared__ float s_hn[32];
  __shared__ float s_max[2];  // max |c|^2 / 2 and an upper bound of max |c|
  const int lane = threadIdx.x & 31;
  if (threadIdx.x < 32) {
    float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
    if ((int)threadIdx.x < n_codewords) w = __ldg(reinterpret_cast<const float4*>(codebook) + threadIdx.x);
    s_cb[threadIdx.x] = w;
    // |c|^2 / 2 in binary32: its rounding (relative 2^-23 of |c|^2 / 2) is inside the 1e-5 |F| term of the bound
    s_hn[threadIdx.x] = (int)threadIdx.x < n_codewords
                            ? __fmul_rn(0.5f, __fadd_rn(__fadd_rn(__fmul_rn(w.x, w.x), __fmul_rn(w.y, w.y)),
                                                        __fadd_rn(__fmul_rn(w.z, w.z), __fmul_rn(w.w, w.w))))
                            : 3.0e38f;
    const float h = (int)threadIdx.x < n_codewords ? s_hn[threadIdx.x] : 0.0f;
    const float hmax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(h)));  // h >= +0 (or NaN: never certain)
    if (threadIdx.x == 0) {
      s_max[0] = hmax;
      s_max[1] = __fmul_rn(PKV_FSQRT_UP(__fmul_rn(2.0f, hmax)), 1.001f);
    }
  }
  __syncthreads();
  const float hn_max = s_max[0], c_max = s_max[1];
  const int64_t g0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  // whole warps stay in the loop together (the exact tier is cooperative)
  for (int64_t base = g0 - lane; base < n_groups; base += (int64_t)gridDim.x * blockDim.x) {
    const int64_t grp = base + lane;
    const int64_t b0 = grp * 16;                                     // first block of this thread's group
    const int nb = grp < n_groups ? (int)((n_blocks - b0) < 16 ? (n_blocks - b0) : 16) : 0;
    float y[64];
#pragma unroll
    for (int b = 0; b < 16; b++) {
      const float4 t = b < nb ? __ldg(reinterpret_cast<const float4*>(input) + b0 + b) : make_float4(0.f, 0.f, 0.f, 0.f);
      y[4 * b] = t.x; y[4 * b + 1] = t.y; y[4 * b + 2] = t.z; y[4 * b + 3] = t.w;
    }
    float best[16], second[16];
#pragma unroll
    for (int b = 0; b < 16; b++) best[b] = second[b] = __int_as_float(0x7f800000);
#pragma unroll 1
    for (int c = 0; c < n_codewords; c += 2) {
      const float4 w0 = s_cb[c], w1 = s_cb[c + 1];
      const float hn0 = s_hn[c], hn1 = s_hn[c + 1];
#pragma unroll
      for (int b = 0; b < 16; b++)
        pkv_fib_top2_pair(&best[b], &second[b],
                          pkv_fib_key(y[4 * b], y[4 * b + 1], y[4 * b + 2], y[4 * b + 3], w0.x, w0.y, w0.z, w0.w, hn0,
                                      (uint32_t)c),
                          pkv_fib_key(y[4 * b], y[4 * b + 1], y[4 * b + 2], y[4 * b + 3], w1.x, w1.y, w1.z, w1.w, hn1,
                                      (uint32_t)c + 1u));
    }
    uint32_t idx[16];
    uint32_t flagged = 0;
#pragma unroll
    for (int b = 0; b < 16; b++) {
      idx[b] = __float_as_uint(best[b]) & 31u;
      // finite, moderate values only: the bound's arithmetic must not overflow or meet a NaN
      const float mag = fmaxf(fmaxf(fabsf(y[4 * b]), fabsf(y[4 * b + 1])), fmaxf(fabsf(y[4 * b + 2]), fabsf(y[4 * b + 3])));
      const bool tame = mag < 1.0e15f;  // false for NaN and infinities as well
      // rounding of the fused scores: 4 u (max |c|^2 / 2 + |s| max |c|), |s| <= 2 mag
      const float score_abs = __fmul_rn(2.41e-7f, __fmaf_rn(__fmul_rn(2.0f, mag), c_max, hn_max));
      if (b < nb && !(tame && pkv_fib_certify_eta(best[b], second[b], y[4 * b], y[4 * b + 1], y[4 * b + 2],
                                                  y[4 * b + 3], 0.0f, score_abs)))
        flagged |= 1u << b;
    }
    for (unsigned pending = __ballot_sync(0xffffffffu, flagged != 0); pending; pending &= pending - 1) {
      const int src = __ffs(pending) - 1;
      uint32_t todo = __shfl_sync(0xffffffffu, flagged, src);
      const int64_t sb0 = (base + src) * 16;
      while (todo) {
        const int b = __ffs(todo) - 1;
        todo &= todo - 1;
        const float4 s = __ldg(reinterpret_cast<const float4*>(input) + sb0 + b);
        const float4 w = s_cb[lane];
        const float d0 = __fsub_rn(s.x, w.x), d1 = __fsub_rn(s.y, w.y), d2 = __fsub_rn(s.z, w.z), d3 = __fsub_rn(s.w, w.w);
        const float dist =
            __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(0.0f, __fmul_rn(d0, d0)), __fmul_rn(d1, d1)), __fmul_rn(d2, d2)),
                      __fmul_rn(d3, d3));
        // sums of squares are >= +0 or NaN: the bit patterns of the ones below +inf order like the values
        const uint32_t key = (lane < n_codewords && dist < __int_as_float(0x7f800000)) ? __float_as_uint(dist) : 0xffffffffu;
        const uint32_t least = __reduce_min_sync(0xffffffffu, key);
        const int win = least == 0xffffffffu ? 0 : __ffs(__ballot_sync(0xffffffffu, key == least)) - 1;
        if (lane == src) {
#pragma unroll
          for (int k = 0; k < 16; k++)
            if (k == b) idx[k] = (uint32_t)win;
        }
      }
    }
#pragma unroll
    for (int b = 0; b < 16; b += 4)
      if (b + 4 <= nb) {
        *reinterpret_cast<uint4*>(out + b0 + b) = make_uint4(idx[b], idx[b + 1], idx[b + 2], idx[b + 3]);
      } else {
#pragma unroll
        for (int t = 0; t < 4; t++)
          if (b + t < nb) out[b0 + b + t] = idx[b + t];
      }
  }
}

int sm_count() {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

}  // namespace

extern "C" int pkv_hadamard_batch_dev(float* data_dev, int64_t n, int32_t dim, uint64_t seed, void* stream) {
  if (!data_dev || n < 0 || dim <= 0) return PKV_ERR_INVALID_ARGUMENT;
  if ((uintptr_t)data_dev & 3) return PKV_ERR_INVALID_ARGUMENT;
  if (n == 0) return PKV_OK;
  int pd = 1;
  while (pd < dim) pd <<= 1;  // dim.next_power_of_two(), fallback.rs:14
  if (pd > 1024) return PKV_ERR_UNSUPPORTED;
  WhtSigns sg;
  memset(&sg, 0, sizeof(sg));
  uint64_t state = seed;  // generate_signs_impl, fallback.rs:76-88
  for (int i = 0; i < pd; i++) {
    state = state * 6364136223846793005ull + 1442695040888963407ull;
    if (((state >> 32) & 1) == 0) sg.neg[i >> 5] |= 1u << (i & 31);
  }
  const float scale = 1.0f / sqrtf((float)pd);
  cudaStream_t s = (cudaStream_t)stream;
  if (pd < 32) {
    const int64_t blocks = (n + 127) / 128;
    if (blocks > 0x7fffffff) return PKV_ERR_UNSUPPORTED;
    hadamard_batch_small_kernel<<<(unsigned)blocks, 128, 0, s>>>(data_dev, n, dim, pd, sg, scale);
  } else {
    // vector accesses need every row to start on a 16-byte boundary
    const int vec_ok = (dim % 4 == 0) && (((uintptr_t)data_dev & 15) == 0);
    const int64_t want = (n + 7) / 8;  // 8 warps per CTA
    const int64_t cap = (int64_t)sm_count() * 8;
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    if (vec_ok && pd <= 64) {
      const int vpw = pd == 64 ? 2 : 4;
      const int64_t want_n = (n + 8 * vpw * 4 - 1) / (8 * vpw * 4);  // 8 warps x vpw vectors x 4 passes per CTA and round
      const unsigned grid_n = (unsigned)(want_n < cap ? want_n : cap);
      if (pd == 64) hadamard_batch_narrow_kernel<16><<<grid_n, 256, 0, s>>>(data_dev, n, dim, sg, scale);
      else hadamard_batch_narrow_kernel<8><<<grid_n, 256, 0, s>>>(data_dev, n, dim, sg, scale);
    } else
    switch (pd / 32) {
      case 1: hadamard_batch_kernel<1><<<grid, 256, 0, s>>>(data_dev, n, dim, sg, scale, 0); break;
      case 2: hadamard_batch_kernel<2><<<grid, 256, 0, s>>>(data_dev, n, dim, sg, scale, vec_ok || (dim % 2 == 0 && ((uintptr_t)data_dev & 7) == 0)); break;
      case 4: hadamard_batch_kernel<4><<<grid, 256, 0, s>>>(data_dev, n, dim, sg, scale, vec_ok); break;
      case 8: hadamard_batch_kernel<8><<<grid, 256, 0, s>>>(data_dev, n, dim, sg, scale, vec_ok); break;
      case 16: hadamard_batch_kernel<16><<<grid, 256, 0, s>>>(data_dev, n, dim, sg, scale, vec_ok); break;
      default: hadamard_batch_kernel<32><<<grid, 256, 0, s>>>(data_dev, n, dim, sg, scale, vec_ok); break;
    }
  }
  pkv_count_launch();
  return pkv_cuda_status(cudaGetLastError());
}

extern "C" int pkv_codebook_lookup_batch_dev(const float* input_dev, const float* codebook_dev, int64_t n, int32_t dim,
                                             int32_t k, int32_t n_codewords, uint32_t* indices_dev, void* stream) {
  if (!input_dev || !codebook_dev || !indices_dev || n < 0 || dim <= 0 || k <= 0 || n_codewords < 1)
    return PKV_ERR_INVALID_ARGUMENT;
  if (dim % k) return PKV_ERR_INVALID_ARGUMENT;  // "dim must be divisible by k", fallback.rs:267-272
  if (k != 4 || n_codewords > 32) return PKV_ERR_UNSUPPORTED;
  if (((uintptr_t)input_dev | (uintptr_t)codebook_dev | (uintptr_t)indices_dev) & 15) return PKV_ERR_INVALID_ARGUMENT;
  const int64_t n_blocks = n * (dim / 4);
  if (n_blocks == 0) return PKV_OK;
  const int64_t n_groups = (n_blocks + 15) / 16;
  const int64_t want = (n_groups + 127) / 128;
  const int64_t cap = (int64_t)sm_count() * 3 * 8;
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  codebook_lookup_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(input_dev, n_groups, n_blocks, codebook_dev,
                                                                 n_codewords, indices_dev);
  pkv_count_launch();
  return pkv_cuda_status(cudaGetLastError());
}
