// Thin wrappers over the sm_100a tensor-core instructions used by the turbo-quant encoder's QJL
// product: tensor-memory allocation, one-CTA TF32 matrix multiply-accumulate from shared-memory
// descriptors, completion through an mbarrier, and the accumulator read-back.
//
// Operand tiles use the K-major layout with the 128-byte swizzle: a tile of R rows x K f32 is
// stored as K/32 slabs of [R rows][128 bytes]; inside each group of 8 rows (1024 bytes, aligned to
// 1024) the 16-byte piece j of row r sits at r * 128 + ((j ^ (r & 7)) * 16).  A descriptor points
// at the first row; consecutive K steps of 8 elements advance the start address by 32 bytes.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace pkv_tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// Byte offset of the 16-byte piece c (elements 4c..4c+3) of row r in a swizzled tile whose slabs
// are slab_bytes apart.
__device__ __forceinline__ uint32_t sw_piece(int slab_bytes, int r, int c) {
  return (uint32_t)((c >> 3) * slab_bytes + (r >> 3) * 1024 + (r & 7) * 128 + (((c & 7) ^ (r & 7)) << 4));
}
// element j of row r
__device__ __forceinline__ const float* tile_at(const uint8_t* t, int slab_bytes, int r, int j) {
  return reinterpret_cast<const float*>(t + sw_piece(slab_bytes, r, j >> 2) + (j & 3) * 4);
}

// Shared-memory matrix descriptor (sm_100 format) for that layout: start address in units of 16
// bytes in bits 0-13, leading offset (unused with a swizzle; 1) in bits 16-29, stride offset
// between 8-row groups (1024 bytes, in units of 16) in bits 32-45, descriptor version 1 in bits
// 46-47, layout type 2 (128-byte swizzle) in bits 61-63.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}

// Instruction descriptor for kind::tf32: f32 accumulator (bits 4-5 = 1), A and B in TF32
// (bits 7-9, 10-12 = 2), both K-major (bits 15, 16 = 0), N / 8 in bits 17-22, M / 16 in bits 24-28.
__host__ __device__ constexpr uint32_t idesc_tf32(int m, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Allocate `cols` (power of two, >= 32) tensor-memory columns; the base address lands in *slot.
// Whole-warp call; the same warp frees the columns with tmem_free.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}

__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Shared-memory writes made with ordinary stores become visible to the tensor core's reads.
__device__ __forceinline__ void fence_smem_to_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T for one K step of 8 TF32 elements; single-thread issue.
__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

// The KSTEPS K steps of one product A B^T, operands in the tile layout above with slabs a_slab / b_slab
// bytes apart.  The descriptors of the steps differ from the first one by constants (the start-address
// field counts 16-byte units), so the unrolled chain costs two 64-bit additions per step; rebuilding the
// descriptor in a rolled loop made the lone issuing thread spend about 140 cycles per step on dependent
// scalar code, more than the tensor cores need for the step itself.
template <int KSTEPS>
__device__ __forceinline__ void mma_tf32_chain(uint32_t tmem_d, uint32_t a_addr, uint32_t a_slab, uint32_t b_addr,
                                               uint32_t b_slab, uint32_t idesc, bool accumulate_first) {
  const uint64_t da0 = smem_desc_sw128(a_addr), db0 = smem_desc_sw128(b_addr);
#pragma unroll
  for (int k = 0; k < KSTEPS; k++) {
    const uint64_t da = da0 + (uint64_t)(((uint32_t)(k >> 2) * a_slab + (uint32_t)(k & 3) * 32u) >> 4);
    const uint64_t db = db0 + (uint64_t)(((uint32_t)(k >> 2) * b_slab + (uint32_t)(k & 3) * 32u) >> 4);
    mma_tf32(tmem_d, da, db, idesc, (k > 0 || accumulate_first) ? 1u : 0u);
  }
}

// The barrier gets one arrival when every multiply issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Bounded wait for the barrier phase `parity`; false if it never completed within `limit` polls.
constexpr int kWaitPolls = 1 << 20;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int limit = kWaitPolls) {
  const uint32_t a = smem_u32(bar);
  for (int it = 0; it < limit; it++) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok)
        : "r"(a), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// 32 consecutive accumulator columns of this thread's tensor-memory lane (lane = 32 * (warp % 4)
// + lane id); whole-warp call.
__device__ __forceinline__ void tmem_load32(uint32_t taddr, float (&d)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  // the registers are listed as operands so that no use of them can move above the wait
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
#pragma unroll
  for (int i = 0; i < 32; i++) d[i] = __uint_as_float(r[i]);
}

// N = 4 or 8 consecutive accumulator columns of this thread's tensor-memory lane; whole-warp call.
template <int N>
__device__ __forceinline__ void tmem_load(uint32_t taddr, float (&d)[N]) {
  static_assert(N == 4 || N == 8, "column count");
  uint32_t r[N];
  if constexpr (N == 8) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
                 :
                 : "memory");
  } else {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]) : : "memory");
  }
#pragma unroll
  for (int i = 0; i < N; i++) d[i] = __uint_as_float(r[i]);
}

}  // namespace pkv_tc
