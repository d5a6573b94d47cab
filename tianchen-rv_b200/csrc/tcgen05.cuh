// Inline-PTX wrappers for the Blackwell tensor-core path: tensor memory (TMEM) allocation,
// tcgen05.mma with shared-memory operand descriptors, tcgen05.commit onto an mbarrier,
// tcgen05.ld for the epilogue, and tiled TMA loads (cp.async.bulk.tensor, no multicast).
#pragma once

#include <cuda.h>
#include <stdint.h>

#include "async_copy.cuh"

namespace tcrv {

// ---- TMA: 2-D tiled load global -> shared, completion counted on an mbarrier.
// The innermost coordinate (x) times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(void *dst_smem, const CUtensorMap *map, int x, int y, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_addr(dst_smem)),
      "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// ---- TMEM allocation (one full warp executes these)
__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(dst_smem)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_alloc_permit() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before_thread_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after_thread_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- shared-memory matrix descriptor, K-major operand, 128-byte swizzle.
// Rows are 128 bytes apart inside an 8-row swizzle atom (1024 bytes); atoms of 8 rows follow
// one another every 1024 bytes (the stride byte offset).  The tile base must be 1024-byte
// aligned; a K step of 32 bytes inside the 128-byte row advances the start address by 32.
__device__ __forceinline__ uint64_t umma_desc_k_major_sw128(uint32_t smem_byte_addr) {
  uint64_t desc = 0;
  desc |= static_cast<uint64_t>((smem_byte_addr & 0x3ffffu) >> 4);  // start address, bits [0,14)
  desc |= static_cast<uint64_t>(1) << 16;                           // leading byte offset (unused here)
  desc |= static_cast<uint64_t>(1024 >> 4) << 32;                   // stride byte offset, bits [32,46)
  desc |= static_cast<uint64_t>(1) << 46;                           // descriptor version (Blackwell)
  desc |= static_cast<uint64_t>(2) << 61;                           // layout type: SWIZZLE_128B
  return desc;
}

// ---- instruction descriptor for kind::i8: signed int8 A and B, both K-major, int32 D.
__host__ __device__ constexpr uint32_t umma_idesc_s8(int m, int n) {
  return (2u << 4)                                 // D format: S32
         | (1u << 7)                               // A: signed 8-bit
         | (1u << 10)                              // B: signed 8-bit
         | (static_cast<uint32_t>(n >> 3) << 17)   // N / 8
         | (static_cast<uint32_t>(m >> 4) << 24);  // M / 16
}

// D[tmem] = A[smem] * B[smem] (kAccumulate false) or D += A * B.  One thread issues.
template <bool kAccumulate>
__device__ __forceinline__ void umma_s8_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "n"(kAccumulate ? 1 : 0)
      : "memory");
}

// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
               : "memory");
}

// ---- instruction descriptor for kind::f8f6f4 with e4m3 A and B (format code 0), both K-major,
// fp32 D.
__host__ __device__ constexpr uint32_t umma_idesc_e4m3(int m, int n) {
  return (1u << 4)                                 // D format: F32
         | (static_cast<uint32_t>(n >> 3) << 17)   // N / 8
         | (static_cast<uint32_t>(m >> 4) << 24);  // M / 16
}

template <bool kAccumulate>
__device__ __forceinline__ void umma_f8_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "n"(kAccumulate ? 1 : 0)
      : "memory");
}

// 32 lanes x N consecutive 32-bit columns (N = 16 or 32): thread i of the warp receives lane
// (base+i).
template <int N>
__device__ __forceinline__ void tmem_ld_32x32b(uint32_t taddr, uint32_t (&v)[N]);

template <>
__device__ __forceinline__ void tmem_ld_32x32b<32>(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

template <>
__device__ __forceinline__ void tmem_ld_32x32b<16>(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace tcrv
