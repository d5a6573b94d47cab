// Thin wrappers over the sm_90+/sm_100 asynchronous-copy PTX used by the streaming kernels:
// mbarrier objects in shared memory and the 1-D bulk copy engine (cp.async.bulk), which
// moves a contiguous, 16-byte-aligned byte range global -> shared and signals an mbarrier
// with the number of bytes written.  Every wait is bounded: a caller that sees `false`
// records an error and leaves instead of spinning forever.
#pragma once

#include <stdint.h>

namespace tcrv {

__device__ __forceinline__ uint32_t smem_addr(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t arrive_count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrive_count) : "memory");
}

// Makes barrier initialisation visible to the async proxy (the copy engine).
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// The same test with a suspend-time hint: the thread may sleep in hardware for up to `hint_ns`
// and is woken when the phase completes, instead of returning at once.  A waiter that spins on
// the plain form re-reads the barrier word every few cycles; with many warps waiting on one
// barrier those reads compete with the arrivals on the same word and with the other warps'
// issue slots.
__device__ __forceinline__ bool mbar_try_wait_suspend(uint64_t *bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity), "r"(hint_ns)
      : "memory");
  return done != 0;
}

// Bounded wait for the phase with the given parity: gives up after kMbarTimeoutNs of wall
// time, far beyond any legitimate wait of these kernels (microseconds).  Each poll may sleep up
// to kMbarSuspendNs in hardware (see mbar_try_wait_suspend); the global nanosecond timer is
// read every 16 polls.  `abort_flag`, when given, is a shared-memory word another role sets
// after its own wait failed, so that the whole CTA leaves promptly.
constexpr uint64_t kMbarTimeoutNs = 2000000000ull;
constexpr uint32_t kMbarSuspendNs = 20000u;

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity,
                                                  volatile uint32_t *abort_flag = nullptr) {
  if (mbar_try_wait(bar, parity))
    return true;
  uint64_t start = 0;
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait_suspend(bar, parity, kMbarSuspendNs))
      return true;
    if ((i & 15u) == 0) {
      if (abort_flag != nullptr && *abort_flag != 0)
        return false;
      const uint64_t now = global_timer_ns();
      if (start == 0)
        start = now;
      else if (now - start > kMbarTimeoutNs)
        return false;
    }
  }
}

// global -> shared bulk copy; dst, src and bytes must be multiples of 16.
__device__ __forceinline__ void bulk_copy_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes,
                                              uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_addr(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
      : "memory");
}

}  // namespace tcrv
