// cp.async helpers (global -> shared copies that bypass registers).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace k2b {

__device__ __forceinline__ void CpAsync4(void *smem_dst, const void *gmem_src) {
  unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(dst), "l"(gmem_src));
}
// Both addresses must be 16-byte aligned.
__device__ __forceinline__ void CpAsync16(void *smem_dst, const void *gmem_src) {
  unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src));
}
__device__ __forceinline__ void CpAsyncCommit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void CpAsyncWait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
// Wait until at most n (0..6) of this thread's copy groups are still in flight.
__device__ __forceinline__ void CpAsyncWaitDyn(int n) {
  switch (n) {
    case 0: CpAsyncWait<0>(); break;
    case 1: CpAsyncWait<1>(); break;
    case 2: CpAsyncWait<2>(); break;
    case 3: CpAsyncWait<3>(); break;
    case 4: CpAsyncWait<4>(); break;
    case 5: CpAsyncWait<5>(); break;
    default: CpAsyncWait<6>(); break;
  }
}

// ---- bulk (TMA) copies global -> shared, completion on an mbarrier ------------
__device__ __forceinline__ unsigned SmemAddr(const void *p) {
  return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void MbarInit(uint64_t *bar, int arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(arrivals));
}
__device__ __forceinline__ void MbarInitFence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// One arrival that also announces `bytes` of bulk-copy traffic for this phase.
__device__ __forceinline__ void MbarArriveExpectTx(uint64_t *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool MbarTryWait(uint64_t *bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(SmemAddr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false when the phase did not complete within `max_spins` polls.
__device__ __forceinline__ bool MbarWaitBounded(uint64_t *bar, unsigned parity,
                                                int max_spins = 4000000) {
  for (int spins = 0; spins < max_spins; ++spins)
    if (MbarTryWait(bar, parity)) return true;
  return false;
}
// src, dst 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void BulkCopyG2S(void *smem_dst, const void *gmem_src, unsigned bytes,
                                            uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          SmemAddr(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(SmemAddr(bar))
      : "memory");
}

}  // namespace k2b
