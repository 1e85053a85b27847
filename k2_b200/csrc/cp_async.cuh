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

}  // namespace k2b
