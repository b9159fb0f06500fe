// Shared-memory mbarrier helpers and the untiled bulk copy (global -> shared, completion on an mbarrier).
// Every wait is bounded (about one second): callers record a status code and leave on expiry.
#pragma once
#include <stdint.h>
#include <cuda_runtime.h>

namespace b200 {

constexpr long long kWaitCycles = 2000000000LL;  // ~1 s

// The status word lives in pinned host memory mapped into the device (the host reads it after draining the stream):
// a plain system-scope store, no atomic.  Any one of several codes written at once may win.
__device__ __forceinline__ void report_status(int32_t *status, int32_t code) {
  *reinterpret_cast<volatile int32_t *>(status) = code;
  __threadfence_system();
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
// bounded wait; false on expiry
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i) if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > kWaitCycles) return false;
  }
}
// Contiguous copy of `bytes` (multiple of 16; both addresses 16-byte aligned) into this CTA's shared memory.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

}  // namespace b200
