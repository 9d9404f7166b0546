// Device-side plumbing shared by the kernels: shared-memory addressing,
// mbarrier waits with an iteration limit, 1-D bulk (TMA) copies global->shared
// without multicast, and small block-wide reductions.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace aot {

// Error word bits written by kernels instead of trapping.
enum DevErr : int { DEVERR_MBAR_TIMEOUT = 1, DEVERR_BAD_ARGS = 2, DEVERR_GRID_TIMEOUT = 4 };

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Wait for phase `parity` with an iteration limit. On expiry the error word is
// set and false is returned; the caller leaves its loop and the kernel returns
// normally (its copies in flight are bounded by the barrier's own transaction
// count, the context stays usable).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  if (err) atomicOr(err, DEVERR_MBAR_TIMEOUT);
  return false;
}

// cp.async.bulk global -> shared::cta of this CTA, completion on `bar`.
// dst, src 16-byte aligned; bytes a multiple of 16. No multicast.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}

// Copy the byte range [src, src+len) so that it lands at `slot + (src & 15)`:
// the aligned superset [src & ~15, roundup16(src+len)) is what is transferred,
// which keeps both addresses 16-byte aligned for any 2- or 4-byte aligned row.
// Returns the number of bytes the barrier must expect. The weights allocation
// is padded so the superset never leaves it.
__device__ __forceinline__ uint32_t bulk_superset_bytes(const void* src, uint32_t len) {
  uint32_t mis = (uint32_t)((uintptr_t)src & 15u);
  return (mis + len + 15u) & ~15u;
}
__device__ __forceinline__ void bulk_g2s_superset(void* slot, const void* src, uint32_t len, uint64_t* bar) {
  uintptr_t a = (uintptr_t)src & ~(uintptr_t)15;
  bulk_g2s(slot, (const void*)a, bulk_superset_bytes(src, len), bar);
}

__device__ __forceinline__ uint32_t funnel_r(uint32_t lo, uint32_t hi, uint32_t shift_bits) {
  return __funnelshift_r(lo, hi, shift_bits);
}

// Programmatic dependent launch: let the next kernel in the stream start its
// prologue, and wait for everything the previous kernel wrote.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

}  // namespace aot
