// mbarrier and bulk-async-copy wrappers shared by the tensor-core GEMMs and the staged LayerNorm
// kernels.  Waits are bounded: they give up after a cycle limit and report it.
#pragma once
#include <stdint.h>

namespace fdp {

constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;  // about a second

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}

// Where a wait that ran out reports it.  `abort_flag` (shared memory) stops the other waits of the
// CTA; `status` is the call's status word in its workspace (may be null); `sticky` is the device's
// slot of the library's host-visible status array (may be null): the next entry-point call on that
// device reads it on the host, without any synchronisation, and returns FDP_ERR_TIMEOUT.
struct WaitCtx {
  volatile int* abort_flag;
  int* status;
  volatile int* sticky;
  long long limit;      // cycles of clock64
};

// Bounded wait; false when it gave up (own limit, or another thread of the CTA already did).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& w, int code) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (mbar_try(bar, parity)) return true;
    if (*w.abort_flag != 0) return false;
    if (clock64() - t0 > w.limit) {
      *w.abort_flag = 1;
      if (w.status != nullptr) atomicCAS(w.status, 0, code);
      if (w.sticky != nullptr) { *w.sticky = code; __threadfence_system(); }
      return false;
    }
  }
}
// The same verdict for every lane of a (converged) warp: each lane waits on its own, then the warp
// votes -- it goes on only if all 32 lanes saw the phase complete.  What follows such a wait are
// warp-wide instructions (tcgen05.ld.sync.aligned, shuffles) that need the whole warp.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const WaitCtx& w, int code) {
  const bool ok = mbar_wait(bar, parity, w, code);
  return __all_sync(0xffffffffu, ok);
}
// contiguous global -> shared copy (16-byte aligned, size a multiple of 16), completion on an mbarrier
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

}  // namespace fdp
