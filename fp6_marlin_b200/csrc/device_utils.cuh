// Device-side building blocks for sm_100a: mbarrier + bulk-TMA wrappers with BOUNDED waits and
// small logic / permute helpers.
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

namespace fp6m {

constexpr int kStatusTimeout = 8;  // == FP6M_ERR_TIMEOUT

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// try_wait with a suspend-time hint: the hardware may park the thread until the phase completes or
// the hint (nanoseconds) runs out, instead of burning issue slots in a polling loop.
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}

// Wait with a limit (about one second).  When the limit runs out the thread records
// FP6M_ERR_TIMEOUT in *status, marks itself `dead` and carries on as if the wait had succeeded:
// every address the kernels form is independent of loaded data, so the kernel still terminates
// (with garbage results and a status the host reads) instead of hanging the GPU.  A dead thread
// skips all later waits.
// Bounded wait.  `kSleepNs` > 0 is for roles that run far ahead of their consumers (producers): they
// sleep between polls, so their polling does not take issue slots from the working warps.
template <int kSleepNs = 0>
__device__ __forceinline__ void mbar_wait_bounded(uint32_t bar, uint32_t parity, int* status, bool& dead) {
  // fast path: one potentially-blocking try_wait; in steady state the phase is complete already
  if (mbar_try_wait(bar, parity)) return;
  if (dead) return;
#pragma unroll 1
  for (int i = 0; i < (1 << 16); ++i) {                      // up to 65536 x (16 us + sleep)
    if (kSleepNs > 0) __nanosleep(kSleepNs);
    if (mbar_try_wait_hint(bar, parity, 16384u)) return;
  }
  dead = true;
  if (status) atomicExch(status, kStatusTimeout);
}

// ---- bulk TMA (1-D, global -> shared of this CTA, completion on an mbarrier) -------------------
// With an L2 evict-first policy for data that is streamed once (the weights).
__device__ __forceinline__ void tma_load_1d_stream(uint32_t dst_smem, const void* src, uint32_t bytes,
                                                   uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t make_evict_first_policy() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// ---- named barrier among a subset of warps ---------------------------------------------------
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---- logic / permute helpers -------------------------------------------------------------------
template <int lut>
__device__ __forceinline__ uint32_t lop3(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(r) : "r"(a), "r"(b), "r"(c), "n"(lut));
  return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ uint32_t h2_as_u32(half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<half2*>(&u); }

}  // namespace fp6m
