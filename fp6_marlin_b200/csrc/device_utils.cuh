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

// Wait with a limit (about one second).  When the limit runs out the thread records
// FP6M_ERR_TIMEOUT in *status, marks itself `dead` and carries on as if the wait had succeeded:
// every address the kernels form is independent of loaded data, so the kernel still terminates
// (with garbage results and a status the host reads) instead of hanging the GPU.  A dead thread
// skips all later waits.
// A failed mbarrier.try_wait comes back after well under 100 ns on this hardware, so a warp that
// polls in a plain loop issues instructions all the time and takes issue slots from the warps that
// work (measured: four in ten of a kernel's executed instructions were polling).  Hence the loop
// sleeps between polls: `kSleepNs` is the grain - short where the wake-up latency adds to a chain
// the pipeline depends on, long for roles that run far ahead of their consumers.
template <int kSleepNs = 32>
__device__ __forceinline__ void mbar_wait_bounded(uint32_t bar, uint32_t parity, int* status, bool& dead) {
  // fast path: in steady state the phase is complete already
  if (mbar_try_wait(bar, parity)) return;
  if (dead) return;
  constexpr uint32_t kSleep = kSleepNs > 0 ? kSleepNs : 1;
  constexpr uint32_t kLimit = 1u << 24;                       // x (sleep + poll) of at least ~60 ns each: about a second
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .u32 i;\n"
      "mov.u32 i, 0;\n"
      "FP6M_WAIT_LOOP:\n"
      "nanosleep.u32 %3;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "@p bra FP6M_WAIT_DONE;\n"
      "add.u32 i, i, 1;\n"
      "setp.lt.u32 p, i, %4;\n"
      "@p bra FP6M_WAIT_LOOP;\n"
      "setp.ne.u32 p, 0, 0;\n"
      "FP6M_WAIT_DONE:\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "n"(kSleep), "n"(kLimit)
      : "memory");
  if (ok) return;
  dead = true;
  if (status) atomicExch(status, kStatusTimeout);
}

// The same bounded wait without a branch in the caller: the common case - the phase is complete - costs
// the try_wait and one branch inside the block.  `w.limit` is the number of polls still allowed (a wait
// that ran out sets it to 1, so that later waits of the thread give up at once) and `w.failed` remembers
// that a wait ran out; the role reports it once, at its end (report_waits).
struct WaitState {
  uint32_t limit = 1u << 24;      // x (sleep + poll) of at least ~60 ns each: about a second
  uint32_t failed = 0;
};
template <int kSleepNs = 32>
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, WaitState& w) {
  constexpr uint32_t kSleep = kSleepNs > 0 ? kSleepNs : 1;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .u32 i;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%2], %3;\n"
      "@p bra FP6M_WAIT_DONE;\n"
      "mov.u32 i, 0;\n"
      "FP6M_WAIT_LOOP:\n"
      "nanosleep.u32 %4;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%2], %3;\n"
      "@p bra FP6M_WAIT_DONE;\n"
      "add.u32 i, i, 1;\n"
      "setp.lt.u32 p, i, %0;\n"
      "@p bra FP6M_WAIT_LOOP;\n"
      "mov.u32 %0, 1;\n"
      "mov.u32 %1, 1;\n"
      "FP6M_WAIT_DONE:\n"
      "}\n"
      : "+r"(w.limit), "+r"(w.failed)
      : "r"(bar), "r"(parity), "n"(kSleep)
      : "memory");
}
__device__ __forceinline__ void report_waits(const WaitState& w, int* status) {
  if (w.failed && status) atomicExch(status, kStatusTimeout);
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

__device__ __forceinline__ void named_bar_arrive(int id, int threads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory");
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
