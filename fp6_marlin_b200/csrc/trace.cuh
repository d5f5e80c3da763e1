// Optional in-kernel timeline (compiled in only with -DFP6M_TRACE; the shipped library has none of it).
// Lane 0 of every warp of the CTAs listed in kTraceCtas appends {tag, argument, SM clock} records to its
// own region of a device array; fp6m_trace_read copies the array out after a launch.
#pragma once

#include <stdint.h>

namespace fp6m {

#ifdef FP6M_TRACE
constexpr int kTraceCtaCount = 2;
constexpr int kTraceWarps = 32;
constexpr int kTraceEntries = 1024;
__device__ const int kTraceCtas[kTraceCtaCount] = {2, 99};     // both reduce a strip when K = N = 8192 runs on 148 SMs
__device__ unsigned long long g_trace[kTraceCtaCount][kTraceWarps][kTraceEntries];

// start / end of every CTA of the last 64 launches in nanoseconds (%globaltimer), indexed by launch epoch
__device__ unsigned long long g_launch_times[64][160][2];
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

struct Tracer {
  unsigned long long* buf;
  long long t0;
  int count;
  __device__ __forceinline__ void init(int cta, int warp, int lane) {
    buf = nullptr;
    count = 0;
    t0 = 0;
    if (lane != 0 || warp >= kTraceWarps) return;
    for (int i = 0; i < kTraceCtaCount; ++i)
      if (kTraceCtas[i] == cta) buf = g_trace[i][warp];
    if (buf) {
      t0 = clock64();
      buf[0] = 0;
    }
  }
  __device__ __forceinline__ void operator()(int tag, int arg) {
    if (buf && count < kTraceEntries - 2) {
      const unsigned long long t = (unsigned long long)(clock64() - t0) & 0xffffffffull;
      buf[++count] = ((unsigned long long)tag << 56) | ((unsigned long long)(arg & 0xffffff) << 32) | t;
      buf[0] = count;
    }
  }
};
#define FP6M_TRACE_DECL(name) Tracer name
#define FP6M_TRACE_INIT(name, cta, warp, lane) name.init(cta, warp, lane)
#define FP6M_TRACE_EVENT(name, tag, arg) name(tag, arg)
#else
#define FP6M_TRACE_DECL(name)
#define FP6M_TRACE_INIT(name, cta, warp, lane)
#define FP6M_TRACE_EVENT(name, tag, arg)
#endif

}  // namespace fp6m
