// Peer memory for the N-sharded GEMM: buffers that the other GPUs of the node can store into (CUDA IPC,
// plain peer stores over NVLink - no multicast), and the two small kernels that turn the per-rank GEMMs
// into an all-gather: `signal` tells every rank that this rank's shard of step t has landed, `wait`
// holds the stream until every rank has said so.  Waiting is bounded; a wait that runs out records
// FP6M_ERR_TIMEOUT in the status word and lets the stream go on.  The reference has no multi-GPU code.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fp6m.h"

namespace {

struct Guard {
  int prev = -1;
  explicit Guard(int dev) {
    cudaGetDevice(&prev);
    if (dev >= 0 && dev != prev) cudaSetDevice(dev);
  }
  ~Guard() {
    int cur = -1;
    cudaGetDevice(&cur);
    if (prev >= 0 && cur != prev) cudaSetDevice(prev);
  }
};

struct FlagPointers {
  int* peer[8];
};

// polls of a flag before a wait gives up (each poll sleeps >= 100 ns: the default is about half a second,
// inside the ~1 s bound of the GEMM kernels' own waits)
int g_wait_polls = 1 << 22;

// n threads.  The GEMM of this step ran before this kernel on the same stream, so its stores to the peers have
// been issued; one system-scope fence per thread orders them before the flags, then thread q writes rank q's
// flag - the n remote stores travel in parallel (a release store per peer from one thread costs one NVLink
// round trip each: measured 2.4 us per peer).
__global__ void signal_kernel(FlagPointers flags, int n, int rank, int* step) {
  __shared__ int target;
  if (threadIdx.x == 0) {
    target = *step + 1;
    *step = target;
  }
  __syncthreads();
  __threadfence_system();
  if (threadIdx.x < n) {
    asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(flags.peer[threadIdx.x] + rank), "r"(target) : "memory");
  }
}

// n threads: thread r waits until rank r has signalled the step that this rank's signal kernel last started
__global__ void wait_kernel(const int* flags, int n, const int* step, int* status, int max_polls) {
  const int r = threadIdx.x;
  if (r >= n) return;
  if (status && *status != 0) return;      // an earlier wait already ran out: do not stall every later step
  const int t = *step;
  int seen = 0;
  for (int spin = 0; spin < max_polls; ++spin) {
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(flags + r) : "memory");
    if (seen - t >= 0) return;
    __nanosleep(100);
  }
  if (status) atomicExch(status, FP6M_ERR_TIMEOUT);
}

// Both in one launch (a launch costs more than the hand-shake): thread r signals rank r, then waits for rank r.
__global__ void signal_wait_kernel(FlagPointers flags, int n, int rank, int* step, int* status, int max_polls) {
  // the next GEMM of the stream may set itself up and prefetch its weights during the hand-shake; it touches
  // activations, outputs and scratch only after this kernel has completed (its own griddepcontrol.wait)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  __shared__ int target;
  if (threadIdx.x == 0) {
    target = *step + 1;
    *step = target;
  }
  __syncthreads();
  __threadfence_system();
  const int r = threadIdx.x;
  if (r >= n) return;
  // thread r: this rank's flag to rank r (the n remote stores travel in parallel), then wait for rank r's flag
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(flags.peer[r] + rank), "r"(target) : "memory");
  if (status && *status != 0) return;
  const int t = target;
  int seen = 0;
  for (int spin = 0; spin < max_polls; ++spin) {
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(flags.peer[rank] + r) : "memory");
    if (seen - t >= 0) return;
    __nanosleep(100);
  }
  if (status) atomicExch(status, FP6M_ERR_TIMEOUT);
}

// Lets the kernels behind it in the stream launch at once (programmatic dependent launch) and then keeps one
// warp busy for `ns` nanoseconds: a long-running predecessor for tests of the launch overlap.
__global__ void busy_kernel(unsigned long long ns) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  unsigned long long t0, t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  do {
    __nanosleep(2000);
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  } while (t - t0 < ns);
}

}  // namespace

extern "C" {

int fp6m_debug_busy_kernel(int milliseconds, int dev, void* stream) {
  if (milliseconds < 0 || milliseconds > 5000) return FP6M_ERR_BAD_ARG;
  Guard guard(dev);
  busy_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>((unsigned long long)milliseconds * 1000000ull);
  return cudaGetLastError() == cudaSuccess ? FP6M_OK : FP6M_ERR_CUDA;
}

int fp6m_peer_alloc(size_t bytes, int dev, void** ptr, void* handle64) {
  if (!ptr || !handle64 || bytes == 0) return FP6M_ERR_BAD_ARG;
  Guard guard(dev);
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return FP6M_ERR_CUDA;
  if (cudaMemset(p, 0, bytes) != cudaSuccess) { cudaFree(p); return FP6M_ERR_CUDA; }
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) { cudaFree(p); return FP6M_ERR_CUDA; }
  static_assert(sizeof(h) == 64, "IPC handle size");
  __builtin_memcpy(handle64, &h, 64);
  *ptr = p;
  return FP6M_OK;
}

int fp6m_peer_open(const void* handle64, int dev, void** ptr) {
  if (!handle64 || !ptr) return FP6M_ERR_BAD_ARG;
  Guard guard(dev);
  cudaIpcMemHandle_t h;
  __builtin_memcpy(&h, handle64, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return FP6M_ERR_CUDA;
  *ptr = p;
  return FP6M_OK;
}

int fp6m_peer_close(void* ptr, int dev) {
  Guard guard(dev);
  return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? FP6M_OK : FP6M_ERR_CUDA;
}

int fp6m_peer_free(void* ptr, int dev) {
  Guard guard(dev);
  return cudaFree(ptr) == cudaSuccess ? FP6M_OK : FP6M_ERR_CUDA;
}

int fp6m_peer_signal(void* const* flag_arrays, int n, int rank, int* step_dev, int dev, void* stream) {
  if (!flag_arrays || n < 1 || n > 8 || rank < 0 || rank >= n || !step_dev) return FP6M_ERR_BAD_ARG;
  Guard guard(dev);
  FlagPointers f = {};
  for (int q = 0; q < n; ++q) f.peer[q] = static_cast<int*>(flag_arrays[q]);
  signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, n, rank, step_dev);
  return cudaGetLastError() == cudaSuccess ? FP6M_OK : FP6M_ERR_CUDA;
}

int fp6m_peer_signal_wait(void* const* flag_arrays, int n, int rank, int* step_dev, int* status_dev, int dev, void* stream) {
  if (!flag_arrays || n < 1 || n > 8 || rank < 0 || rank >= n || !step_dev) return FP6M_ERR_BAD_ARG;
  Guard guard(dev);
  FlagPointers f = {};
  for (int q = 0; q < n; ++q) f.peer[q] = static_cast<int*>(flag_arrays[q]);
  // (launching this kernel as a programmatic dependent of the GEMM was measured: no gain)
  signal_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f, n, rank, step_dev, status_dev, g_wait_polls);
  return cudaGetLastError() == cudaSuccess ? FP6M_OK : FP6M_ERR_CUDA;
}

int fp6m_set_peer_wait_polls(int polls) {
  const int before = g_wait_polls;
  if (polls > 0) g_wait_polls = polls;
  return before;
}

int fp6m_peer_wait(const void* flags_local, int n, const int* step_dev, int* status_dev, int dev, void* stream) {
  if (!flags_local || n < 1 || n > 8 || !step_dev) return FP6M_ERR_BAD_ARG;
  Guard guard(dev);
  wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const int*>(flags_local), n, step_dev, status_dev, g_wait_polls);
  return cudaGetLastError() == cudaSuccess ? FP6M_OK : FP6M_ERR_CUDA;
}

}  // extern "C"
