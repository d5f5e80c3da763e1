// Micro-benchmark: what one launch of a (nearly) empty kernel costs inside a CUDA graph, as a function of the
// parameter bytes, the dynamic shared memory, the block size, a tensor-memory allocation and programmatic
// dependent launch - the floor under the per-launch time of the GEMM kernels, whose launch shape it copies
// (148 CTAs x 896 threads, 222 KB of shared memory, all 512 TMEM columns, 2.8 KB of parameters).
// Build and run (one B200):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o launch_cost launch_cost.cu && ./launch_cost
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
template <int WORDS> struct P { int v[WORDS]; };
template <int WORDS, bool TMEM>
__global__ void k(const __grid_constant__ P<WORDS> p, int* out) {
  extern __shared__ uint8_t sm[];
  __shared__ uint32_t tbase;
  if (TMEM) {
    if (threadIdx.x < 32) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(&tbase)), "r"(512) : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tbase), "r"(512) : "memory");
  }
  if (p.v[blockIdx.x % WORDS] == 12345 && threadIdx.x == 0) out[0] = sm[0];
}
template <int WORDS, bool TMEM>
void run(int threads, int smem, bool pdl, const char* name) {
  P<WORDS> p = {};
  int* out; cudaMalloc(&out, 4);
  cudaFuncSetAttribute(k<WORDS, TMEM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  cudaStream_t st; cudaStreamCreate(&st);
  cudaGraph_t g; cudaGraphExec_t ge;
  const int reps = 200;
  cudaStreamBeginCapture(st, cudaStreamCaptureModeGlobal);
  for (int i = 0; i < reps; ++i) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(148); cfg.blockDim = dim3(threads); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    cudaLaunchKernelEx(&cfg, k<WORDS, TMEM>, p, out);
  }
  cudaStreamEndCapture(st, &g);
  cudaGraphInstantiate(&ge, g, 0);
  cudaGraphLaunch(ge, st); cudaStreamSynchronize(st);
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  float best = 1e9;
  for (int it = 0; it < 5; ++it) {
    cudaEventRecord(e0, st); cudaGraphLaunch(ge, st); cudaEventRecord(e1, st); cudaStreamSynchronize(st);
    float ms; cudaEventElapsedTime(&ms, e0, e1); if (ms < best) best = ms;
  }
  printf("%-40s params=%5d B threads=%4d smem=%6d tmem=%d pdl=%d: %.2f us per launch (%s)\n", name, WORDS * 4, threads, smem, (int)TMEM, (int)pdl, best * 1e3 / reps, cudaGetErrorString(cudaGetLastError()));
  cudaFree(out);
}
int main() {
  run<32, false>(128, 0, false, "small");
  run<32, false>(896, 0, false, "896 threads");
  run<32, false>(896, 222000, false, "896 threads + 222 KB smem");
  run<32, true>(896, 222000, false, "+ TMEM alloc/dealloc");
  run<700, true>(896, 222000, false, "+ 2.8 KB params");
  run<700, false>(128, 0, false, "small + 2.8 KB params");
  run<32, true>(896, 222000, true, "PDL: + TMEM");
  run<700, true>(896, 222000, true, "PDL: + TMEM + 2.8 KB params");
  run<32, false>(896, 100000, false, "896 threads + 100 KB smem");
  run<32, false>(512, 100000, false, "512 threads + 100 KB smem");
  return 0;
}
