// GPU half of the C ABI (include/fp6m.h): argument validation that mirrors the reference's host
// dispatcher, the stripe schedule, and the kernel launches.  No allocation, no synchronisation.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>

#include "../../include/fp6m.h"
#include "fp6m_layout.h"
#include "gemm_params.h"

namespace {

using namespace fp6m;

thread_local char g_cuda_error[256] = "";

int cuda_fail(cudaError_t e, const char* where) {
  std::snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", where, cudaGetErrorString(e));
  return FP6M_ERR_CUDA;
}

int sm_count(int dev) {
  static int cached[64] = {};
  if (dev < 0 || dev >= 64) return 0;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) switched = cudaSetDevice(dev) == cudaSuccess;
  }
  ~DeviceGuard() { if (switched) cudaSetDevice(prev); }
};

// How a GEMM of M rows is cut into launches: kernel, tile of rows, rows per launch, grid.
struct LaunchPlan {
  bool wide;        // the kernel with scaled operands and tiles of 256 rows
  int tile;         // rows of A per MMA tile
  int rows;         // rows of A per launch
  int ctas;         // grid of the first (largest) launch
};

// `sms` <= 0: the largest grid any device can get (an upper bound for sizing buffers).
LaunchPlan plan_launches(int M, const Geometry& geo, int sms, int two_launches = -1) {
  LaunchPlan lp;
  // 129 to 256 rows on a layer with few blocks per CTA: two launches of the kernel for up to 128 rows beat one
  // 256-row tile of the other kernel, whose split-K partials are 256 KB per CTA and strip.  Measured at 256 / 160
  // rows: K = N = 8192 (28 blocks per CTA) 59 -> 57 / 58 -> 44 us, 4096 x 4096 46.5 -> 40, 11008 x 4096 59 -> 53,
  // 4096 x 22016 (37 blocks) 70.5 -> 69.8; K = N = 16384 (111 blocks) is 4 % slower that way, and so are three launches
  // for 384 rows.  `two_launches`: -1 decides here, 0 / 1 force (sizing a buffer for either).
  bool two = false;
  if (M > kTc5MaxRows && M <= 2 * kTc5MaxRows) {
    const long long blocks = (long long)(geo.strips4 + geo.strips6) * geo.k128;
    two = two_launches < 0 ? blocks <= 48ll * (sms > 0 ? sms : 148) : two_launches != 0;
  }
  lp.wide = M > kTc5MaxRows && !two;
  lp.tile = lp.wide ? wide_tile_rows(M) : tc5_tile_rows(M < kTc5MaxRows ? M : kTc5MaxRows);
  // CTAs own contiguous ranges of (tile, strip) pairs, so the tiles of a launch are all in flight at once:
  // keep their activations (tile x K halves each) within half of L2
  // (measured at K = 16384: 64 MB of activations per launch are as fast as 32 MB on a full layer and 23 % faster
  // on a shard of 2048 columns, whose 16 strips need eight row tiles to give every CTA a strip; 96 MB are slower)
  int max_tiles = (int)((64ll << 20) / ((long long)lp.tile * geo.K * 2));
  if (max_tiles < 1) max_tiles = 1;
  if (max_tiles > kMaxRowTiles) max_tiles = kMaxRowTiles;
  lp.rows = lp.wide ? lp.tile * max_tiles : lp.tile;
  const int launch_rows = M < lp.rows ? M : lp.rows;
  const int row_tiles = lp.wide ? (launch_rows + lp.tile - 1) / lp.tile : 1;
  const int cap = lp.wide ? kMaxWideCtas : kMaxCtas;
  long long want = sms > 0 ? (long long)sms * (lp.wide ? 1 : tc5_ctas_per_sm(launch_rows)) : cap;
  int ctas = want < cap ? (int)want : cap;
  // at least ~16 units per CTA, also when that leaves SMs idle: a small GEMM split over every SM spends
  // its time in the split-K reduction (16 contributors per strip for N = 1024), not in streaming
  const long long total_units = (long long)row_tiles * (geo.strips4 + geo.strips6) * units_per_strip(geo);
#ifndef FP6M_MIN_UNITS_PER_CTA
#define FP6M_MIN_UNITS_PER_CTA 16
#endif
  long long by_work = total_units / FP6M_MIN_UNITS_PER_CTA;
  if (by_work < 1) by_work = 1;
  if (ctas > by_work) ctas = (int)by_work;
  if (ctas < 1) ctas = 1;
  lp.ctas = ctas;
  return lp;
}

size_t scratch_bytes_of(const LaunchPlan& lp) {
  const size_t b = lp.wide ? wide_scratch_bytes(lp.ctas, lp.tile) : tc5_scratch_bytes(lp.ctas, lp.tile);
  return (b + 255) & ~(size_t)255;
}

}  // namespace

extern "C" {

size_t fp6m_mul_scratch_bytes(int M, int N, int K, int quant_cols, int sms) {
  if (M <= 0 || N <= 0 || K <= 0) {
    // no shape given: the bound over every configuration (the largest grid with the largest partial tile)
    size_t b = tc5_scratch_bytes(kMaxCtas, kTc5MaxRows);
    const size_t w = wide_scratch_bytes(kMaxWideCtas, wide_rows_per_pass());
    if (w > b) b = w;
    return (b + 255) & ~(size_t)255;
  }
  const int qc = quant_cols < 0 ? 0 : (quant_cols > N ? N : quant_cols);
  const Geometry geo = make_geometry(K, N, qc, 128);
  if (sms <= 0 && M > kTc5MaxRows && M <= 2 * kTc5MaxRows) {
    // no device given: enough for either way of cutting 129 to 256 rows into launches
    const size_t a = scratch_bytes_of(plan_launches(M, geo, sms, 0)), b = scratch_bytes_of(plan_launches(M, geo, sms, 1));
    return a > b ? a : b;
  }
  return scratch_bytes_of(plan_launches(M, geo, sms));
}

int fp6m_mul_launches(int M, int N, int K, int quant_cols, int sms, int* many_rows_kernel) {
  if (many_rows_kernel) *many_rows_kernel = 0;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int qc = quant_cols < 0 ? 0 : (quant_cols > N ? N : quant_cols);
  const LaunchPlan lp = plan_launches(M, make_geometry(K, N, qc, 128), sms);
  if (many_rows_kernel) *many_rows_kernel = lp.wide ? 1 : 0;
  return (M + lp.rows - 1) / lp.rows;
}

}  // extern "C"

namespace {

int mul_impl(const void* A, const void* B, void* C, const void* s, int M, int N, int K,
             void* workspace, size_t workspace_bytes, void* scratch, size_t scratch_bytes,
             int dev, void* stream, int thread_k, int thread_n, int sms, int max_par,
             int quant_cols, int group_size, int layout, int* status_dev, const OutputMap& out,
             int epilogue = kEpilogueNone, const void* residual = nullptr) {
  // --- the checks of the reference dispatcher, in its order (fp6_marlin_cuda_kernel.cu:885-907)
  if (M < 0 || N < 0 || K < 0) return FP6M_ERR_BAD_ARG;
  if (thread_k == -1 || thread_n == -1) {
    if (M <= 16) { thread_k = 128; thread_n = 128; } else { thread_k = 64; thread_n = 256; }
  }
  if (thread_k <= 0 || thread_n <= 0) return FP6M_ERR_KERN_SHAPE;
  if (N % thread_n != 0 || K % thread_k != 0) return FP6M_ERR_PROB_SHAPE;
  if (M == 0 || N == 0 || K == 0) return FP6M_OK;
  // the reference has kernels for 128x128 tiles with at most 16 rows and for 64x256 tiles (:933-942)
  const bool shape_ok = (thread_k == 128 && thread_n == 128 && M <= 16) || (thread_k == 64 && thread_n == 256);
  if (!shape_ok) return FP6M_ERR_KERN_SHAPE;

  // --- checks of this implementation
  if (max_par < 1) max_par = 1;
  if (workspace_bytes < (size_t)(N / 128) * max_par * 4) return FP6M_ERR_WORKSPACE;  // fp6_marlin_cuda.cpp:62-63
  if (layout != FP6M_LAYOUT_B200) return FP6M_ERR_BAD_ARG;
  if (!(group_size == 128 || group_size <= 0)) return FP6M_ERR_BAD_ARG;
  const int qc = quant_cols < 0 ? 0 : quant_cols;
  if (qc > N || qc % 8 || (N - qc) % 8 || K % 8) return FP6M_ERR_PROB_SHAPE;
  if (group_size == 128 && K % 128) return FP6M_ERR_PROB_SHAPE;
  if (!A || !B || (!C && out.n_out == 0) || !s || !workspace || !scratch) return FP6M_ERR_BAD_ARG;
  if (!aligned16(A) || !aligned16(B) || !aligned16(C) || !aligned16(s) || !aligned16(scratch)) return FP6M_ERR_BAD_ARG;
  if (epilogue != kEpilogueNone && epilogue != kEpilogueSiluMul && epilogue != kEpilogueResidual) return FP6M_ERR_BAD_ARG;
  if (epilogue != kEpilogueNone && out.n_out != 0) return FP6M_ERR_BAD_ARG;       // not together with the scattered output
  if (epilogue == kEpilogueResidual && (!residual || (reinterpret_cast<uintptr_t>(residual) & 1))) return FP6M_ERR_BAD_ARG;

  DeviceGuard guard(dev);
  if (sms <= 0) sms = sm_count(dev);
  if (sms <= 0) return cuda_fail(cudaGetLastError(), "cudaDeviceGetAttribute");
  MulParams p;
  p.geo = make_geometry(K, N, qc, group_size);
  if ((long long)kMaxRowTiles * (p.geo.strips4 + p.geo.strips6) * units_per_strip(p.geo) > 0x3fffffff) return FP6M_ERR_PROB_SHAPE;
  // up to kTc5MaxRows rows (up to twice as many on a small layer, in two launches): the kernel with fp32 group
  // scaling; more: the wide kernel, tiles of 256 rows, up to kMaxRowTiles tiles per launch
  const LaunchPlan lp = plan_launches(M, p.geo, sms);
  const bool wide = lp.wide;
  const int tile = lp.tile, rows = lp.rows, ctas = lp.ctas;
  if (scratch_bytes < scratch_bytes_of(lp)) return FP6M_ERR_SCRATCH;
  p.B = static_cast<const uint8_t*>(B);
  p.S = static_cast<const half*>(s);
  p.N = N; p.K = K;
  p.counters = static_cast<int*>(workspace);
  p.epochs = static_cast<unsigned int*>(scratch);
  p.partials = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(scratch) + kEpochWords * sizeof(unsigned int));
  p.status = status_dev;
  p.out = out;
  p.epilogue = epilogue;
  p.R = nullptr;
  {
    // 16-byte stores of finished rows need every row start and both column bases on 16-byte boundaries
    const int ld = out.n_out ? out.ld : N;
    const int base4 = out.n_out ? out.col4 : 0, base6 = out.n_out ? out.col6 : N - qc;
    bool ok = epilogue == kEpilogueNone && ld % 8 == 0 && base4 % 8 == 0 && base6 % 8 == 0;
    for (int q = 0; q < out.n_out; ++q) ok = ok && aligned16(out.peer[q]);
    p.vec_rows = ok ? 1 : 0;
  }
  // Expanding before the grid dependency resolves pays on a chain of launches when the next launch's CTAs get
  // onto their SMs early enough: measured -10 % on a 4096 x 4096 layer (128 CTAs), -2 to -3 % with 32 to 128 rows
  // or 19 blocks per CTA, +1 % (worse) with 28 blocks per CTA on every SM and 16 rows.
  {
    const long long blocks = (long long)(p.geo.strips4 + p.geo.strips6) * p.geo.k128;
    p.expand_early = (!wide && (tile > 16 || blocks <= 20ll * ctas)) ? 1 : 0;
  }

  for (int m0 = 0; m0 < M; m0 += rows) {
    p.A = static_cast<const half*>(A) + (size_t)m0 * K;
    // with the gate / up epilogue C has N / 2 columns
    p.C = C ? static_cast<half*>(C) + (size_t)m0 * (epilogue == kEpilogueSiluMul ? N / 2 : N) : nullptr;
    p.R = epilogue == kEpilogueResidual ? static_cast<const half*>(residual) + (size_t)m0 * N : nullptr;
    for (int q = 0; q < out.n_out; ++q) p.out.peer[q] = out.peer[q] + (size_t)m0 * out.ld;
    p.M = (M - m0) < rows ? (M - m0) : rows;
    p.row_tiles = wide ? (p.M + tile - 1) / tile : 1;
    make_schedule(p.geo, ctas, &p.sched, p.row_tiles);
    if (!wide) align_schedule_to_blocks(&p.sched);
    cudaError_t e = wide ? launch_gemm_wide(p, tile, static_cast<cudaStream_t>(stream)) : launch_gemm_tc5(p, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return cuda_fail(e, wide ? "w46_gemm_wide launch" : "w46_gemm_tc5 launch");
  }
  return FP6M_OK;
}

}  // namespace

extern "C" {

int fp6m_mul(const void* A, const void* B, void* C, const void* s, int M, int N, int K,
             void* workspace, size_t workspace_bytes, void* scratch, size_t scratch_bytes,
             int dev, void* stream, int thread_k, int thread_n, int sms, int max_par,
             int quant_cols, int group_size, int layout, int* status_dev) {
  OutputMap out = {};
  return mul_impl(A, B, C, s, M, N, K, workspace, workspace_bytes, scratch, scratch_bytes, dev, stream, thread_k, thread_n,
                  sms, max_par, quant_cols, group_size, layout, status_dev, out);
}

int fp6m_mul_fused(const void* A, const void* B, void* C, const void* s, int M, int N, int K,
                   void* workspace, size_t workspace_bytes, void* scratch, size_t scratch_bytes,
                   int dev, void* stream, int thread_k, int thread_n, int sms, int max_par,
                   int quant_cols, int group_size, int layout, int* status_dev, int epilogue, const void* residual) {
  OutputMap out = {};
  return mul_impl(A, B, C, s, M, N, K, workspace, workspace_bytes, scratch, scratch_bytes, dev, stream, thread_k, thread_n,
                  sms, max_par, quant_cols, group_size, layout, status_dev, out, epilogue, residual);
}

int fp6m_mul_scatter(const void* A, const void* B, void* const* outputs, int n_outputs, int ld_out, int col4_base, int col6_base,
                     const void* s, int M, int N, int K, void* workspace, size_t workspace_bytes, void* scratch,
                     size_t scratch_bytes, int dev, void* stream, int thread_k, int thread_n, int sms, int max_par,
                     int quant_cols, int group_size, int layout, int* status_dev) {
  if (!outputs || n_outputs < 1 || n_outputs > 8 || ld_out < N || col4_base < 0 || col6_base < 0) return FP6M_ERR_BAD_ARG;
  {
    // both column ranges must lie inside a row of the outputs: the stores go to peer memory unchecked
    const int qc = quant_cols < 0 ? 0 : quant_cols;
    if (qc > N || (long long)col4_base + (N - qc) > ld_out || (long long)col6_base + qc > ld_out) return FP6M_ERR_BAD_ARG;
  }
  OutputMap out = {};
  out.n_out = n_outputs;
  out.ld = ld_out;
  out.col4 = col4_base;
  out.col6 = col6_base;
  for (int q = 0; q < n_outputs; ++q) {
    if (!outputs[q] || (reinterpret_cast<uintptr_t>(outputs[q]) & 1)) return FP6M_ERR_BAD_ARG;
    out.peer[q] = static_cast<half*>(outputs[q]);
  }
  return mul_impl(A, B, nullptr, s, M, N, K, workspace, workspace_bytes, scratch, scratch_bytes, dev, stream, thread_k,
                  thread_n, sms, max_par, quant_cols, group_size, layout, status_dev, out);
}

// Scratch of fp6m_mul_static_scratch.  In host code this name is only a handle: the device address
// comes from cudaGetSymbolAddress, once per device.
static __device__ __align__(256) unsigned char g_static_scratch[FP6M_STATIC_SCRATCH_BYTES];

int fp6m_mul_static_scratch(const void* A, const void* B, void* C, const void* s, int M, int N, int K,
                            void* workspace, size_t workspace_bytes, int dev, void* stream,
                            int thread_k, int thread_n, int sms, int max_par,
                            int quant_cols, int group_size, int layout, int* status_dev) {
  static void* scratch_of_device[64] = {};
  if (dev < 0 || dev >= 64) return FP6M_ERR_BAD_ARG;
  if (!scratch_of_device[dev]) {
    DeviceGuard guard(dev);                 // the symbol has one instance per device: ask with `dev` current
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || !ptr) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
    scratch_of_device[dev] = ptr;
  }
  // fp6m_mul checks the size it needs against what it is given and returns FP6M_ERR_SCRATCH if it is short
  return fp6m_mul(A, B, C, s, M, N, K, workspace, workspace_bytes, scratch_of_device[dev],
                  (size_t)FP6M_STATIC_SCRATCH_BYTES, dev, stream, thread_k, thread_n, sms, max_par,
                  quant_cols, group_size, layout, status_dev);
}

int fp6m_dump_operands(const void* B, const void* s, void* W_out, int N, int K, int quant_cols,
                       int group_size, int dev, void* stream) {
  if (!B || !s || !W_out || N <= 0 || K <= 0) return FP6M_ERR_BAD_ARG;
  if (!(group_size == 128 || group_size <= 0)) return FP6M_ERR_BAD_ARG;
  const int qc = quant_cols < 0 ? 0 : quant_cols;
  if (qc > N) return FP6M_ERR_BAD_ARG;
  DeviceGuard guard(dev);
  cudaError_t e = launch_dump_operands(static_cast<const uint8_t*>(B), static_cast<const half*>(s),
                                       static_cast<half*>(W_out), make_geometry(K, N, qc, group_size),
                                       static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? FP6M_OK : cuda_fail(e, "dump_operands launch");
}

int fp6m_set_launch_overlap(int enable) {
  const int before = tc5_get_overlap() ? 1 : 0;
  if (enable >= 0) tc5_set_overlap(enable != 0);
  return before;
}

int fp6m_set_ordered_sums(int enable) {
  const int before = tc5_get_ordered_sums() ? 1 : 0;
  if (enable >= 0) tc5_set_ordered_sums(enable != 0);
  return before;
}

const char* fp6m_last_cuda_error(void) { return g_cuda_error; }

const char* fp6m_version(void) { return "fp6m-b200 0.1 (sm_100a)"; }

}  // extern "C"
