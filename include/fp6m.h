/*
 * fp6m - C ABI of the B200-native W(4&6)A16 GEMM path.
 *
 * Plain pointers and sizes only; no torch types.  Every entry point names the reference interface
 * it stands in for (paths are relative to the reference project).  All functions return one of
 * the FP6M_* codes below unless stated otherwise.  Host functions never touch the GPU; GPU
 * functions never allocate, never synchronise and never touch host memory: they enqueue work on
 * the stream they are given, so the caller owns every buffer and every lifetime.
 */
#ifndef FP6M_H_
#define FP6M_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  FP6M_OK = 0,
  FP6M_ERR_PROB_SHAPE = 1,   /* same value and meaning as ERR_PROB_SHAPE, fp6_marlin_cuda_kernel.cu:861 */
  FP6M_ERR_KERN_SHAPE = 2,   /* same value and meaning as ERR_KERN_SHAPE, fp6_marlin_cuda_kernel.cu:862 */
  FP6M_ERR_VALUE_RANGE = 3,  /* a value cannot be represented in FP6 (weight_quant.cpp:48-53 throws) */
  FP6M_ERR_BAD_ARG = 4,      /* null / misaligned pointer, bad size, unknown layout or group size */
  FP6M_ERR_WORKSPACE = 5,    /* workspace smaller than the reference demands (fp6_marlin_cuda.cpp:62-63) */
  FP6M_ERR_SCRATCH = 6,      /* scratch buffer smaller than fp6m_mul_scratch_bytes() */
  FP6M_ERR_CUDA = 7,         /* a CUDA runtime call failed; see fp6m_last_cuda_error() */
  FP6M_ERR_TIMEOUT = 8       /* device status word: a bounded wait inside a kernel ran out */
};

enum { FP6M_LAYOUT_REFERENCE = 0, FP6M_LAYOUT_B200 = 1 };

/* ------------------------------------------------------------------------------------------ */
/* Host side: weight preparation                                                              */
/* ------------------------------------------------------------------------------------------ */

/* fp16 -> dense FP6 E3M2 stream, rows*cols*6/8 bytes, truncating cast, byte-identical to
 * weight_prepacking_fp16_to_fp6 (fp6_marlin/weight_quant.cpp:106-124; binding pybind.cpp:42-59).
 * The row-major memory of `w` is packed as it lies.  cols must be a multiple of 4.
 * FP6M_ERR_VALUE_RANGE replaces the reference's std::invalid_argument. */
int fp6m_quantize_fp6(const uint16_t* w, uint8_t* out, size_t rows, size_t cols);

/* fp16 -> one FP6 E3M2 code (0..63) per byte, `count` values; the per-element half of
 * cast_fp16_fp6 (fp6_marlin/weight_quant.cpp:27-91) without the 4-in-3 byte packing. */
int fp6m_encode_fp6(const uint16_t* w, uint8_t* codes, size_t count);

/* FP6 stream viewed as (n rows, k cols) -> the reference's "2+4" tensor-core layout (k*n*3/4
 * bytes), byte-identical to weight_matrix_prepacking (fp6_marlin/weight_prepacking.cpp:123-177;
 * binding pybind.cpp:18-31).  n and k must be multiples of 64. */
int fp6m_prepack_fp6(const uint8_t* fp6, uint8_t* out, size_t n, size_t k);

/* FP6 stream (n rows, k cols) and a per-row fp16 scale -> (n, k) fp16, bit-identical to
 * dequantMatrix_fp6_to_fp16 (fp6_marlin/weight_prepacking.cpp:180-217; binding pybind.cpp:70-87). */
int fp6m_dequant_fp6(const uint8_t* fp6, const uint16_t* scale, uint16_t* out, size_t n, size_t k);

/* Sizes of the b200 layout: bytes of the packed weight buffer and number of fp16 scales.
 * group_size is 128 (INT4 group scales) or -1 (per-channel, the reference's only mode,
 * fp6_marlin_cuda_kernel.cu:447-448).  qc = number of FP6 columns, -1 or 0 for none. */
int64_t fp6m_b200_weight_bytes(int K, int N, int qc);
int64_t fp6m_b200_scale_count(int K, int N, int qc, int group_size);

/* Logical codes -> b200 layout.  q4: K x (N-qc) INT4 codes 0..15 (uint8, row-major);
 * c6: K x qc FP6 codes 0..63; s4: groups x (N-qc) fp16 scales (groups = ceil(K/128) or 1);
 * s6: qc fp16 scales.  The counterpart of the packing half of gen_int4_weight / gen_mixed_weight
 * (test.py:106-114, 123-152) for the Blackwell tiling. */
int fp6m_pack_b200(const uint8_t* q4, const uint8_t* c6, const uint16_t* s4, const uint16_t* s6,
                   int K, int N, int qc, int group_size, uint8_t* B_out, uint16_t* s_out);
int fp6m_unpack_b200(const uint8_t* B, const uint16_t* s, int K, int N, int qc, int group_size,
                     uint8_t* q4, uint8_t* c6, uint16_t* s4, uint16_t* s6);

/* Reference-packed tensors (B = INT4 words then FP6 "2+4" words, s = permuted per-channel scales,
 * exactly what gen_mixed_weight returns, test.py:123-152) -> logical codes and plain scales. */
int fp6m_unpack_reference(const uint8_t* B_ref, const uint16_t* s_ref, int K, int N, int qc,
                          uint8_t* q4, uint8_t* c6, uint16_t* s4, uint16_t* s6);
/* Reference-packed tensors -> b200 layout (per-channel scales). */
int fp6m_repack_from_reference(const uint8_t* B_ref, const uint16_t* s_ref, int K, int N, int qc,
                               uint8_t* B_out, uint16_t* s_out);

/* The stripe schedule the GEMM uses for this shape on `ctas` CTAs: writes ctas+1 boundaries, in
 * units of 64 rows of one 128-column strip, into `bounds` (see fp6m_layout.h).  Returns the
 * number of units, or -1.
 * Stands in for the reference's in-kernel stripe arithmetic (fp6_marlin_cuda_kernel.cu:308-408). */
int fp6m_schedule(int K, int N, int qc, int group_size, int ctas, int* bounds);

/* ------------------------------------------------------------------------------------------ */
/* GPU side: the GEMM                                                                         */
/* ------------------------------------------------------------------------------------------ */

/* Bytes of scratch (device memory) fp6m_mul needs for this shape; 256-byte aligned.  The buffer must be
 * all zero the first time it is used and is otherwise private to fp6m_mul: keep passing it as it was left
 * (it holds per-strip epoch words and tagged split-K slots), or pass a freshly zeroed one. */
size_t fp6m_mul_scratch_bytes(int M, int N, int K, int quant_cols, int sms);

/* How fp6m_mul cuts this shape into kernel launches on a device with `sms` multiprocessors (the reference's
 * dispatcher likewise covers M in several launches, fp6_marlin_cuda_kernel.cu:917-948): returns their number;
 * *many_rows_kernel (may be null) = 1 if the kernel for more than 128 rows runs, 0 if the one for up to 128. */
int fp6m_mul_launches(int M, int N, int K, int quant_cols, int sms, int* many_rows_kernel);

/* C[M,N] (fp16, row-major, overwritten) = A[M,K] (fp16, row-major) x dequant(B, s).
 * Stands in for fp6_marlin_cuda(...) (fp6_marlin/fp6_marlin_cuda_kernel.cu:864-951) as called from
 * fp6_marlin_mul (fp6_marlin/fp6_marlin_cuda.cpp:47-92): same pointer roles, same tuning
 * arguments (thread_k, thread_n, sms, max_par are validated exactly as the reference validates
 * them and otherwise treated as hints), same return codes 0/1/2, asynchronous on `stream`.
 *   workspace       >= N/128*max_par 32-bit words, all zero on entry, left all zero on exit
 *                   (the reference's lock array; validated like the reference does, not written)
 *   scratch         >= fp6m_mul_scratch_bytes(...) bytes of device memory for the split-K partials,
 *                   zeroed before its first use (see fp6m_mul_scratch_bytes)
 *   quant_cols      number of FP6 columns (last columns of B); -1 = none
 *   group_size      128 or -1 (per-channel)
 *   layout          FP6M_LAYOUT_B200 (tensors in the reference's layout are converted first, on the
 *                   host, by fp6m_repack_from_reference)
 *   status_dev      optional device int: set to FP6M_ERR_TIMEOUT if a bounded wait ran out
 * Output columns keep the order of B: INT4 columns first, FP6 columns last. */
int fp6m_mul(const void* A, const void* B, void* C, const void* s, int M, int N, int K,
             void* workspace, size_t workspace_bytes, void* scratch, size_t scratch_bytes,
             int dev, void* stream, int thread_k, int thread_n, int sms, int max_par,
             int quant_cols, int group_size, int layout, int* status_dev);

/* fp6m_mul with the step that follows the GEMM in a transformer block fused into its epilogue, on the fp32
 * sums before the one rounding to fp16 (the reference's write_result, fp6_marlin_cuda_kernel.cu:698-749,
 * only scales and stores; its layer lists name the neighbours, bench.py:53-86):
 *   FP6M_EPILOGUE_SILU_MUL  gate / up projection in one matrix whose columns 2j and 2j+1 - inside the INT4
 *                           region and inside the FP6 region - are gate_j and up_j: C is M x N/2 and receives
 *                           silu(gate_j) * up_j, INT4 pairs first, then FP6 pairs;
 *   FP6M_EPILOGUE_RESIDUAL  C = A W + residual, residual an M x N fp16 matrix laid out like C (may be C).
 * FP6M_EPILOGUE_NONE makes it fp6m_mul.  Everything else as fp6m_mul.  No counterpart in the reference. */
enum { FP6M_EPILOGUE_NONE = 0, FP6M_EPILOGUE_SILU_MUL = 1, FP6M_EPILOGUE_RESIDUAL = 2 };
int fp6m_mul_fused(const void* A, const void* B, void* C, const void* s, int M, int N, int K,
                   void* workspace, size_t workspace_bytes, void* scratch, size_t scratch_bytes,
                   int dev, void* stream, int thread_k, int thread_n, int sms, int max_par,
                   int quant_cols, int group_size, int layout, int* status_dev, int epilogue, const void* residual);

/* Same GEMM as fp6m_mul for callers that may not allocate device memory at all: plug-ins living
 * inside a host runtime that owns the whole memory arena, code running after an allocator freeze
 * or while other threads hold the device in a state where cudaMalloc's implicit synchronisation is
 * not acceptable.  The split-K scratch is a static array inside the library (FP6M_STATIC_SCRATCH_BYTES,
 * 16 MiB, resident on every GPU that loads the library until the process exits); the caller still
 * passes A, B, C, s and the workspace.  This entry point has no counterpart in the reference.
 *   - Enough for up to 16 rows of A per call on grids of up to 511 CTAs, i.e. on every GPU with fewer
 *     than 512 SMs (larger M fits when `sms` limits the grid); a call that would need more returns
 *     FP6M_ERR_SCRATCH and launches nothing.
 *   - The first call on each device looks the array's device address up (cudaGetSymbolAddress); make
 *     that first call outside any stream capture.
 *   - All calls share the one array: calls that can overlap on the GPU (different streams) race.
 *     It starts out zeroed and needs no attention between calls.
 *   - Never calls cudaMalloc, cudaFree or any allocating routine. */
#define FP6M_STATIC_SCRATCH_BYTES (16u << 20)
int fp6m_mul_static_scratch(const void* A, const void* B, void* C, const void* s, int M, int N, int K,
                            void* workspace, size_t workspace_bytes, int dev, void* stream,
                            int thread_k, int thread_n, int sms, int max_par,
                            int quant_cols, int group_size, int layout, int* status_dev);

/* Debug: the dequantised weights W_deq[K, N] (fp16, row-major), produced by the expansion routines the
 * GEMM kernels use (exact q - 8, exact E3M2 value / 4096) followed by one fp16 multiply by the scale.
 * Lets a test prove bit-exactness against the reference's dequantisers (dequant_8int4 / dequant_8fp6,
 * fp6_marlin_cuda_kernel.cu:195-286) and its dequantised weights (test.py:98, weight_prepacking.cpp:199-212). */
int fp6m_dump_operands(const void* B, const void* s, void* W_out, int N, int K, int quant_cols,
                       int group_size, int dev, void* stream);

/* The GEMM of one shard of an N-sharded layer, with the all-gather of the output columns fused into its
 * epilogue: instead of C, every value is stored into `n_outputs` (1..8) full-width output buffers of `ld_out`
 * columns - the ranks' own buffer and the peers' buffers mapped with fp6m_peer_open - at column
 * `col4_base + j` for the shard's INT4 column j and `col6_base + j` for its FP6 column j.  Plain stores over
 * NVLink, no collective call, no multicast.  Everything else as fp6m_mul.  No counterpart in the reference. */
int fp6m_mul_scatter(const void* A, const void* B, void* const* outputs, int n_outputs, int ld_out, int col4_base, int col6_base,
                     const void* s, int M, int N, int K, void* workspace, size_t workspace_bytes, void* scratch,
                     size_t scratch_bytes, int dev, void* stream, int thread_k, int thread_n, int sms, int max_par,
                     int quant_cols, int group_size, int layout, int* status_dev);

/* Peer memory and the hand-shake that completes the fused all-gather.  These ALLOCATE / map device memory
 * and are meant for set-up and tear-down, not for the hot path:
 *   fp6m_peer_alloc   cudaMalloc + zero + CUDA IPC handle (64 bytes) to send to the other ranks of the node
 *   fp6m_peer_open    maps a buffer of another process from its handle (peer access enabled lazily)
 *   fp6m_peer_close / fp6m_peer_free   undo the two above
 * Hot path, asynchronous on `stream`, stream-ordered after the GEMM of the step:
 *   fp6m_peer_signal  increments this rank's device step counter and writes it, with system-scope release,
 *                     to slot `rank` of every rank's flag array (n arrays of n ints, zero at start)
 *   fp6m_peer_wait    holds the stream until every slot of this rank's own flag array has reached this rank's
 *                     step counter; bounded (about a second), then FP6M_ERR_TIMEOUT goes to `status_dev`.
 * Each rank runs the same sequence GEMM, signal, wait; the outputs should be double-buffered by the caller
 * (a rank may start writing step t+1 while another still reads step t). */
int fp6m_peer_alloc(size_t bytes, int dev, void** ptr, void* handle64);
int fp6m_peer_open(const void* handle64, int dev, void** ptr);
int fp6m_peer_close(void* ptr, int dev);
int fp6m_peer_free(void* ptr, int dev);
int fp6m_peer_signal(void* const* flag_arrays, int n, int rank, int* step_dev, int dev, void* stream);
int fp6m_peer_wait(const void* flags_local, int n, const int* step_dev, int* status_dev, int dev, void* stream);
/* Process-wide: how many times a wait polls a flag (sleeping at least 100 ns in between) before it gives up and
 * records FP6M_ERR_TIMEOUT; returns the previous value, a value <= 0 only queries.  Default 1 << 22 (about
 * half a second).  The reference's counterpart, barrier_acquire, spins without limit
 * (fp6_marlin_cuda_kernel.cu:79-86). */
int fp6m_set_peer_wait_polls(int polls);
/* fp6m_peer_signal followed by fp6m_peer_wait in one launch (flag_arrays[rank] is this rank's own array). */
int fp6m_peer_signal_wait(void* const* flag_arrays, int n, int rank, int* step_dev, int* status_dev, int dev, void* stream);
/* Test aid: enqueues a one-warp kernel that lets the kernels behind it launch at once (programmatic dependent
 * launch) and then stays busy for `milliseconds` (0..5000): a long-running predecessor for a GEMM with launch
 * overlap on, whose bounded waits must not start before that predecessor has finished.  No counterpart in the
 * reference. */
int fp6m_debug_busy_kernel(int milliseconds, int dev, void* stream);

/* Device-side weight preparation.  The reference prepares weights in single-threaded host loops
 * (fp6_marlin/weight_quant.cpp:106-124, fp6_marlin/weight_prepacking.cpp:123-177); these two do the same
 * work on the GPU, asynchronously on `stream`, with device pointers, and produce the same bytes as
 * fp6m_encode_fp6 and fp6m_pack_b200.  An out-of-range FP6 input is coded 0 and FP6M_ERR_VALUE_RANGE is
 * written to the optional device int `status_dev`.  No counterpart in the reference. */
int fp6m_encode_fp6_device(const void* w, void* codes, size_t count, int dev, void* stream, int* status_dev);
int fp6m_pack_b200_device(const void* q4, const void* c6, const void* s4, const void* s6, int K, int N, int quant_cols,
                          int group_size, void* B_out, void* s_out, int dev, void* stream);

/* Process-wide option, off by default; returns the previous setting (a negative argument only queries).
 * When on, the GEMM kernels are launched with programmatic stream serialisation: a GEMM may begin its
 * set-up and prefetch B while the kernel before it in the stream is still finishing.  Everything else
 * (A, C, scratch, workspace) is only touched after that kernel has completed.  Turn it on only when the
 * kernel that precedes a GEMM in its stream does not write that GEMM's B or s.  No counterpart in the
 * reference. */
int fp6m_set_launch_overlap(int enable);

/* Process-wide option, off by default; returns the previous setting (a negative argument only queries).
 * The GEMM for up to 128 rows of A normally lets two threads issue the tensor-core instructions of one
 * 128-row block, one per 64-row half, into one accumulator: the hardware may retire the halves in either
 * order, so the last bit of a result can differ between two runs on the same inputs (same products, same
 * fp32 adds, different order).  When on, one thread issues a block's instructions in a fixed order and two
 * runs agree bit for bit, at some cost in speed.  The reference's serial, lock-ordered reduction is
 * deterministic (fp6_marlin_cuda_kernel.cu:645-696). */
int fp6m_set_ordered_sums(int enable);

/* Message of the last CUDA error seen by this library on the calling thread ("" if none). */
const char* fp6m_last_cuda_error(void);

/* Library version tag, e.g. "fp6m-b200 0.1 (sm_100a)". */
const char* fp6m_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FP6M_H_ */
