// Parameter block shared by the host dispatcher and the GEMM kernels.  It travels by value in
// kernel parameter space (no host-to-device copy, safe under stream capture).
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "fp6m_layout.h"

namespace fp6m {

// Where the results go.  n_out == 0: to C (M x N, this GEMM's own columns).  n_out > 0 (N-sharded layer): the
// kernel stores every value straight into the full-width output buffers of all ranks (its own included; peer
// memory mapped through CUDA IPC), at the shard's place among the layer's columns - the all-gather of the output
// columns happens inside the epilogue, as plain stores over NVLink.
struct OutputMap {
  half* peer[8];
  int n_out;
  int ld;                // row stride of the full-width outputs = N of the whole layer
  int col4, col6;        // column of the whole layer where this shard's INT4 / FP6 columns start
};

// What happens to the fp32 sums (times the column scale) before they are rounded to fp16 and stored.
enum Epilogue {
  kEpilogueNone = 0,
  // gate / up projection pairs: columns 2j and 2j + 1 of each region hold gate_j and up_j; C has N / 2
  // columns and receives silu(gate_j) * up_j, INT4 pairs first, then FP6 pairs
  kEpilogueSiluMul = 1,
  // C = A W + R with R an M x N fp16 matrix laid out like C (R may be C itself)
  kEpilogueResidual = 2,
};

struct MulParams {
  const half* A;        // M x K, row-major
  const uint8_t* B;     // packed weights, b200 layout
  half* C;              // M x N (M x N / 2 with kEpilogueSiluMul), row-major
  const half* R;        // kEpilogueResidual: the matrix to add
  int epilogue;         // Epilogue
  const half* S;        // scales, b200 order
  int M, N, K;
  int row_tiles;        // wide kernel: tiles of rows of A covered by this launch (virtual strips = row_tiles x strips)
  Geometry geo;
  int* counters;        // one zero-initialised int per strip (the caller's workspace; left untouched)
  unsigned int* epochs;            // scratch header: [0] launch epoch, [1] CTAs of this launch that have read it
  unsigned long long* partials;    // split-K slots (scratch): {fp32 value, epoch tag} per 64-bit word
  int* status;          // optional device status word
  OutputMap out;
  int expand_early;     // kernel for up to 128 rows: the teams expand their first segments before the grid dependency
  int vec_rows;         // kernel for more than 128 rows: finished rows leave as 16-byte stores (every row start and both
                        // column bases are multiples of 8 halves, no fused epilogue)
  Schedule sched;
};

constexpr int kEpochWords = 64;     // scratch header size in 32-bit words

// gemm_tc5.cu
int tc5_ctas_per_sm(int rows);
int tc5_tile_rows(int rows);
#ifndef FP6M_TC5_MAX_ROWS
#define FP6M_TC5_MAX_ROWS 128
#endif
constexpr int kTc5MaxRows = FP6M_TC5_MAX_ROWS;     // rows of A the kernel of gemm_tc5.cu covers; more rows go to gemm_wide.cu
size_t tc5_scratch_bytes(int ctas, int rows);
void tc5_set_overlap(bool on);
bool tc5_get_overlap();
void tc5_set_ordered_sums(bool on);
bool tc5_get_ordered_sums();
cudaError_t launch_gemm_tc5(const MulParams& p, cudaStream_t stream);

// gemm_wide.cu
cudaError_t encode_activation_map(const half* A, int M, int K, int box_rows, CUtensorMap* map);
cudaError_t encode_activation_segment_map(const half* A, int M, int K, int box_rows, CUtensorMap* map);
cudaError_t encode_output_map(const half* base, int rows, int ld, CUtensorMap* map);
constexpr int kMaxWideCtas = 192;   // one CTA per SM
constexpr int kMaxRowTiles = 32;    // 8192 rows of A per launch
int wide_rows_per_pass();
int wide_tile_rows(int rows);
size_t wide_scratch_bytes(int ctas, int rows);
cudaError_t launch_gemm_wide(const MulParams& p, int tile_rows, cudaStream_t stream);

// dump_operands.cu
cudaError_t launch_dump_operands(const uint8_t* B, const half* S, half* W, const Geometry& geo, cudaStream_t stream);

}  // namespace fp6m
