// Debug kernel: expands a packed b200 weight buffer to the plain K x N fp16 matrix W_deq with the
// expanders the GEMM kernels themselves use (tc5_common.cuh: exact q - 8 or exact E3M2 value / 4096),
// times the scale with one fp16 rounding.  A test compares it bit-for-bit with the reference's
// dequantisation rules (test.py:98 for INT4, weight_prepacking.cpp:199-212 for FP6).  The GEMM for
// more than 128 rows feeds exactly these values to the tensor cores for group-scaled INT4 columns; in
// the other cases the kernels feed the unscaled expansion and apply the scale to the fp32 sums.
#include "device_utils.cuh"
#include "gemm_params.h"
#include "tc5_common.cuh"

namespace fp6m {

namespace {

__global__ void dump_operands_kernel(const uint8_t* __restrict__ B, const half* __restrict__ S,
                                     half* __restrict__ W, Geometry geo) {
  // one thread per (strip, unit, column)
  const int ups = units_per_strip(geo);
  const int strips = geo.strips4 + geo.strips6;
  const long long total = (long long)strips * ups * kStripCols;
  const half2 k4096 = __float2half2_rn(4096.0f);
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(idx % kStripCols);
    const int unit = (int)((idx / kStripCols) % ups);
    const int strip_lin = (int)(idx / ((long long)kStripCols * ups));
    const bool is6 = strip_lin >= geo.strips4;
    const int strip = is6 ? strip_lin - geo.strips4 : strip_lin;
    const int ncols_region = is6 ? geo.n6 : geo.n4;
    const int col = strip * kStripCols + c;
    if (col >= ncols_region) continue;
    const int nq = strip_quads(ncols_region, strip);
    const uint8_t* base = B + (is6 ? fp6_unit_offset(geo, strip, unit) : int4_unit_offset(geo, strip, unit));
    const int group = (!is6 && geo.groups > 1) ? (unit >> 1) : 0;
    const half sc = S[(is6 ? fp6_scale_offset(geo, strip) : int4_scale_offset(geo, strip, group)) + c];
    half2 s2 = __half2half2(sc);
    if (is6) s2 = __hmul2(s2, k4096);
    const int gcol = (is6 ? geo.n4 : 0) + col;
    for (int w8 = 0; w8 < 8; ++w8) {
      const uint32_t word = *reinterpret_cast<const uint32_t*>(base + word_offset(c, w8));
      uint32_t b[4];
      if (is6) {
        const uint32_t two = *reinterpret_cast<const uint32_t*>(base + nq * kInt4UnitQuadBytes + c * 16 + (w8 >> 1) * 4);
        expand_fp6_scaled(word, two, 4 * (w8 & 1), s2, b);
      } else {
        expand_int4_scaled(word, s2, b);
      }
      for (int i = 0; i < 8; ++i) {
        const int row = unit * kUnitRows + 8 * w8 + i;
        if (row >= geo.K) continue;
        const half2 pair = u32_as_h2(b[i >> 1]);
        W[(size_t)row * geo.N + gcol] = (i & 1) ? __high2half(pair) : __low2half(pair);
      }
    }
  }
}

}  // namespace

cudaError_t launch_dump_operands(const uint8_t* B, const half* S, half* W, const Geometry& geo, cudaStream_t stream) {
  const long long total = (long long)(geo.strips4 + geo.strips6) * units_per_strip(geo) * kStripCols;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  dump_operands_kernel<<<blocks, 256, 0, stream>>>(B, S, W, geo);
  return cudaGetLastError();
}

}  // namespace fp6m
