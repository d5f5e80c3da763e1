// Debug kernel: writes the fp16 values that the GEMM kernels hand to the tensor cores as a plain
// K x N matrix, using the very same device dequantisers (device_utils.cuh).  A test compares it
// bit-for-bit with the reference's dequantisation rules (test.py:98 for INT4,
// weight_prepacking.cpp:199-212 for FP6).
#include "device_utils.cuh"
#include "gemm_params.h"

namespace fp6m {

namespace {

__global__ void dump_operands_kernel(const uint8_t* __restrict__ B, const half* __restrict__ S,
                                     half* __restrict__ W, Geometry geo) {
  // one thread per (strip, kb, w, jq, lane); it expands its four words (jr = 0..3)
  const int strips = geo.strips4 + geo.strips6;
  const long long total = (long long)strips * geo.k128 * 4 * 4 * 32;
  const half2 k4096 = __float2half2_rn(4096.0f);
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int lane = idx & 31;
    const int jq = (idx >> 5) & 3;
    const int w = (idx >> 7) & 3;
    const long long blk = idx >> 9;
    const int kb = (int)(blk % geo.k128);
    const int strip_lin = (int)(blk / geo.k128);
    const bool is6 = strip_lin >= geo.strips4;
    const int strip = is6 ? strip_lin - geo.strips4 : strip_lin;
    const int ncols_region = is6 ? geo.n6 : geo.n4;
    const int nq = strip_quads(ncols_region, strip);
    if (jq >= nq) continue;
    const int g = lane >> 2, t = lane & 3;
    const uint8_t* base = B + (is6 ? fp6_block_offset(geo, strip, kb) : int4_block_offset(geo, strip, kb));
    const uint4 q = reinterpret_cast<const uint4*>(base)[(w * nq + jq) * 32 + lane];
    uint2 two = make_uint2(0, 0);
    if (is6) two = reinterpret_cast<const uint2*>(base + nq * kInt4QuadBytes)[(w * nq + jq) * 32 + lane];
    const int group = (!is6 && geo.groups > 1) ? kb : 0;
    const half* sp = S + (is6 ? fp6_scale_offset(geo, strip) : int4_scale_offset(geo, strip, group));
    const uint32_t qs[4] = {q.x, q.y, q.z, q.w};
    for (int jr = 0; jr < 4; ++jr) {
      half2 s2 = __half2half2(sp[scale_index(8 * (4 * jq + jr) + g, nq)]);
      uint32_t b[4];
      if (is6) {
        s2 = __hmul2(s2, k4096);
        dequant_fp6_word(qs[jr], (jr < 2) ? two.x : two.y, 4 * (jr & 1), s2, b);
      } else {
        dequant_int4_word(qs[jr], s2, b);
      }
      const int col = strip * kStripCols + 8 * (4 * jq + jr) + g;
      if (col >= ncols_region) continue;
      const int gcol = (is6 ? geo.n4 : 0) + col;
      for (int i = 0; i < 8; ++i) {
        const int row = kb * kBlockRows + 32 * w + 8 * t + i;
        if (row >= geo.K) continue;
        const half2 pair = u32_as_h2(b[i >> 1]);
        W[(size_t)row * geo.N + gcol] = (i & 1) ? __high2half(pair) : __low2half(pair);
      }
    }
  }
}

}  // namespace

cudaError_t launch_dump_operands(const uint8_t* B, const half* S, half* W, const Geometry& geo, cudaStream_t stream) {
  const long long total = (long long)(geo.strips4 + geo.strips6) * geo.k128 * 512;
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  dump_operands_kernel<<<blocks, 256, 0, stream>>>(B, S, W, geo);
  return cudaGetLastError();
}

}  // namespace fp6m
