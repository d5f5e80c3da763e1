// Device-side weight preparation: the truncating fp16 -> FP6 E3M2 cast and the packing of logical
// INT4 / FP6 codes and scales into the b200 layout, bit for bit what the host functions of
// host_pack.cpp produce.  The reference prepares weights in single-threaded host loops
// (fp6_marlin/weight_quant.cpp:106-124, fp6_marlin/weight_prepacking.cpp:123-177); for 70B-scale
// layers that takes seconds per layer, here it is a few memory-bound kernels.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/fp6m.h"
#include "fp6m_layout.h"

namespace fp6m {

namespace {

// fp16 bits -> code `s eee mm`, mantissa truncated, FP6 subnormals by shifting the mantissa with its
// implicit one (weight_quant.cpp:27-91); values outside {0} U [0.0625, 28] are reported and coded 0.
__global__ void encode_fp6_kernel(const uint16_t* __restrict__ w, uint8_t* __restrict__ codes, size_t count, int* status) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const uint16_t h = w[i];
  const int sign = h >> 15, exp = (h >> 10) & 0x1F, man = h & 0x3FF;
  const uint16_t mag = h & 0x7FFF;
  uint8_t code = 0;
  if ((mag != 0 && mag < 0x2C00) || mag > 0x4F00) {
    if (status) atomicExch(status, FP6M_ERR_VALUE_RANGE);
  } else {
    int e6 = 0, m6 = 0;
    if (exp != 0) {
      const int unbiased = exp - 15;
      m6 = man >> 8;
      if (unbiased < -2) {
        m6 = (m6 | 4) >> (-2 - unbiased);
      } else {
        e6 = unbiased + 3;
      }
    }
    code = (uint8_t)((sign << 5) | (e6 << 2) | m6);
  }
  codes[i] = code;
}

// one thread per (strip, unit, column): the column's eight words of the unit
__global__ void pack_int4_kernel(const uint8_t* __restrict__ q4, Geometry geo, uint8_t* __restrict__ B_out) {
  const int ups = units_per_strip(geo);
  const int c = threadIdx.x;                          // column inside the strip
  const int unit = blockIdx.x % ups, strip = blockIdx.x / ups;
  const int nq = strip_quads(geo.n4, strip);
  if (c >= kQuadCols * nq) return;
  uint8_t* base = B_out + int4_unit_offset(geo, strip, unit);
  const int col = strip * kStripCols + c;
  for (int w8 = 0; w8 < 8; ++w8) {
    uint32_t word = 0;
    for (int i = 0; i < 8; ++i) {
      const int row = unit * kUnitRows + 8 * w8 + i;
      uint32_t q = 8;                                 // padding dequantises to zero
      if (row < geo.K && col < geo.n4) q = q4[(size_t)row * geo.n4 + col] & 15u;
      word |= q << (4 * int4_nibble_pos(i));
    }
    *reinterpret_cast<uint32_t*>(base + word_offset(c, w8)) = word;
  }
}

__global__ void pack_fp6_kernel(const uint8_t* __restrict__ c6, Geometry geo, uint8_t* __restrict__ B_out) {
  const int ups = units_per_strip(geo);
  const int c = threadIdx.x;
  const int unit = blockIdx.x % ups, strip = blockIdx.x / ups;
  const int nq = strip_quads(geo.n6, strip);
  if (c >= kQuadCols * nq) return;
  uint8_t* base = B_out + fp6_unit_offset(geo, strip, unit);
  uint8_t* base2 = base + (size_t)nq * kInt4UnitQuadBytes;
  const int col = strip * kStripCols + c;
  uint32_t two[4] = {0, 0, 0, 0};
  for (int w8 = 0; w8 < 8; ++w8) {
    uint32_t four = 0;
    for (int i = 0; i < 8; ++i) {
      const int row = unit * kUnitRows + 8 * w8 + i;
      uint32_t code = 0;
      if (row < geo.K && col < geo.n6) code = c6[(size_t)row * geo.n6 + col] & 63u;
      const int b = i & 3, js = 2 * (w8 & 1) + (i >> 2);
      four |= (code & 15u) << (8 * b + 4 * (i >> 2));
      two[w8 >> 1] |= ((code >> 5) & 1u) << ((8 * b + 7 - 2 * js + 32) & 31);
      two[w8 >> 1] |= ((code >> 4) & 1u) << ((8 * b + 4 - 2 * js + 32) & 31);
    }
    *reinterpret_cast<uint32_t*>(base + word_offset(c, w8)) = four;
  }
  *reinterpret_cast<uint4*>(base2 + c * 16) = make_uint4(two[0], two[1], two[2], two[3]);
}

// scales in plain column order per strip (and per group); padding columns get 1.0
__global__ void pack_scales_kernel(const uint16_t* __restrict__ s4, const uint16_t* __restrict__ s6, Geometry geo,
                                   uint16_t* __restrict__ s_out) {
  const int c = threadIdx.x;
  const int rows4 = geo.strips4 * geo.groups;
  const int b = blockIdx.x;
  if (b < rows4) {
    const int strip = b / geo.groups, grp = b % geo.groups;
    if (c >= kQuadCols * strip_quads(geo.n4, strip)) return;
    const int col = strip * kStripCols + c;
    s_out[int4_scale_offset(geo, strip, grp) + c] = col < geo.n4 ? s4[(size_t)grp * geo.n4 + col] : (uint16_t)0x3C00;
  } else {
    const int strip = b - rows4;
    if (c >= kQuadCols * strip_quads(geo.n6, strip)) return;
    const int col = strip * kStripCols + c;
    s_out[fp6_scale_offset(geo, strip) + c] = col < geo.n6 ? s6[col] : (uint16_t)0x3C00;
  }
}

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

}  // namespace
}  // namespace fp6m

using namespace fp6m;

extern "C" {

int fp6m_encode_fp6_device(const void* w, void* codes, size_t count, int dev, void* stream, int* status_dev) {
  if (!w || !codes) return FP6M_ERR_BAD_ARG;
  if (count == 0) return FP6M_OK;
  Guard guard(dev);
  const int threads = 256;
  const size_t blocks = (count + threads - 1) / threads;
  if (blocks > 0x7fffffffu) return FP6M_ERR_BAD_ARG;
  encode_fp6_kernel<<<(unsigned)blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(w), static_cast<uint8_t*>(codes), count, status_dev);
  return cudaGetLastError() == cudaSuccess ? FP6M_OK : FP6M_ERR_CUDA;
}

int fp6m_pack_b200_device(const void* q4, const void* c6, const void* s4, const void* s6, int K, int N, int qc, int group_size,
                          void* B_out, void* s_out, int dev, void* stream) {
  if (K <= 0 || N <= 0 || qc > N || !B_out || !s_out) return FP6M_ERR_BAD_ARG;
  if (!(group_size == 128 || group_size <= 0)) return FP6M_ERR_BAD_ARG;
  const Geometry geo = make_geometry(K, N, qc, group_size);
  if ((geo.n4 > 0 && (!q4 || !s4)) || (geo.n6 > 0 && (!c6 || !s6))) return FP6M_ERR_BAD_ARG;
  Guard guard(dev);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int ups = units_per_strip(geo);
  if (geo.strips4 > 0)
    pack_int4_kernel<<<geo.strips4 * ups, kStripCols, 0, st>>>(static_cast<const uint8_t*>(q4), geo, static_cast<uint8_t*>(B_out));
  if (geo.strips6 > 0)
    pack_fp6_kernel<<<geo.strips6 * ups, kStripCols, 0, st>>>(static_cast<const uint8_t*>(c6), geo, static_cast<uint8_t*>(B_out));
  pack_scales_kernel<<<geo.strips4 * geo.groups + geo.strips6, kStripCols, 0, st>>>(
      static_cast<const uint16_t*>(s4), static_cast<const uint16_t*>(s6), geo, static_cast<uint16_t*>(s_out));
  return cudaGetLastError() == cudaSuccess ? FP6M_OK : FP6M_ERR_CUDA;
}

}  // extern "C"
