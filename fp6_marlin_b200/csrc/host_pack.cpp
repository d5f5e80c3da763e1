// Host-side weight preparation behind the C ABI (include/fp6m.h): FP6 E3M2 cast and stream
// packing, the reference's "2+4" tensor-core layout, FP6 dequantisation, and the Blackwell
// ("b200") tiling with its converters.  Pure integer / fp16 work, multi-threaded over rows or
// blocks; nothing here touches the GPU.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

#include "../../include/fp6m.h"
#include "fp6m_layout.h"

namespace {

using namespace fp6m;

// ---- small fp16 helpers (host, no CUDA headers needed) ---------------------------------------
inline float half_bits_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h >> 15) << 31;
  uint32_t exp = (h >> 10) & 0x1F;
  uint32_t man = h & 0x3FF;
  uint32_t f;
  if (exp == 0) {
    if (man == 0) {
      f = sign;
    } else {  // subnormal: normalise
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400));
      f = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
    }
  } else if (exp == 31) {
    f = sign | 0x7F800000u | (man << 13);
  } else {
    f = sign | ((exp + 112) << 23) | (man << 13);
  }
  float out;
  std::memcpy(&out, &f, 4);
  return out;
}

// float -> fp16 bits, round to nearest even (values here are finite).
inline uint16_t float_to_half_bits(float x) {
  uint32_t f;
  std::memcpy(&f, &x, 4);
  uint32_t sign = (f >> 16) & 0x8000;
  int32_t exp = (int32_t)((f >> 23) & 0xFF) - 127 + 15;
  uint32_t man = f & 0x7FFFFF;
  if (((f >> 23) & 0xFF) == 0xFF) return (uint16_t)(sign | 0x7C00 | (man ? 0x200 : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7C00);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000;
    int shift = 14 - exp;
    uint32_t half_man = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_man & 1))) ++half_man;
    return (uint16_t)(sign | half_man);
  }
  uint32_t half_man = man >> 13;
  uint32_t rem = man & 0x1FFF;
  uint16_t out = (uint16_t)(sign | ((uint32_t)exp << 10) | half_man);
  if (rem > 0x1000 || (rem == 0x1000 && (half_man & 1))) ++out;  // carry into the exponent is correct
  return out;
}

// One fp16 multiply with a single rounding (the product of two fp16 values is exact in fp32).
inline uint16_t half_mul(uint16_t a, uint16_t b) {
  return float_to_half_bits(half_bits_to_float(a) * half_bits_to_float(b));
}

template <typename F>
void parallel_for(size_t n, F&& body) {
  unsigned hw = std::thread::hardware_concurrency();
  size_t threads = std::min<size_t>(hw ? hw : 1, 16);
  if (n < 64 || threads <= 1) { body(0, n); return; }
  threads = std::min(threads, n);
  std::vector<std::thread> pool;
  size_t chunk = (n + threads - 1) / threads;
  for (size_t t = 0; t < threads; ++t) {
    size_t lo = t * chunk, hi = std::min(n, lo + chunk);
    if (lo >= hi) break;
    pool.emplace_back([=, &body] { body(lo, hi); });
  }
  for (auto& th : pool) th.join();
}

// ---- FP6 E3M2 ---------------------------------------------------------------------------------
// fp16 bits -> 6-bit code `s eee mm`, truncating (weight_quant.cpp:27-91).  Returns false when the
// value is outside {0} U [0.0625, 28].
inline bool fp6_encode(uint16_t h, uint8_t* code) {
  const int sign = h >> 15;
  const int exp = (h >> 10) & 0x1F;
  const int man = h & 0x3FF;
  const uint16_t mag = h & 0x7FFF;
  // 0.0625 = 0x2C00, 28 = 0x4F00 as fp16 magnitudes; NaN/inf have exp 31 and fail the upper test.
  if ((mag != 0 && mag < 0x2C00) || mag > 0x4F00) return false;
  int e6 = 0, m6 = 0;
  if (exp != 0) {
    const int unbiased = exp - 15;
    m6 = man >> 8;
    if (unbiased < -2) {             // FP6 subnormal: shift the mantissa with its implicit one
      m6 = (m6 | 4) >> (-2 - unbiased);
      e6 = 0;
    } else {
      e6 = unbiased + 3;
    }
  }
  *code = (uint8_t)((sign << 5) | (e6 << 2) | m6);
  return true;
}

// Exact value of a code as fp16 bits: `s 00eee mm 00000000` times 2^12 (weight_prepacking.cpp:199-212).
inline uint16_t fp6_code_to_half(uint8_t c) {
  const int s = c >> 5, e = (c >> 2) & 7, m = c & 3;
  if (e == 0) {
    // m/16: 0, 0.0625, 0.125, 0.1875
    static const uint16_t sub[4] = {0x0000, 0x2C00, 0x3000, 0x3200};
    return (uint16_t)((s << 15) | sub[m]);
  }
  return (uint16_t)((s << 15) | ((e + 12) << 10) | (m << 8));
}

inline uint8_t stream_code(const uint8_t* stream, size_t idx) {
  const uint8_t* p = stream + (idx >> 2) * 3;
  switch (idx & 3) {
    case 0: return p[0] >> 2;
    case 1: return (uint8_t)(((p[0] & 3) << 4) | (p[1] >> 4));
    case 2: return (uint8_t)(((p[1] & 15) << 2) | (p[2] >> 6));
    default: return p[2] & 63;
  }
}

// ---- reference fragment order ----------------------------------------------------------------
// Lane 4g+t of chunk (kb, ch) holds, for sub-tile j and half h, v0..v3 at rows
// 16kb + {2t, 2t+1, 2t+8, 2t+9} and column 64ch + 16j + 8h + g (test.py:60-79).
inline int frag_row(int kb, int t, int v) { return 16 * kb + 2 * t + (v & 1) + 8 * (v >> 1); }
inline int frag_col(int ch, int j, int h, int g) { return 64 * ch + 16 * j + 8 * h + g; }
// Byte (0 = least significant) of a (j, h) group that carries value v in the FP6 "2+4" words.
constexpr int kByteOfV[4] = {1, 3, 0, 2};
// Scale order inside every aligned group of 32 columns (test.py:48-53).
inline int ref_scale_perm(int i) {
  static const int tail[8] = {0, 1, 8, 9, 16, 17, 24, 25};
  return 2 * (i / 8) + tail[i % 8];
}

}  // namespace

extern "C" {

int fp6m_quantize_fp6(const uint16_t* w, uint8_t* out, size_t rows, size_t cols) {
  if (!w || !out || cols % 4) return FP6M_ERR_BAD_ARG;
  std::vector<int> bad(1, 0);
  int* bad_flag = bad.data();
  parallel_for(rows, [=](size_t lo, size_t hi) {
    for (size_t r = lo; r < hi; ++r) {
      const uint16_t* src = w + r * cols;
      uint8_t* dst = out + r * (cols / 4 * 3);
      for (size_t c = 0; c < cols; c += 4, dst += 3) {
        uint8_t q[4];
        for (int i = 0; i < 4; ++i)
          if (!fp6_encode(src[c + i], &q[i])) { *bad_flag = 1; q[i] = 0; }
        dst[0] = (uint8_t)((q[0] << 2) | (q[1] >> 4));
        dst[1] = (uint8_t)(((q[1] & 15) << 4) | (q[2] >> 2));
        dst[2] = (uint8_t)(((q[2] & 3) << 6) | q[3]);
      }
    }
  });
  return bad[0] ? FP6M_ERR_VALUE_RANGE : FP6M_OK;
}

int fp6m_encode_fp6(const uint16_t* w, uint8_t* codes, size_t count) {
  if (!w || !codes) return FP6M_ERR_BAD_ARG;
  std::vector<int> bad(1, 0);
  int* bad_flag = bad.data();
  parallel_for(count, [=](size_t lo, size_t hi) {
    for (size_t i = lo; i < hi; ++i)
      if (!fp6_encode(w[i], &codes[i])) { *bad_flag = 1; codes[i] = 0; }
  });
  return bad[0] ? FP6M_ERR_VALUE_RANGE : FP6M_OK;
}

int fp6m_prepack_fp6(const uint8_t* fp6, uint8_t* out, size_t n, size_t k) {
  if (!fp6 || !out || n % 64 || k % 64) return FP6M_ERR_BAD_ARG;
  uint32_t* w2 = reinterpret_cast<uint32_t*>(out);
  uint32_t* w4 = w2 + k * n / 16;
  const size_t chunks_n = n / 64;
  parallel_for(k / 16, [=](size_t lo, size_t hi) {
    for (size_t kb = lo; kb < hi; ++kb)
      for (size_t ch = 0; ch < chunks_n; ++ch)
        for (int lane = 0; lane < 32; ++lane) {
          const int g = lane >> 2, t = lane & 3;
          const size_t base = (kb * chunks_n + ch) * 32 + lane;
          uint32_t two[2] = {0, 0}, four[4] = {0, 0, 0, 0};
          for (int j = 0; j < 4; ++j)
            for (int h = 0; h < 2; ++h)
              for (int v = 0; v < 4; ++v) {
                const size_t row = frag_row((int)kb, t, v), col = frag_col((int)ch, j, h, g);
                const uint32_t code = stream_code(fp6, col * k + row);   // stream is (n, k) row-major
                const int by = kByteOfV[v];
                four[j] |= (code & 15u) << (8 * by + (h == 0 ? 4 : 0));
                two[j >> 1] |= (code >> 4) << (8 * by + 6 - (4 * (j & 1) + 2 * h));
              }
          w2[base * 2 + 0] = two[0];
          w2[base * 2 + 1] = two[1];
          for (int j = 0; j < 4; ++j) w4[base * 4 + j] = four[j];
        }
  });
  return FP6M_OK;
}

int fp6m_dequant_fp6(const uint8_t* fp6, const uint16_t* scale, uint16_t* out, size_t n, size_t k) {
  if (!fp6 || !scale || !out || k % 4) return FP6M_ERR_BAD_ARG;
  parallel_for(n, [=](size_t lo, size_t hi) {
    for (size_t r = lo; r < hi; ++r) {
      const uint16_t s = scale[r];
      for (size_t c = 0; c < k; ++c)
        out[r * k + c] = half_mul(fp6_code_to_half(stream_code(fp6, r * k + c)), s);
    }
  });
  return FP6M_OK;
}

int64_t fp6m_b200_weight_bytes(int K, int N, int qc) {
  if (K <= 0 || N <= 0 || qc > N) return -1;
  return weight_bytes(make_geometry(K, N, qc, -1));
}

int64_t fp6m_b200_scale_count(int K, int N, int qc, int group_size) {
  if (K <= 0 || N <= 0 || qc > N || !(group_size == 128 || group_size <= 0)) return -1;
  return scale_count(make_geometry(K, N, qc, group_size));
}

int fp6m_pack_b200(const uint8_t* q4, const uint8_t* c6, const uint16_t* s4, const uint16_t* s6,
                   int K, int N, int qc, int group_size, uint8_t* B_out, uint16_t* s_out) {
  if (K <= 0 || N <= 0 || qc > N || !B_out || !s_out) return FP6M_ERR_BAD_ARG;
  if (!(group_size == 128 || group_size <= 0)) return FP6M_ERR_BAD_ARG;
  const Geometry geo = make_geometry(K, N, qc, group_size);
  if ((geo.n4 > 0 && (!q4 || !s4)) || (geo.n6 > 0 && (!c6 || !s6))) return FP6M_ERR_BAD_ARG;
  const int ups = units_per_strip(geo);

  // INT4 units
  parallel_for((size_t)geo.strips4 * ups, [=](size_t lo, size_t hi) {
    for (size_t idx = lo; idx < hi; ++idx) {
      const int strip = (int)(idx / ups), unit = (int)(idx % ups);
      const int nq = strip_quads(geo.n4, strip);
      uint8_t* base = B_out + int4_unit_offset(geo, strip, unit);
      for (int c = 0; c < kQuadCols * nq; ++c)
        for (int w8 = 0; w8 < 8; ++w8) {
          const int col = strip * kStripCols + c;
          uint32_t word = 0;
          for (int i = 0; i < 8; ++i) {
            const int row = unit * kUnitRows + 8 * w8 + i;
            uint32_t q = 8;
            if (row < K && col < geo.n4) q = q4[(size_t)row * geo.n4 + col] & 15u;
            word |= q << (4 * int4_nibble_pos(i));
          }
          std::memcpy(base + word_offset(c, w8), &word, 4);
        }
    }
  });
  // FP6 units
  parallel_for((size_t)geo.strips6 * ups, [=](size_t lo, size_t hi) {
    for (size_t idx = lo; idx < hi; ++idx) {
      const int strip = (int)(idx / ups), unit = (int)(idx % ups);
      const int nq = strip_quads(geo.n6, strip);
      uint8_t* base = B_out + fp6_unit_offset(geo, strip, unit);
      uint8_t* base2 = base + (size_t)nq * kInt4UnitQuadBytes;
      for (int c = 0; c < kQuadCols * nq; ++c) {
        const int col = strip * kStripCols + c;
        uint32_t two[4] = {0, 0, 0, 0};
        for (int w8 = 0; w8 < 8; ++w8) {
          uint32_t four = 0;
          for (int i = 0; i < 8; ++i) {
            const int row = unit * kUnitRows + 8 * w8 + i;
            uint32_t code = 0;
            if (row < K && col < geo.n6) code = c6[(size_t)row * geo.n6 + col] & 63u;
            const int b = i & 3, js = 2 * (w8 & 1) + (i >> 2);
            four |= (code & 15u) << (8 * b + 4 * (i >> 2));
            two[w8 >> 1] |= ((code >> 5) & 1u) << ((8 * b + 7 - 2 * js + 32) & 31);
            two[w8 >> 1] |= ((code >> 4) & 1u) << ((8 * b + 4 - 2 * js + 32) & 31);
          }
          std::memcpy(base + word_offset(c, w8), &four, 4);
        }
        std::memcpy(base2 + c * 16, two, 16);
      }
    }
  });
  // scales, plain column order, padding columns get 1.0
  const uint16_t one = 0x3C00;
  for (int strip = 0; strip < geo.strips4; ++strip) {
    const int nq = strip_quads(geo.n4, strip);
    for (int grp = 0; grp < geo.groups; ++grp) {
      uint16_t* dst = s_out + int4_scale_offset(geo, strip, grp);
      for (int c = 0; c < kQuadCols * nq; ++c) {
        const int col = strip * kStripCols + c;
        dst[c] = col < geo.n4 ? s4[(size_t)grp * geo.n4 + col] : one;
      }
    }
  }
  for (int strip = 0; strip < geo.strips6; ++strip) {
    const int nq = strip_quads(geo.n6, strip);
    uint16_t* dst = s_out + fp6_scale_offset(geo, strip);
    for (int c = 0; c < kQuadCols * nq; ++c) {
      const int col = strip * kStripCols + c;
      dst[c] = col < geo.n6 ? s6[col] : one;
    }
  }
  return FP6M_OK;
}

int fp6m_unpack_b200(const uint8_t* B, const uint16_t* s, int K, int N, int qc, int group_size,
                     uint8_t* q4, uint8_t* c6, uint16_t* s4, uint16_t* s6) {
  if (K <= 0 || N <= 0 || qc > N || !B || !s) return FP6M_ERR_BAD_ARG;
  if (!(group_size == 128 || group_size <= 0)) return FP6M_ERR_BAD_ARG;
  const Geometry geo = make_geometry(K, N, qc, group_size);
  if ((geo.n4 > 0 && (!q4 || !s4)) || (geo.n6 > 0 && (!c6 || !s6))) return FP6M_ERR_BAD_ARG;
  const int ups = units_per_strip(geo);
  for (int strip = 0; strip < geo.strips4; ++strip) {
    const int nq = strip_quads(geo.n4, strip);
    for (int unit = 0; unit < ups; ++unit) {
      const uint8_t* base = B + int4_unit_offset(geo, strip, unit);
      for (int c = 0; c < kQuadCols * nq; ++c)
        for (int w8 = 0; w8 < 8; ++w8) {
          const int col = strip * kStripCols + c;
          uint32_t word;
          std::memcpy(&word, base + word_offset(c, w8), 4);
          for (int i = 0; i < 8; ++i) {
            const int row = unit * kUnitRows + 8 * w8 + i;
            if (row < K && col < geo.n4)
              q4[(size_t)row * geo.n4 + col] = (word >> (4 * int4_nibble_pos(i))) & 15u;
          }
        }
    }
    for (int grp = 0; grp < geo.groups; ++grp) {
      const uint16_t* src = s + int4_scale_offset(geo, strip, grp);
      for (int c = 0; c < kQuadCols * nq; ++c) {
        const int col = strip * kStripCols + c;
        if (col < geo.n4) s4[(size_t)grp * geo.n4 + col] = src[c];
      }
    }
  }
  for (int strip = 0; strip < geo.strips6; ++strip) {
    const int nq = strip_quads(geo.n6, strip);
    for (int unit = 0; unit < ups; ++unit) {
      const uint8_t* base = B + fp6_unit_offset(geo, strip, unit);
      const uint8_t* base2 = base + (size_t)nq * kInt4UnitQuadBytes;
      for (int c = 0; c < kQuadCols * nq; ++c) {
        const int col = strip * kStripCols + c;
        uint32_t two[4];
        std::memcpy(two, base2 + c * 16, 16);
        for (int w8 = 0; w8 < 8; ++w8) {
          uint32_t four;
          std::memcpy(&four, base + word_offset(c, w8), 4);
          for (int i = 0; i < 8; ++i) {
            const int row = unit * kUnitRows + 8 * w8 + i;
            const int b = i & 3, js = 2 * (w8 & 1) + (i >> 2);
            const uint32_t lo = (four >> (8 * b + 4 * (i >> 2))) & 15u;
            const uint32_t sg = (two[w8 >> 1] >> ((8 * b + 7 - 2 * js + 32) & 31)) & 1u;
            const uint32_t e2 = (two[w8 >> 1] >> ((8 * b + 4 - 2 * js + 32) & 31)) & 1u;
            if (row < K && col < geo.n6)
              c6[(size_t)row * geo.n6 + col] = (uint8_t)((sg << 5) | (e2 << 4) | lo);
          }
        }
      }
    }
    const uint16_t* src = s + fp6_scale_offset(geo, strip);
    for (int c = 0; c < kQuadCols * nq; ++c) {
      const int col = strip * kStripCols + c;
      if (col < geo.n6) s6[col] = src[c];
    }
  }
  return FP6M_OK;
}

int fp6m_unpack_reference(const uint8_t* B_ref, const uint16_t* s_ref, int K, int N, int qc,
                          uint8_t* q4, uint8_t* c6, uint16_t* s4, uint16_t* s6) {
  if (K <= 0 || N <= 0 || qc > N || !B_ref || !s_ref) return FP6M_ERR_BAD_ARG;
  const int n6 = qc < 0 ? 0 : qc, n4 = N - n6;
  if (K % 16 || n4 % 64 || n6 % 64) return FP6M_ERR_PROB_SHAPE;
  if ((n4 > 0 && (!q4 || !s4)) || (n6 > 0 && (!c6 || !s6))) return FP6M_ERR_BAD_ARG;
  const uint32_t* int4_words = reinterpret_cast<const uint32_t*>(B_ref);
  const uint32_t* fp6_two = int4_words + (size_t)K * n4 / 8;          // INT4 region is K*n4/2 bytes
  const uint32_t* fp6_four = fp6_two + (size_t)K * n6 / 16;
  static const int nib_src[8] = {0, 2, 4, 6, 1, 3, 5, 7};             // nibble p holds value index
  for (int kb = 0; kb < K / 16; ++kb) {
    for (int ch = 0; ch < n4 / 64; ++ch)
      for (int lane = 0; lane < 32; ++lane) {
        const int g = lane >> 2, t = lane & 3;
        for (int j = 0; j < 4; ++j) {
          const uint32_t word = int4_words[(((size_t)kb * (n4 / 64) + ch) * 32 + lane) * 4 + j];
          for (int p = 0; p < 8; ++p) {
            const int vi = nib_src[p], h = vi >> 2, v = vi & 3;
            q4[(size_t)frag_row(kb, t, v) * n4 + frag_col(ch, j, h, g)] = (word >> (4 * p)) & 15u;
          }
        }
      }
    for (int ch = 0; ch < n6 / 64; ++ch)
      for (int lane = 0; lane < 32; ++lane) {
        const int g = lane >> 2, t = lane & 3;
        const size_t base = ((size_t)kb * (n6 / 64) + ch) * 32 + lane;
        for (int j = 0; j < 4; ++j)
          for (int h = 0; h < 2; ++h)
            for (int v = 0; v < 4; ++v) {
              const int by = kByteOfV[v];
              const uint32_t lo = (fp6_four[base * 4 + j] >> (8 * by + (h == 0 ? 4 : 0))) & 15u;
              const uint32_t hi = (fp6_two[base * 2 + (j >> 1)] >> (8 * by + 6 - (4 * (j & 1) + 2 * h))) & 3u;
              c6[(size_t)frag_row(kb, t, v) * n6 + frag_col(ch, j, h, g)] = (uint8_t)((hi << 4) | lo);
            }
      }
  }
  for (int i = 0; i < n4; ++i) s4[(i / 32) * 32 + ref_scale_perm(i % 32)] = s_ref[i];
  for (int i = 0; i < n6; ++i) s6[(i / 32) * 32 + ref_scale_perm(i % 32)] = s_ref[n4 + i];
  return FP6M_OK;
}

int fp6m_repack_from_reference(const uint8_t* B_ref, const uint16_t* s_ref, int K, int N, int qc,
                               uint8_t* B_out, uint16_t* s_out) {
  if (K <= 0 || N <= 0 || qc > N) return FP6M_ERR_BAD_ARG;
  const int n6 = qc < 0 ? 0 : qc, n4 = N - n6;
  std::vector<uint8_t> q4((size_t)K * n4), c6((size_t)K * n6);
  std::vector<uint16_t> s4(n4), s6(n6);
  int rc = fp6m_unpack_reference(B_ref, s_ref, K, N, qc, q4.data(), c6.data(), s4.data(), s6.data());
  if (rc) return rc;
  return fp6m_pack_b200(q4.data(), c6.data(), s4.data(), s6.data(), K, N, qc, -1, B_out, s_out);
}

int fp6m_schedule(int K, int N, int qc, int group_size, int ctas, int* bounds) {
  if (K <= 0 || N <= 0 || qc > N || ctas < 1 || ctas > kMaxCtas || !bounds) return -1;
  Schedule sch;
  make_schedule(make_geometry(K, N, qc, group_size), ctas, &sch);
  for (int c = 0; c <= sch.ctas; ++c) bounds[c] = sch.bound[c];
  return sch.total_units;
}

}  // extern "C"
