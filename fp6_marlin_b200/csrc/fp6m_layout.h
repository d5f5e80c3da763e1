// Blackwell weight layout ("b200", layout id 1) and the stripe schedule, shared by the host
// packers, the kernels and the host dispatcher.
//
// Logical content is the reference's: a K x N weight matrix whose first N4 = N - qc columns are
// INT4 codes q in 0..15 (value q - 8; fp6_marlin_cuda_kernel.cu:249-286) and whose last N6 = qc
// columns are FP6 E3M2 codes `s eee mm` (weight_quant.cpp:27-96).  Only the tiling differs from
// the reference's 16 x 64 fragment order (test.py:60-83, weight_prepacking.cpp:123-177): on B200
// the weights are the TMEM operand of tcgen05.mma, one TMEM lane = one weight column, so a thread
// dequantises ONE column and the layout is column-major inside small units.
//
// Tiling.  Each region (INT4, then FP6) is cut into STRIPS of 128 columns; the last strip of a
// region may be narrower and is padded to a multiple of 32 columns (nq "quads" of 32).  Along K a
// strip is a sequence of UNITS of 64 rows, stored one after the other (so any K range of a strip
// is one contiguous range of HBM); two units form a BLOCK of 128 rows = one INT4 scale group.
//
//   INT4 unit: nq * 1024 bytes.  Column c (0 .. 32 nq - 1) owns 32 bytes at c * 32 = eight words;
//     word w8 (0..7) holds rows 64 u + 8 w8 + i (i = 0..7) of that column, nibble p (from the least
//     significant) holding i = {0,2,4,6,1,3,5,7}[p] - so `word & 0x000f000f` is the row pair
//     (i0, i1), `word & 0x00f000f0` the pair (i2, i3), and the same after `>> 8`.
//     Inside its 32 bytes word w8 sits at 16 * ((w8 >> 2) ^ ((c >> 2) & 1)) + 4 * (w8 & 3): the two
//     16-byte halves are swapped for every other group of four columns, which makes a warp's
//     16-byte loads (32 consecutive columns) free of shared-memory bank conflicts.
//
//   FP6 unit: nq * 1536 bytes = a four-bit part (nq * 1024 bytes, laid out exactly as above; byte b
//     of word w8 has (code(i = b) & 15) in its low nibble and (code(i = 4 + b) & 15) in its high
//     nibble) followed by a two-bit part (nq * 512 bytes; column c owns 16 bytes at c * 16 = four
//     words; word w4 serves the four-bit words 2 w4 and 2 w4 + 1).  Two-bit word: for set
//     js = 2 (w8 & 1) + (i / 4) and byte b = i % 4, the sign bit of the code sits at bit
//     (8 b + 7 - 2 js) mod 32 and the top exponent bit at (8 b + 4 - 2 js) mod 32, so that
//     rotl(word, 2 js) & 0x90909090 supplies bits 7 and 4 of four bytes `s 0 0 e e e m m`.
//
// Rows >= K and columns past a region's width are padding: INT4 nibble 8 (value 0), FP6 code 0.
//
// Scales (fp16), plain column order.  INT4: per strip, per group (group size 128 = one block; or a
// single group in per-channel mode), 32 nq values.  FP6: per-column scales after all INT4 scales.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define FP6M_HD __host__ __device__ inline
#else
#define FP6M_HD inline
#endif

namespace fp6m {

constexpr int kStripCols = 128;       // columns per full strip
constexpr int kBlockRows = 128;       // rows per block (= the INT4 scale group)
constexpr int kUnitRows = 64;         // rows per unit
constexpr int kQuadCols = 32;         // padding granularity of a strip
constexpr int kInt4UnitQuadBytes = 1024;  // one quad of one unit, INT4
constexpr int kFp6UnitQuadBytes = 1536;   // one quad of one unit, FP6 (1024 four-bit + 512 two-bit)
constexpr int kMaxCtas = 640;         // upper bound on the persistent grid

constexpr int kLayoutReference = 0;
constexpr int kLayoutB200 = 1;

FP6M_HD int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Geometry of one problem in the b200 layout.
struct Geometry {
  int K, N, qc;            // qc = number of FP6 columns (0 = INT4 only)
  int n4, n6;              // columns per region
  int k128;                // blocks per strip
  int strips4, strips6;    // strips per region
  int groups;              // scale groups along K for INT4: k128 (group 128) or 1 (per-channel)
};

FP6M_HD Geometry make_geometry(int K, int N, int qc, int group_size) {
  Geometry g;
  g.K = K; g.N = N; g.qc = qc < 0 ? 0 : qc;
  g.n6 = g.qc; g.n4 = N - g.qc;
  g.k128 = ceil_div(K, kBlockRows);
  g.strips4 = ceil_div(g.n4, kStripCols);
  g.strips6 = ceil_div(g.n6, kStripCols);
  g.groups = group_size > 0 ? g.k128 : 1;
  return g;
}

FP6M_HD int units_per_strip(const Geometry& g) { return 2 * g.k128; }

// Number of quads (32-column groups) of strip `s` of a region that is `n_cols` wide.
FP6M_HD int strip_quads(int n_cols, int s) {
  int left = n_cols - s * kStripCols;
  if (left >= kStripCols) return 4;
  return ceil_div(left, kQuadCols);
}
// Number of real (unpadded) columns of strip `s`.
FP6M_HD int strip_cols(int n_cols, int s) {
  int left = n_cols - s * kStripCols;
  return left >= kStripCols ? kStripCols : left;
}

// Byte offsets.  All full strips come first in a region, so a strip's offset is linear in s.
FP6M_HD int64_t int4_region_bytes(const Geometry& g) {
  return (int64_t)ceil_div(g.n4, kQuadCols) * units_per_strip(g) * kInt4UnitQuadBytes;
}
FP6M_HD int64_t fp6_region_bytes(const Geometry& g) {
  return (int64_t)ceil_div(g.n6, kQuadCols) * units_per_strip(g) * kFp6UnitQuadBytes;
}
FP6M_HD int64_t weight_bytes(const Geometry& g) { return int4_region_bytes(g) + fp6_region_bytes(g); }

FP6M_HD int64_t int4_unit_offset(const Geometry& g, int strip, int unit) {
  return ((int64_t)strip * 4 * units_per_strip(g) + (int64_t)unit * strip_quads(g.n4, strip)) * kInt4UnitQuadBytes;
}
FP6M_HD int64_t fp6_unit_offset(const Geometry& g, int strip, int unit) {
  return int4_region_bytes(g) +
         ((int64_t)strip * 4 * units_per_strip(g) + (int64_t)unit * strip_quads(g.n6, strip)) * kFp6UnitQuadBytes;
}
// Byte offset of word w8 of column c inside the four-bit part of a unit.
FP6M_HD int word_offset(int c, int w8) { return c * 32 + (((w8 >> 2) ^ ((c >> 2) & 1)) << 4) + ((w8 & 3) << 2); }

// Scale element (fp16) offsets.
FP6M_HD int64_t int4_scale_count(const Geometry& g) {
  return (int64_t)ceil_div(g.n4, kQuadCols) * kQuadCols * g.groups;
}
FP6M_HD int64_t fp6_scale_count(const Geometry& g) { return (int64_t)ceil_div(g.n6, kQuadCols) * kQuadCols; }
FP6M_HD int64_t scale_count(const Geometry& g) { return int4_scale_count(g) + fp6_scale_count(g); }
FP6M_HD int64_t int4_scale_offset(const Geometry& g, int strip, int group) {
  return ((int64_t)strip * kStripCols * g.groups) + (int64_t)group * strip_quads(g.n4, strip) * kQuadCols;
}
FP6M_HD int64_t fp6_scale_offset(const Geometry& g, int strip) {
  return int4_scale_count(g) + (int64_t)strip * kStripCols;
}

// Position of a nibble inside an INT4 word for row offset i (0..7).
FP6M_HD int int4_nibble_pos(int i) { return (i & 1) ? 4 + (i >> 1) : (i >> 1); }

// ---------------------------------------------------------------------------------------------
// Stripe schedule.  Units are ordered strip-major (INT4 strips, then FP6 strips), rows fastest,
// and weighted by their cost (unit_cost: 8 per INT4 unit, 11 per FP6 unit).  CTA c owns the units
// [bound[c], bound[c+1]); a strip that is shared by several CTAs is reduced in fp32 by the last
// of them to finish.  Replaces the reference's static INT4/FP6 SM split and its stripe
// arithmetic (fp6_marlin_cuda_kernel.cu:308-408).
// ---------------------------------------------------------------------------------------------
struct Schedule {
  int ctas;
  int total_units;
  int bound[kMaxCtas + 1];
};

// Cost of one unit for the schedule.  The kernels are bound by per-unit instruction work, which does
// not depend on how many of the strip's 128 columns exist and is larger for FP6 than for INT4, but by less
// than the byte count (measured: CTAs given FP6 units by their byte count, 12 : 8, finished early; with 9 : 8
// the few CTAs that hold the FP6 strips finished last and every step waited a microsecond for them; 10.5 to
// 12 : 8 are equal within the noise).
constexpr int kInt4UnitCost = 8, kFp6UnitCost = 11;
FP6M_HD int unit_cost(const Geometry& g, int strip_linear) {
  // with several row tiles per launch the strips repeat (virtual strip = tile * strips + strip)
  return strip_linear % (g.strips4 + g.strips6) < g.strips4 ? kInt4UnitCost : kFp6UnitCost;
}

// First unit u in [u0, u1] such that the weight of [u0, u) is >= target (u1 if never).
FP6M_HD int unit_at_cost(const Geometry& g, int u0, int u1, long long target) {
  const int ups = units_per_strip(g);
  int u = u0;
  long long acc = 0;
  while (u < u1) {
    const int strip = u / ups;
    const int c = unit_cost(g, strip);
    int strip_end = (strip + 1) * ups;
    if (strip_end > u1) strip_end = u1;
    const long long span = (long long)(strip_end - u) * c;
    if (acc + span <= target) { acc += span; u = strip_end; continue; }
    return u + (int)((target - acc + c - 1) / c);
  }
  return u1;
}

FP6M_HD long long range_cost(const Geometry& g, int u0, int u1) {
  const int ups = units_per_strip(g);
  long long acc = 0;
  int u = u0;
  while (u < u1) {
    const int strip = u / ups;
    int strip_end = (strip + 1) * ups;
    if (strip_end > u1) strip_end = u1;
    acc += (long long)(strip_end - u) * unit_cost(g, strip);
    u = strip_end;
  }
  return acc;
}

// `row_tiles` > 1: the launch covers that many tiles of rows of A; the units of tile t follow those of
// tile t - 1 (virtual strips), so a CTA mostly works on whole strips of one tile.
inline void make_schedule(const Geometry& g, int ctas, Schedule* out, int row_tiles = 1) {
  if (ctas > kMaxCtas) ctas = kMaxCtas;
  if (ctas < 1) ctas = 1;
  const int ups = units_per_strip(g);
  const int nstrips = g.strips4 + g.strips6;
  const int total_units = row_tiles * nstrips * ups;
  const long long total_cost = (long long)row_tiles * ups * ((long long)kInt4UnitCost * g.strips4 + (long long)kFp6UnitCost * g.strips6);
  out->ctas = ctas;
  out->total_units = total_units;
  // A CTA whose range starts inside a strip and reaches the strip's end reduces that strip at its own end
  // (the kernel for up to 128 rows): such CTAs get `kReducerPenalty` cost units (one segment) less work than
  // the others - measured 1 to 2 % on the steps of the Llama-2 layers; two or four segments less are no better.
  // Which CTAs they are depends on the boundaries, so the shares are settled in a few rounds.
  constexpr int kReducerPenalty = 16;
  double share[kMaxCtas];
  for (int c = 0; c < ctas; ++c) share[c] = 1.0;
  const int rounds = (kReducerPenalty > 0 && row_tiles == 1) ? 4 : 1;
  for (int round = 0; round < rounds; ++round) {
    double share_total = 0.0;
    for (int c = 0; c < ctas; ++c) share_total += share[c];
    // bound[c] = first unit at which the cost of the units before it reaches CTA c's target, all of them in
    // one walk over the strips (the targets rise with c)
    int strip = 0, real = 0;          // the strip the walk is in; its index among the strips of one row tile
    long long acc = 0;                // cost of the units before that strip
    double before = 0.0;
    for (int c = 0; c < ctas; ++c) {
      const long long target = rounds == 1 ? total_cost * c / ctas : (long long)((double)total_cost * (before / share_total));
      before += share[c];
      int cost = real < g.strips4 ? kInt4UnitCost : kFp6UnitCost;
      while (acc + (long long)ups * cost <= target) {
        acc += (long long)ups * cost;
        ++strip;
        if (++real == nstrips) real = 0;
        cost = real < g.strips4 ? kInt4UnitCost : kFp6UnitCost;
      }
      out->bound[c] = strip * ups + (int)((target - acc + cost - 1) / cost);
    }
    out->bound[ctas] = total_units;
    if (round + 1 < rounds) {
      const double per_cta = (double)total_cost / ctas;
      for (int c = 0; c < ctas; ++c) {
        const int u0 = out->bound[c], u1 = out->bound[c + 1];
        const bool reduces = (u0 % ups) != 0 && u1 >= (u0 / ups + 1) * ups;
        share[c] = reduces ? 1.0 - (double)kReducerPenalty / per_cta : 1.0;
        if (share[c] < 0.25) share[c] = 0.25;
      }
    }
  }
}

// Moves every inner boundary to a whole block (an even unit): the kernel for up to 128 rows works on
// 128-row blocks.  The number of units per strip is even, so strips and the total stay aligned.
inline void align_schedule_to_blocks(Schedule* s) {
  for (int c = 1; c < s->ctas; ++c) s->bound[c] = (s->bound[c] + 1) & ~1;
}

}  // namespace fp6m
