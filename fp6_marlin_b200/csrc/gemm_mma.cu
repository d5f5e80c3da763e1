// W(4&6)A16 GEMM for the memory-bound regime (up to 32 rows of A per pass): a persistent,
// warp-specialised sm_100a kernel.
//
//   * The byte-weighted stripe schedule (fp6m_layout.h) gives each CTA a contiguous run of 64-row
//     units of the packed weights - a contiguous range of HBM inside each 128-column strip.
//   * One producer lane streams the run with bulk TMA copies (cp.async.bulk, completion on
//     mbarriers) into a ring of shared-memory stages; a stage holds KS consecutive units
//     (KS = 4: 256 rows x 128 columns, 16 KB of INT4 words) and their group scales.
//   * 4 KS consumer warps = KS K-slices x four column quads.  A warp expands the words of its
//     unit and quad (32 columns) in registers and feeds the tensor cores with mma.sync (fp32
//     accumulate), activations coming straight from L2 into registers.
//     INT4 nibbles are OR-ed into fp16 constants (1024 + q and 64 + q: exact), and the constant
//     part is removed once per unit by a "correction" tile whose weights are the negated
//     constants, so each unit accumulates sum a * (q - 8) - the value the reference's
//     dequant_8int4 feeds its tensor cores (fp6_marlin_cuda_kernel.cu:249-286) - at a third of
//     its ALU cost.  FP6 codes are placed as `s 00eee mm` fp16 bit patterns (value / 4096, what
//     dequant_8fp6 builds before its multiply, :195-237); the factor 4096 and the column scale
//     are applied in fp32 in the epilogue.  Group scales multiply the fp32 partial sum of their
//     own unit; per-channel scales are applied in the epilogue as the reference does (:698-749).
//   * At the end of a strip the K-slices are summed through shared memory.  When several CTAs
//     share a strip each publishes its fp32 partial in a scratch slot and bumps a counter in the
//     caller's workspace (one acq_rel atomic); whichever CTA arrives last sums the slots in a
//     fixed order and writes fp16.  No CTA ever waits for another, so nothing can hang and
//     results are deterministic.
//
// This replaces the reference's fp6_kernel_marlin (fp6_marlin/fp6_marlin_cuda_kernel.cu:288-837).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "device_utils.cuh"
#include "fp6m_layout.h"
#include "gemm_params.h"

namespace fp6m {

namespace {

constexpr int kRedStride = kStripCols + 8;          // floats per row of the reduction buffer
constexpr int kRedSliceFloats = 16 * kRedStride;
constexpr int kUnitW = 6144;                        // one FP6 unit of a full strip: 4096 four-bit + 2048 two-bit
constexpr int kUnitS = 256;                         // group scales of one block: 128 fp16
constexpr int kEpilogueThreads = 256;               // 16 rows x 16 groups of 8 columns

template <int MB_, int KS_, int STAGES_>
struct Cfg {
  static constexpr int MB = MB_;                    // 16-row blocks of A per pass
  static constexpr int KS = KS_;                    // units (K-slices) per pipeline item
  static constexpr int kStages = STAGES_;
  static constexpr int kConsumerWarps = 4 * KS;
  static constexpr int kConsumerThreads = 32 * kConsumerWarps;
  static constexpr int kThreads = kConsumerThreads + 128;   // + one producer warpgroup (one lane works)
  static constexpr int kStageW = KS * kUnitW;
  static constexpr int kStageTwoBit = KS * 4096;    // where the two-bit planes of an FP6 item start
  static constexpr int kStageBytes = kStageW + KS * kUnitS;
  static constexpr int kRingBytes = kStages * kStageBytes;
  static constexpr int kRedBytes = KS * kRedSliceFloats * 4;
  static constexpr int kBarBytes = 2 * kStages * 8;
  static constexpr int kSmemBytes = kRingBytes + kRedBytes + kBarBytes + 64;
  static constexpr int kSlotFloats = MB * 16 * kStripCols;
};

// Walks the units [u0, u1) of a CTA as pipeline items: up to KS consecutive units of one strip.
// Only init() divides; next() is incremental because one lane runs this on the critical path.
struct ItemIter {
  int u, end, ups, per_item;
  int strip_lin, first, count;   // first = unit index inside the strip
  bool valid;
  __device__ __forceinline__ void init(int u0, int u1, int ups_, int per_item_) {
    u = u0; end = u1; ups = ups_; per_item = per_item_;
    strip_lin = u / ups;
    first = u - strip_lin * ups;
    set_count();
  }
  __device__ __forceinline__ void set_count() {
    valid = u < end;
    count = min(per_item, min(ups - first, end - u));
  }
  __device__ __forceinline__ void next() {
    u += count;
    first += count;
    if (first == ups) { first = 0; ++strip_lin; }
    set_count();
  }
};

// Per-strip constants of the producer, recomputed only when the strip changes.
struct StripSource {
  int strip_lin = -1;
  bool is6, group;
  int nq;
  const uint8_t* w;       // INT4: first unit of the strip; FP6: first block of the strip
  const half* s;          // group scales of the strip's first block
  __device__ __forceinline__ void set(const MulParams& p, int lin) {
    const Geometry& geo = p.geo;
    strip_lin = lin;
    is6 = lin >= geo.strips4;
    if (!is6) {
      nq = strip_quads(geo.n4, lin);
      w = p.B + int4_block_offset(geo, lin, 0);
      group = geo.groups > 1;
      s = p.S + int4_scale_offset(geo, lin, 0);
    } else {
      const int strip = lin - geo.strips4;
      nq = strip_quads(geo.n6, strip);
      w = p.B + fp6_block_offset(geo, strip, 0);
      group = false;
      s = nullptr;
    }
  }
};

// The producer warp issues the copies of one item: lane 0 arms the barrier and copies the INT4
// words (one contiguous run - consecutive units are contiguous in HBM, across blocks too); lane s
// copies what belongs to unit s alone (its group scales, or its two FP6 planes).
template <class C>
__device__ __forceinline__ void issue_item(const StripSource& src, const ItemIter& it, int lane, uint32_t dst, uint32_t bar,
                                           uint64_t policy) {
  const int nq = src.nq;
  if (!src.is6) {
    const uint32_t wbytes = it.count * nq * 1024;
    if (lane == 0) {
      mbar_arrive_expect_tx(bar, wbytes + (src.group ? it.count * nq * 64 : 0));
      tma_load_1d_stream(dst, src.w + (size_t)it.first * nq * 1024, wbytes, bar, policy);
    }
    __syncwarp();
    if (src.group && lane < it.count)
      tma_load_1d(dst + C::kStageW + lane * kUnitS, src.s + (size_t)((it.first + lane) >> 1) * nq * kQuadCols, nq * 64, bar);
  } else {
    if (lane == 0) mbar_arrive_expect_tx(bar, it.count * nq * 1536);
    __syncwarp();
    if (lane < it.count) {
      const int unit = it.first + lane;
      const uint8_t* base = src.w + (size_t)(unit >> 1) * nq * kFp6QuadBytes;
      tma_load_1d_stream(dst + lane * nq * 1024, base + (unit & 1) * nq * 1024, nq * 1024, bar, policy);
      tma_load_1d_stream(dst + C::kStageTwoBit + lane * nq * 512, base + nq * kInt4QuadBytes + (unit & 1) * nq * 512, nq * 512, bar, policy);
    }
  }
}

// D = A * B + C with separate C and D registers (the correction tile seeds many tiles).
__device__ __forceinline__ void mma_cd(float (&d)[4], const float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}
__device__ __forceinline__ void mma_acc(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// INT4 word -> four operand registers holding 1024 + q (rows i0,i1 and i4,i5) and 64 + q (rows
// i2,i3 and i6,i7): exact fp16 values, one logic instruction each.
__device__ __forceinline__ void expand_int4(uint32_t q, uint32_t (&b)[4]) {
  constexpr int kAndOr = (0xf0 & 0xcc) | 0xaa;  // (a & b) | c
  b[0] = lop3<kAndOr>(q, 0x000f000fu, 0x64006400u);
  b[1] = lop3<kAndOr>(q, 0x00f000f0u, 0x54005400u);
  q >>= 8;
  b[2] = lop3<kAndOr>(q, 0x000f000fu, 0x64006400u);
  b[3] = lop3<kAndOr>(q, 0x00f000f0u, 0x54005400u);
}
constexpr uint32_t kNegBiasLo = 0xe408e408u;  // -1032, -1032
constexpr uint32_t kNegBiasHi = 0xd480d480u;  // -72, -72

// FP6 four-bit word + two-bit word -> four operand registers of `s 00eee mm 00000000` patterns.
__device__ __forceinline__ void expand_fp6(uint32_t four, uint32_t two, int rot, uint32_t (&b)[4]) {
  constexpr int kAndOr = (0xf0 & 0xcc) | 0xaa;
  const uint32_t r0 = __funnelshift_l(two, two, rot) & 0x90909090u;
  const uint32_t r1 = __funnelshift_l(two, two, rot + 2) & 0x90909090u;
  const uint32_t x0 = lop3<kAndOr>(four, 0x0f0f0f0fu, r0);
  const uint32_t x1 = lop3<kAndOr>(four >> 4, 0x0f0f0f0fu, r1);
  b[0] = prmt(x0, 0u, 0x1404u);
  b[1] = prmt(x0, 0u, 0x3424u);
  b[2] = prmt(x1, 0u, 0x1404u);
  b[3] = prmt(x1, 0u, 0x3424u);
}

// One window (32 rows) of one quad: expand its four words and issue the tensor-core tiles
// K-step-major, so that consecutive instructions belong to different accumulator tiles.
template <int MB, bool IS6, bool FIRST>
__device__ __forceinline__ void window_mma(const uint4& wq, const uint2& tq, const uint4 (&a)[MB][2][2], int w,
                                           const float (&seed)[MB][4], float (&tmp)[MB][4][4]) {
  const uint32_t ws[4] = {wq.x, wq.y, wq.z, wq.w};
  uint32_t b[4][4];
#pragma unroll
  for (int jr = 0; jr < 4; ++jr) {
    if (IS6) expand_fp6(ws[jr], (jr < 2) ? tq.x : tq.y, 4 * (jr & 1), b[jr]);
    else expand_int4(ws[jr], b[jr]);
  }
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int jr = 0; jr < 4; ++jr) {
      if (FIRST) mma_cd(tmp[mb][jr], seed[mb], a[mb][w][0].x, a[mb][w][1].x, a[mb][w][0].y, a[mb][w][1].y, b[jr][0], b[jr][1]);
      else mma_acc(tmp[mb][jr], a[mb][w][0].x, a[mb][w][1].x, a[mb][w][0].y, a[mb][w][1].y, b[jr][0], b[jr][1]);
    }
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int jr = 0; jr < 4; ++jr)
      mma_acc(tmp[mb][jr], a[mb][w][0].z, a[mb][w][1].z, a[mb][w][0].w, a[mb][w][1].w, b[jr][2], b[jr][3]);
}

// This warp's share of one pipeline item: quad `jq` (four 8-column tiles) of unit `ks` of the stage.
// Byte offsets of this lane's data inside a stage; they change only with the strip.
struct LaneOffsets {
  int four;        // four-bit words of window 0: [unit][window][quad][lane][4 words]
  int four_step;   // distance to window 1
  int two;         // two-bit words of window 0 (FP6)
  int two_step;
  int scale;       // group scales of the unit: [t][tile][2]
  __device__ __forceinline__ void set(int nq, int ks, int jq, int lane, int stage_w, int stage_two) {
    four = ks * nq * 1024 + (jq * 32 + lane) * 16;
    four_step = nq * 512;
    two = stage_two + ks * nq * 512 + (jq * 32 + lane) * 8;
    two_step = nq * 256;
    scale = stage_w + ks * kUnitS + ((lane & 3) * 4 * nq + 4 * jq) * 4;
  }
};

template <class C, bool IS6, bool GROUP>
__device__ __forceinline__ void compute_item(const uint8_t* st, const LaneOffsets& lo,
                                             const uint4 (&a)[C::MB][2][2], float (&acc)[C::MB][4][4]) {
  constexpr int MB = C::MB;
  uint4 wq[2];
  uint2 tq[2] = {make_uint2(0, 0), make_uint2(0, 0)};
  uint4 sc = make_uint4(0, 0, 0, 0);
#pragma unroll
  for (int w = 0; w < 2; ++w) {
    wq[w] = *reinterpret_cast<const uint4*>(st + lo.four + w * lo.four_step);
    if (IS6) tq[w] = *reinterpret_cast<const uint2*>(st + lo.two + w * lo.two_step);
  }
  if (GROUP && !IS6) sc = *reinterpret_cast<const uint4*>(st + lo.scale);

  float seed[MB][4];
#pragma unroll
  for (int mb = 0; mb < MB; ++mb) {
    seed[mb][0] = seed[mb][1] = seed[mb][2] = seed[mb][3] = 0.f;
    if (!IS6) {
#pragma unroll
      for (int w = 0; w < 2; ++w) {
        mma_acc(seed[mb], a[mb][w][0].x, a[mb][w][1].x, a[mb][w][0].y, a[mb][w][1].y, kNegBiasLo, kNegBiasHi);
        mma_acc(seed[mb], a[mb][w][0].z, a[mb][w][1].z, a[mb][w][0].w, a[mb][w][1].w, kNegBiasLo, kNegBiasHi);
      }
    }
  }
  float tmp[MB][4][4];
  window_mma<MB, IS6, true>(wq[0], tq[0], a, 0, seed, tmp);
  window_mma<MB, IS6, false>(wq[1], tq[1], a, 1, seed, tmp);

  const uint32_t scs[4] = {sc.x, sc.y, sc.z, sc.w};
#pragma unroll
  for (int jr = 0; jr < 4; ++jr) {
    float2 f = make_float2(1.f, 1.f);
    if (GROUP && !IS6) f = __half22float2(u32_as_h2(scs[jr]));
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
      float* dst = acc[mb][jr];
      if (GROUP && !IS6) {
        dst[0] = fmaf(f.x, tmp[mb][jr][0], dst[0]);
        dst[1] = fmaf(f.y, tmp[mb][jr][1], dst[1]);
        dst[2] = fmaf(f.x, tmp[mb][jr][2], dst[2]);
        dst[3] = fmaf(f.y, tmp[mb][jr][3], dst[3]);
      } else {
        dst[0] += tmp[mb][jr][0]; dst[1] += tmp[mb][jr][1]; dst[2] += tmp[mb][jr][2]; dst[3] += tmp[mb][jr][3];
      }
    }
  }
}

// Column factors of the epilogue for the 8 columns c8..c8+7 of a strip.
__device__ __forceinline__ void load_col_scales(const MulParams& p, bool is6, int strip, int nq, int c8, float (&cs)[8]) {
  const Geometry& geo = p.geo;
  if (!is6 && geo.groups > 1) {
#pragma unroll
    for (int e = 0; e < 8; ++e) cs[e] = 1.f;
    return;
  }
  const half* sp = p.S + (is6 ? fp6_scale_offset(geo, strip) : int4_scale_offset(geo, strip, 0));
  const float mult = is6 ? 4096.f : 1.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) cs[e] = __half2float(__ldg(sp + scale_index(c8 + e, nq))) * mult;
}

__device__ __forceinline__ void store_c_row(half* dst, const float (&v)[8], const float (&cs)[8]) {
  uint4 o;
  o.x = h2_as_u32(__floats2half2_rn(v[0] * cs[0], v[1] * cs[1]));
  o.y = h2_as_u32(__floats2half2_rn(v[2] * cs[2], v[3] * cs[3]));
  o.z = h2_as_u32(__floats2half2_rn(v[4] * cs[4], v[5] * cs[5]));
  o.w = h2_as_u32(__floats2half2_rn(v[6] * cs[6], v[7] * cs[7]));
  *reinterpret_cast<uint4*>(dst) = o;
}

// One atomic with release (the CTA's partial, ordered before it by a CTA barrier, becomes visible)
// and acquire (the other CTAs' partials are visible to loads that follow) semantics.
__device__ __forceinline__ int atomic_add_acq_rel(int* addr, int v) {
  int old;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(addr), "r"(v) : "memory");
  return old;
}

template <class C, bool GROUP>
__global__ void __launch_bounds__(C::kThreads, 1) w46_gemm_mma_kernel(const __grid_constant__ MulParams p) {
  constexpr int MB = C::MB, KS = C::KS, kStages = C::kStages;
  extern __shared__ __align__(128) uint8_t smem[];
  float* red = reinterpret_cast<float*>(smem + C::kRingBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kRingBytes + C::kRedBytes);
  int* flag = reinterpret_cast<int*>(smem + C::kRingBytes + C::kRedBytes + C::kBarBytes);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kStages);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x;
  const Geometry& geo = p.geo;
  const int ups = units_per_strip(geo);
  const int U0 = p.sched.bound[cta], U1 = p.sched.bound[cta + 1];

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, C::kConsumerWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();
  if (U0 >= U1) return;

  bool dead = false;

  if (warp >= C::kConsumerWarps) {
    // ------------------------------------------------------------------ producer warpgroup
    // Register hand-over between warpgroups.  The registers a setmaxnreg.inc asks for must have been
    // released by a setmaxnreg.dec inside the same CTA (the launch allocation is the pool), or the
    // request blocks for ever: 384 threads x 168 = 64512; 128 x (168 - 40) released = 256 x (232 - 168).
    // 640 threads x 96 = 61440; 128 x (96 - 24) = 9216 released >= 512 x (112 - 96) = 8192 requested.
    if (KS == 2) asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    else asm volatile("setmaxnreg.dec.sync.aligned.u32 24;");
    if (warp == C::kConsumerWarps) {
      const uint64_t policy = make_evict_first_policy();
      ItemIter it;
      it.init(U0, U1, ups, KS);
      StripSource src;
      int n = 0;
      for (; it.valid; it.next(), ++n) {
        const int s = n % kStages;
        if (it.strip_lin != src.strip_lin) src.set(p, it.strip_lin);
        mbar_wait_bounded(empty0 + 8 * s, ((n / kStages) & 1) ^ 1, p.status, dead);
        issue_item<C>(src, it, lane, smem_u32(smem + s * C::kStageBytes), full0 + 8 * s, policy);
      }
      // do not leave while copies may still be landing in this CTA's shared memory
      for (int k = max(0, n - kStages); k < n; ++k)
        mbar_wait_bounded(full0 + 8 * (k % kStages), (k / kStages) & 1, p.status, dead);
    }
    return;
  }

  // -------------------------------------------------------------------- consumer warps
  if (KS == 2) asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
  else asm volatile("setmaxnreg.inc.sync.aligned.u32 112;");
  const int g = lane >> 2, t = lane & 3;
  const int ks = warp >> 2;      // unit of the item (K-slice)
  const int jq = warp & 3;       // column quad of the strip

  float acc[MB][4][4];
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[mb][j][e] = 0.f;

  // activations of this warp's unit: [row block][window][row half], 8 consecutive halves each
  uint4 a[MB][2][2];
  const uint4* a_row[MB][2];
  bool a_row_ok[MB][2];
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = mb * 16 + g + 8 * h;
      a_row_ok[mb][h] = row < p.M;
      a_row[mb][h] = reinterpret_cast<const uint4*>(p.A + (size_t)(a_row_ok[mb][h] ? row : 0) * p.K) + t;
    }
  auto load_a = [&](const ItemIter& it) {
    const int k0 = (it.first + ks) * kUnitRows;      // first row of this warp's unit
    const bool ok = it.valid && ks < it.count;
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int w = 0; w < 2; ++w)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int k = k0 + 32 * w;
          if (ok && a_row_ok[mb][h] && k + 8 * t < p.K)
            a[mb][w][h] = __ldg(a_row[mb][h] + (k >> 3));
          else
            a[mb][w][h] = make_uint4(0, 0, 0, 0);
        }
  };

  ItemIter it;
  it.init(U0, U1, ups, KS);
  load_a(it);
  int stage = 0, phase = 0;
  const int strip_first = it.strip_lin;
  const int r = tid >> 4, c8 = (tid & 15) * 8;   // epilogue (first 256 threads): row and 8 columns

  while (it.valid) {
    const int strip_lin = it.strip_lin;
    const bool is6 = strip_lin >= geo.strips4;
    const int strip = is6 ? strip_lin - geo.strips4 : strip_lin;
    const int nq = strip_quads(is6 ? geo.n6 : geo.n4, strip);
    const int s_begin = strip_lin * ups, s_end = s_begin + ups;
    const int slice_u0 = it.u;
    LaneOffsets lo;
    lo.set(nq, ks, jq, lane, C::kStageW, C::kStageTwoBit);

    while (it.valid && it.strip_lin == strip_lin) {
      mbar_wait_bounded(full0 + 8 * stage, phase, p.status, dead);
      if (ks < it.count && jq < nq) {
        const uint8_t* st = smem + stage * C::kStageBytes;
        if (is6) compute_item<C, true, GROUP>(st, lo, a, acc);
        else compute_item<C, false, GROUP>(st, lo, a, acc);
      }
      it.next();
      load_a(it);   // next item's activations
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * stage);
      if (++stage == kStages) { stage = 0; phase ^= 1; }
    }
    const int slice_u1 = it.valid ? it.u : U1;

    // ---- strip finished for this CTA: sum the K-slices, then write C or publish a partial
    const bool full_strip = slice_u0 == s_begin && slice_u1 == s_end;
    const int ncols = strip_cols(is6 ? geo.n6 : geo.n4, strip);
    const int col0 = (is6 ? geo.n4 : 0) + strip * kStripCols;
    float* slot = p.partials + (size_t)(2 * cta + (strip_lin != strip_first ? 1 : 0)) * C::kSlotFloats;

#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
      float* mine = red + ks * kRedSliceFloats + 32 * jq;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        *reinterpret_cast<float2*>(mine + g * kRedStride + 8 * j + 2 * t) = make_float2(acc[mb][j][0], acc[mb][j][1]);
        *reinterpret_cast<float2*>(mine + (g + 8) * kRedStride + 8 * j + 2 * t) = make_float2(acc[mb][j][2], acc[mb][j][3]);
        acc[mb][j][0] = acc[mb][j][1] = acc[mb][j][2] = acc[mb][j][3] = 0.f;
      }
      named_bar_sync(1, C::kConsumerThreads);
      if (tid < kEpilogueThreads) {
        float v[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = 0.f;
        const float* src = red + r * kRedStride + c8;
#pragma unroll
        for (int w = 0; w < KS; ++w) {
          const float4 x = *reinterpret_cast<const float4*>(src + w * kRedSliceFloats);
          const float4 y = *reinterpret_cast<const float4*>(src + w * kRedSliceFloats + 4);
          v[0] += x.x; v[1] += x.y; v[2] += x.z; v[3] += x.w;
          v[4] += y.x; v[5] += y.y; v[6] += y.z; v[7] += y.w;
        }
        const int row = mb * 16 + r;
        if (full_strip) {
          if (row < p.M && c8 < ncols) {
            float cs[8];
            load_col_scales(p, is6, strip, nq, c8, cs);
            store_c_row(p.C + (size_t)row * p.N + col0 + c8, v, cs);
          }
        } else {
          float4* dst = reinterpret_cast<float4*>(slot + (size_t)row * kStripCols + c8);
          __stcg(dst, make_float4(v[0], v[1], v[2], v[3]));
          __stcg(dst + 1, make_float4(v[4], v[5], v[6], v[7]));
        }
      }
      named_bar_sync(1, C::kConsumerThreads);   // red is free again; all partial stores are issued
    }

    if (!full_strip) {
      // ---- several CTAs share the strip: the last one to arrive sums the slots and writes C
      int c_lo = cta, c_hi = cta;
      while (c_lo > 0 && p.sched.bound[c_lo] > s_begin) --c_lo;
      while (c_hi + 1 < p.sched.ctas && p.sched.bound[c_hi + 1] < s_end) ++c_hi;
      if (tid == 0) {
        int contributors = 0;
        for (int c = c_lo; c <= c_hi; ++c) contributors += p.sched.bound[c] < p.sched.bound[c + 1];
        const int last = atomic_add_acq_rel(p.counters + strip_lin, 1) == contributors - 1;
        if (last) p.counters[strip_lin] = 0;   // the workspace is left zeroed, as the reference leaves its locks
        *flag = last;
      }
      named_bar_sync(1, C::kConsumerThreads);
      if (*flag != 0 && tid < kEpilogueThreads) {
        // sum the contributors' slots in CTA order; the loads of up to 8 slots are issued together
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          const int row = mb * 16 + r;
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = 0.f;
          for (int cbase = c_lo; cbase <= c_hi; cbase += 8) {
            float4 x[8], y[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int c = cbase + i;
              x[i] = y[i] = make_float4(0.f, 0.f, 0.f, 0.f);
              if (c <= c_hi && p.sched.bound[c] < p.sched.bound[c + 1]) {
                const int c_first = p.sched.bound[c] / ups;
                const float* src = p.partials + (size_t)(2 * c + (strip_lin != c_first ? 1 : 0)) * C::kSlotFloats +
                                   (size_t)row * kStripCols + c8;
                x[i] = __ldcg(reinterpret_cast<const float4*>(src));
                y[i] = __ldcg(reinterpret_cast<const float4*>(src) + 1);
              }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              v[0] += x[i].x; v[1] += x[i].y; v[2] += x[i].z; v[3] += x[i].w;
              v[4] += y[i].x; v[5] += y[i].y; v[6] += y[i].z; v[7] += y[i].w;
            }
          }
          if (row < p.M && c8 < ncols) {
            float cs[8];
            load_col_scales(p, is6, strip, nq, c8, cs);
            store_c_row(p.C + (size_t)row * p.N + col0 + c8, v, cs);
          }
        }
      }
      named_bar_sync(1, C::kConsumerThreads);   // the flag may be rewritten by the next strip
    }
  }
}

using CfgRows16 = Cfg<1, 4, 6>;   // 16 consumer warps, 16 KB items
using CfgRows32 = Cfg<2, 2, 8>;   // 8 consumer warps with twice the accumulators, 8 KB items

template <class C, bool GROUP>
cudaError_t launch_one(const MulParams& p, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(w46_gemm_mma_kernel<C, GROUP>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  w46_gemm_mma_kernel<C, GROUP><<<p.sched.ctas, C::kThreads, C::kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

int mma_rows_per_pass() { return 32; }

size_t mma_scratch_bytes(int ctas) { return (size_t)2 * ctas * CfgRows32::kSlotFloats * sizeof(float); }

// Runs the GEMM for rows [0, p.M) with p.M <= 32; the host dispatcher loops over larger M.
cudaError_t launch_gemm_mma(const MulParams& p, cudaStream_t stream) {
  const bool group = p.geo.groups > 1;
  if (p.M <= 16) return group ? launch_one<CfgRows16, true>(p, stream) : launch_one<CfgRows16, false>(p, stream);
  return group ? launch_one<CfgRows32, true>(p, stream) : launch_one<CfgRows32, false>(p, stream);
}

}  // namespace fp6m
