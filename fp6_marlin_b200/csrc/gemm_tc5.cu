// W(4&6)A16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for up to 64 rows of A per pass.
//
// The product is computed transposed, D[n, m] = sum_k W[k, n] * A[m, k]: the 128 weight columns of
// a strip are the M dimension of tcgen05.mma (one TMEM lane per weight column), the rows of A are
// its N dimension (16, 32 or 64), and the dequantised weights are the A operand read from TENSOR
// MEMORY, so they never travel through shared memory.  Legacy mma.sync costs about 32 cycles per
// m16n8k16 tile on B200 and cannot keep up with HBM (profiles/w46_gemm_mma_*); tcgen05 can.
//
// One CTA = six warps:
//   warp 0      producer: bulk TMA copies (cp.async.bulk, mbarrier completion) of one 64-row unit
//               of packed words and its group scales per stage, plus cp.async copies that lay the
//               unit's activations out as canonical K-major 8x16-byte core matrices.
//   warp 1      one lane issues tcgen05.mma (kind::f16, fp32 accumulators in TMEM) and commits
//               completion to mbarriers; the warp also owns the TMEM allocation.
//   warps 2-5   dequantisers: thread = weight column = TMEM lane.  A thread reads its 32 bytes of
//               a unit, expands the eight words in registers and stores them with tcgen05.st into
//               a small TMEM operand ring.  INT4 nibbles become the exact integers q - 8 in fp16
//               (OR into 1024 + q / 64 + q, then subtract 1032 / 72) - bit for bit what the
//               reference's dequant_8int4 feeds its tensor cores (fp6_marlin_cuda_kernel.cu:249-286).
//               FP6 codes become `s 00eee mm` fp16 patterns (exact value / 4096, as dequant_8fp6
//               builds them before its multiply by 4096, :195-237).  After every scale
//               group (128 rows) the same threads read the accumulator tile back (tcgen05.ld),
//               multiply by their column's group scale in fp32 and add to registers; two accumulator
//               tiles alternate so the read-back overlaps the next group's MMAs.
// Work comes from the byte-weighted stripe schedule (fp6m_layout.h); strips shared by several CTAs
// are reduced through fp32 scratch slots by the last CTA to arrive (one acq_rel atomic on a counter
// in the caller's workspace) - no CTA waits for another, every wait in the kernel is bounded.
//
// Replaces the reference's fp6_kernel_marlin (fp6_marlin/fp6_marlin_cuda_kernel.cu:288-837).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "device_utils.cuh"
#include "fp6m_layout.h"
#include "gemm_params.h"

namespace fp6m {

namespace {

constexpr int kThreads = 192;
constexpr int kDequantThreads = 128;
constexpr int kUnitW = 6144;            // packed words of one unit: up to 4096 four-bit + 2048 two-bit
constexpr int kUnitS = 256;             // group scales of the unit's block: 128 fp16
constexpr int kActOffset = kUnitW + kUnitS;
constexpr int kTmemSlots = 3;           // operand ring: 3 units x 4 K-steps x 8 columns

template <int NT_, int STAGES_, int CTAS_PER_SM_>
struct Tc5Cfg {
  static constexpr int NT = NT_;                       // rows of A per pass = N of the MMA
  static constexpr int kStages = STAGES_;
  static constexpr int kCtasPerSm = CTAS_PER_SM_;
  static constexpr int kActBytes = NT * 128;           // NT rows x 64 halves
  static constexpr int kStageBytes = kActOffset + kActBytes;
  static constexpr int kRingBytes = kStages * kStageBytes;
  static constexpr int kNumBars = 2 * kStages + 2 * kTmemSlots + 4;
  static constexpr int kSmemBytes = kRingBytes + kNumBars * 8 + 64;
  static constexpr int kTmemD0 = 0, kTmemD1 = NT, kTmemA = 2 * NT;
  static constexpr int kTmemUsed = kTmemA + kTmemSlots * 32;
  static constexpr int kTmemCols = kTmemUsed <= 128 ? 128 : 256;
  static constexpr int kSlotFloats = NT * kStripCols;
  static constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
};

// ---- tcgen05 wrappers -------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[128 x N] (+)= A[128 x 16] (TMEM) * B[N x 16]^T (shared memory descriptor)
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0)
      : "memory");
}
// K-major, no swizzle: 8-row x 16-byte core matrices of 128 bytes; the two K halves of a step are
// 128 bytes apart (leading offset), 8-row groups 256 bytes apart (stride offset).
__device__ __forceinline__ uint64_t act_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(256 >> 4) << 32) | ((uint64_t)1 << 46);
}
__device__ __forceinline__ void tc_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr) : "memory");
  tc_wait_ld();
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// 16-byte asynchronous copy with zero fill when `valid` is false; completion is reported to an
// mbarrier by cp_async_arrive below.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ int atomic_add_acq_rel(int* addr, int v) {
  int old;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(addr), "r"(v) : "memory");
  return old;
}

// INT4 word -> the exact integers q - 8 as fp16 pairs (rows i0,i1 | i2,i3 | i4,i5 | i6,i7): the nibble is
// OR-ed into the mantissa of 1024 (bits 0-3) or of 64 (bits 4-7) and the constant is subtracted.
__device__ __forceinline__ void expand_int4(uint32_t q, uint32_t* b) {
  constexpr int kAndOr = (0xf0 & 0xcc) | 0xaa;  // (a & b) | c
  const half2 lo_bias = u32_as_h2(0x64086408u);   // 1032
  const half2 hi_bias = u32_as_h2(0x54805480u);   // 72
  b[0] = h2_as_u32(__hsub2(u32_as_h2(lop3<kAndOr>(q, 0x000f000fu, 0x64006400u)), lo_bias));
  b[1] = h2_as_u32(__hsub2(u32_as_h2(lop3<kAndOr>(q, 0x00f000f0u, 0x54005400u)), hi_bias));
  q >>= 8;
  b[2] = h2_as_u32(__hsub2(u32_as_h2(lop3<kAndOr>(q, 0x000f000fu, 0x64006400u)), lo_bias));
  b[3] = h2_as_u32(__hsub2(u32_as_h2(lop3<kAndOr>(q, 0x00f000f0u, 0x54005400u)), hi_bias));
}
// FP6 four-bit word + two-bit word -> `s 00eee mm 00000000` fp16 patterns (value / 4096).
__device__ __forceinline__ void expand_fp6(uint32_t four, uint32_t two, int rot, uint32_t* b) {
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

// Walks the units [u0, u1) of a CTA; every role runs the same walk, so stage, slot and segment
// numbers agree without communication.  A SEGMENT is a run of units inside one block and one strip.
struct UnitIter {
  int u, end, ups;
  int strip_lin, unit;        // unit = index inside the strip
  __device__ __forceinline__ void init(int u0, int u1, int ups_) {
    u = u0; end = u1; ups = ups_;
    strip_lin = u / ups;
    unit = u - strip_lin * ups;
  }
  __device__ __forceinline__ bool valid() const { return u < end; }
  __device__ __forceinline__ bool slice_first(int u0) const { return u == u0 || unit == 0; }
  __device__ __forceinline__ bool slice_last() const { return u + 1 == end || unit + 1 == ups; }
  __device__ __forceinline__ bool seg_first(int u0) const { return slice_first(u0) || (unit & 1) == 0; }
  __device__ __forceinline__ bool seg_last() const { return slice_last() || (unit & 1) == 1; }
  __device__ __forceinline__ void next() {
    ++u;
    if (++unit == ups) { unit = 0; ++strip_lin; }
  }
};

template <class C>
__global__ void __launch_bounds__(kThreads, C::kCtasPerSm) w46_gemm_tc5_kernel(const __grid_constant__ MulParams p) {
  constexpr int NT = C::NT, kStages = C::kStages;
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kRingBytes);
  uint32_t* misc = reinterpret_cast<uint32_t*>(smem + C::kRingBytes + C::kNumBars * 8);   // [0] TMEM base, [1] flag
  const uint32_t full_w = smem_u32(bars), empty_w = full_w + 8 * kStages;
  const uint32_t a_full = empty_w + 8 * kStages, a_empty = a_full + 8 * kTmemSlots;
  const uint32_t d_full = a_empty + 8 * kTmemSlots, d_empty = d_full + 16;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x;
  const Geometry& geo = p.geo;
  const int ups = units_per_strip(geo);
  const int U0 = p.sched.bound[cta], U1 = p.sched.bound[cta + 1];
  if (U0 >= U1) return;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_w + 8 * s, 33);     // the expect_tx arrival + 32 lanes of cp.async completions
      mbar_init(empty_w + 8 * s, 5);     // four dequantiser warps + the MMA commit
    }
    for (int t = 0; t < kTmemSlots; ++t) {
      mbar_init(a_full + 8 * t, 4);
      mbar_init(a_empty + 8 * t, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(d_full + 8 * b, 1);
      mbar_init(d_empty + 8 * b, 4);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(misc)), "r"(C::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = misc[0];
  bool dead = false;

  if (warp == 0) {
    // ================================================================== producer
    const uint64_t policy = make_evict_first_policy();
    UnitIter it;
    it.init(U0, U1, ups);
    int stage = 0, phase = 0;
    int cur_strip = -1, nq = 0;
    bool group = false;
    const uint8_t* wsrc = nullptr;      // next unit's packed words
    const half* ssrc = nullptr;         // group scales of the strip's first block
    uint32_t unit_bytes = 0, sbytes = 0;
    // activations: this lane copies chunks idx = lane + 32 j: row m = idx / 8, 16-byte chunk kc = idx % 8
    // of the unit, into canonical core-matrix order; everything but the K offset is loop-invariant
    const half* a_src[NT / 4];
    uint32_t a_dst[NT / 4];
    bool a_row_ok[NT / 4];
    const int kc = lane & 7;
#pragma unroll
    for (int j = 0; j < NT / 4; ++j) {
      const int m = (lane >> 3) + 4 * j;
      a_row_ok[j] = m < p.M;
      a_src[j] = p.A + (size_t)(a_row_ok[j] ? m : 0) * p.K + 8 * kc;
      a_dst[j] = kActOffset + (kc >> 1) * (NT / 8) * 256 + ((m >> 3) * 2 + (kc & 1)) * 128 + (m & 7) * 16;
    }
    uint32_t dst = smem_u32(smem), bar = full_w;
    for (; it.valid(); it.next()) {
      if (it.strip_lin != cur_strip) {
        cur_strip = it.strip_lin;
        const bool is6 = cur_strip >= geo.strips4;
        if (!is6) {
          nq = strip_quads(geo.n4, cur_strip);
          unit_bytes = nq * kInt4UnitQuadBytes;
          wsrc = p.B + int4_unit_offset(geo, cur_strip, 0) + (size_t)it.unit * unit_bytes;
          group = geo.groups > 1;
          ssrc = p.S + int4_scale_offset(geo, cur_strip, 0);
        } else {
          nq = strip_quads(geo.n6, cur_strip - geo.strips4);
          unit_bytes = nq * kFp6UnitQuadBytes;
          wsrc = p.B + fp6_unit_offset(geo, cur_strip - geo.strips4, 0) + (size_t)it.unit * unit_bytes;
          group = false;
        }
        sbytes = group ? nq * 64 : 0;
      }
      mbar_wait_bounded(empty_w + 8 * stage, phase ^ 1, p.status, dead);
      if (lane == 0) {
        mbar_arrive_expect_tx(bar, unit_bytes + sbytes);
        tma_load_1d_stream(dst, wsrc, unit_bytes, bar, policy);
        if (group) tma_load_1d(dst + kUnitW, ssrc + (it.unit >> 1) * nq * kQuadCols, sbytes, bar);
      }
      wsrc += unit_bytes;
      const int k0 = it.unit * kUnitRows;
      const bool k_ok = k0 + 8 * kc < p.K;
#pragma unroll
      for (int j = 0; j < NT / 4; ++j) {
        const bool ok = a_row_ok[j] && k_ok;
        cp_async16(dst + a_dst[j], ok ? (const void*)(a_src[j] + k0) : (const void*)p.A, ok);
      }
      cp_async_arrive(bar);
      dst += C::kStageBytes;
      bar += 8;
      if (++stage == kStages) { stage = 0; phase ^= 1; dst = smem_u32(smem); bar = full_w; }
    }
  } else if (warp == 1) {
    // ================================================================== MMA issuer
    if (lane == 0) {
      UnitIter it;
      it.init(U0, U1, ups);
      int stage = 0, phase = 0, slot = 0, slot_phase = 0, seg = 0;
      for (; it.valid(); it.next()) {
        const int dbuf = seg & 1;
        const uint32_t d_tmem = tmem + (dbuf ? C::kTmemD1 : C::kTmemD0);
        const bool first = it.seg_first(U0);
        mbar_wait_bounded(full_w + 8 * stage, phase, p.status, dead);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // cp.async wrote the activations
        mbar_wait_bounded(a_full + 8 * slot, slot_phase, p.status, dead);
        if (first) mbar_wait_bounded(d_empty + 8 * dbuf, ((seg >> 1) & 1) ^ 1, p.status, dead);
        tc_fence_after();
        const uint32_t act = smem_u32(smem + stage * C::kStageBytes + kActOffset);
#pragma unroll
        for (int st = 0; st < 4; ++st) {
          const uint64_t desc = act_desc(act + st * (NT / 8) * 256);
          tc_mma_ts(d_tmem, tmem + C::kTmemA + slot * 32 + st * 8, desc, C::kIdesc, (first && st == 0) ? 0u : 1u);
        }
        tc_commit(a_empty + 8 * slot);
        tc_commit(empty_w + 8 * stage);
        if (it.seg_last()) {
          tc_commit(d_full + 8 * dbuf);
          ++seg;
        }
        if (++stage == kStages) { stage = 0; phase ^= 1; }
        if (++slot == kTmemSlots) { slot = 0; slot_phase ^= 1; }
      }
    }
  } else {
    // ================================================================== dequantisers (warps 2..5)
    const int quarter = warp & 3;                    // the TMEM lanes this warp may touch
    const int c = quarter * 32 + lane;               // weight column inside the strip = TMEM lane
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const int dtid = tid - 64;                       // 0..127 among the dequantiser threads
    float acc[NT];
#pragma unroll
    for (int m = 0; m < NT; ++m) acc[m] = 0.f;

    UnitIter it;
    it.init(U0, U1, ups);
    int stage = 0, phase = 0, slot = 0, slot_phase = 0, seg = 0;
    const int strip_first = it.strip_lin;
    bool pending = false;          // a finished segment whose accumulator tile is not read back yet
    int pend_seg = 0;
    float pend_scale = 1.f;

    auto read_back = [&]() {
      const int dbuf = pend_seg & 1;
      mbar_wait_bounded(d_full + 8 * dbuf, (pend_seg >> 1) & 1, p.status, dead);
      tc_fence_after();
      const uint32_t d_tmem = lane_base + (dbuf ? C::kTmemD1 : C::kTmemD0);
#pragma unroll
      for (int m0 = 0; m0 < NT; m0 += 16) {
        float d[16];
        tc_ld16(d_tmem + m0, d);
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[m0 + i] = fmaf(pend_scale, d[i], acc[m0 + i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(d_empty + 8 * dbuf);
      pending = false;
    };

    while (it.valid()) {
      // ---------------- one slice: this CTA's units of one strip
      const int strip_lin = it.strip_lin;
      const bool is6 = strip_lin >= geo.strips4;
      const int strip = is6 ? strip_lin - geo.strips4 : strip_lin;
      const int nq = strip_quads(is6 ? geo.n6 : geo.n4, strip);
      const bool group = !is6 && geo.groups > 1;
      const bool col_live = c < nq * kQuadCols;       // padded quads of a ragged strip hold no data
      const int swz = (c >> 2) & 1;
      const int s_begin = strip_lin * ups, s_end = s_begin + ups;
      const int slice_u0 = it.u;
      float seg_scale = 1.f;

      while (it.valid() && it.strip_lin == strip_lin) {
        mbar_wait_bounded(full_w + 8 * stage, phase, p.status, dead);
        const uint8_t* st = smem + stage * C::kStageBytes;
        uint4 lo = make_uint4(0, 0, 0, 0), hi = lo, two = lo;
        if (col_live) {
          lo = *reinterpret_cast<const uint4*>(st + c * 32 + 16 * swz);          // words 0..3
          hi = *reinterpret_cast<const uint4*>(st + c * 32 + 16 * (swz ^ 1));    // words 4..7
          if (is6) two = *reinterpret_cast<const uint4*>(st + nq * kInt4UnitQuadBytes + c * 16);
          if (group && it.seg_first(U0)) seg_scale = __half2float(*reinterpret_cast<const half*>(st + kUnitW + c * 2));
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_w + 8 * stage);          // the stage's words are in registers
        mbar_wait_bounded(a_empty + 8 * slot, slot_phase ^ 1, p.status, dead);
        tc_fence_after();
        const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
        const uint32_t twos[4] = {two.x, two.y, two.z, two.w};
        const uint32_t a_tmem = lane_base + C::kTmemA + slot * 32;
#pragma unroll
        for (int step = 0; step < 4; ++step) {
          uint32_t r[8];
          if (is6) {
            expand_fp6(words[2 * step], twos[step], 0, r);
            expand_fp6(words[2 * step + 1], twos[step], 4, r + 4);
          } else {
            expand_int4(words[2 * step], r);
            expand_int4(words[2 * step + 1], r + 4);
          }
          tc_st8(a_tmem + step * 8, r);
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(a_full + 8 * slot);
        const bool seg_end = it.seg_last();
        if (seg_end) {
          if (pending) read_back();                   // the previous segment, one segment late
          pending = true;
          pend_seg = seg;
          pend_scale = seg_scale;
          ++seg;
        }
        it.next();
        if (++stage == kStages) { stage = 0; phase ^= 1; }
        if (++slot == kTmemSlots) { slot = 0; slot_phase ^= 1; }
      }
      if (pending) read_back();
      const int slice_u1 = it.valid() ? it.u : U1;

      // ---------------- the strip is finished for this CTA: write C, or publish a partial
      const bool full_strip = slice_u0 == s_begin && slice_u1 == s_end;
      const int ncols = strip_cols(is6 ? geo.n6 : geo.n4, strip);
      const int gcol = (is6 ? geo.n4 : 0) + strip * kStripCols + c;
      const bool writes = c < ncols;
      float col_scale = 1.f;      // per-channel INT4: s; FP6: s * 4096; group INT4: already applied
      if (writes && !group) {
        const half* sp = p.S + (is6 ? fp6_scale_offset(geo, strip) : int4_scale_offset(geo, strip, 0));
        col_scale = __half2float(__ldg(sp + c)) * (is6 ? 4096.f : 1.f);
      }
      if (full_strip) {
        if (writes) {
#pragma unroll
          for (int m = 0; m < NT; ++m)
            if (m < p.M) p.C[(size_t)m * p.N + gcol] = __float2half_rn(acc[m] * col_scale);
        }
      } else {
        float* slot_base = p.partials + (size_t)(2 * cta + (strip_lin != strip_first ? 1 : 0)) * C::kSlotFloats;
#pragma unroll
        for (int m = 0; m < NT; ++m) __stcg(slot_base + m * kStripCols + c, acc[m]);
        int c_lo = cta, c_hi = cta;
        while (c_lo > 0 && p.sched.bound[c_lo] > s_begin) --c_lo;
        while (c_hi + 1 < p.sched.ctas && p.sched.bound[c_hi + 1] < s_end) ++c_hi;
        named_bar_sync(1, kDequantThreads);          // every thread's partial stores are issued
        if (dtid == 0) {
          int contributors = 0;
          for (int cc = c_lo; cc <= c_hi; ++cc) contributors += p.sched.bound[cc] < p.sched.bound[cc + 1];
          const int last = atomic_add_acq_rel(p.counters + strip_lin, 1) == contributors - 1;
          if (last) p.counters[strip_lin] = 0;       // the workspace is left zeroed, as the reference leaves its locks
          misc[1] = last;
        }
        named_bar_sync(1, kDequantThreads);
        if (misc[1] != 0) {
          // the last CTA to arrive sums the slots in CTA order (deterministic) and writes C
          float sum[NT];
#pragma unroll
          for (int m = 0; m < NT; ++m) sum[m] = 0.f;
          constexpr int kBatch = NT <= 32 ? 2 : 1;   // slots whose loads are in flight together
          for (int cbase = c_lo; cbase <= c_hi; cbase += kBatch) {
            float v[kBatch][NT];
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
              const int cc = cbase + i;
              const bool live = cc <= c_hi && p.sched.bound[cc] < p.sched.bound[cc + 1];
              const int cc_first = live ? p.sched.bound[cc] / ups : 0;
              const float* src = p.partials + (size_t)(2 * (live ? cc : cta) + (live && strip_lin != cc_first ? 1 : 0)) * C::kSlotFloats + c;
#pragma unroll
              for (int m = 0; m < NT; ++m) v[i][m] = live ? __ldcg(src + m * kStripCols) : 0.f;
            }
#pragma unroll
            for (int i = 0; i < kBatch; ++i)
#pragma unroll
              for (int m = 0; m < NT; ++m) sum[m] += v[i][m];
          }
          if (writes) {
#pragma unroll
            for (int m = 0; m < NT; ++m)
              if (m < p.M) p.C[(size_t)m * p.N + gcol] = __float2half_rn(sum[m] * col_scale);
          }
        }
        named_bar_sync(1, kDequantThreads);          // the flag may be rewritten by the next strip
      }
#pragma unroll
      for (int m = 0; m < NT; ++m) acc[m] = 0.f;
    }
  }

  // ---- all roles are done with tensor memory: give it back
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::kTmemCols) : "memory");
  }
}

using Tc5Rows16 = Tc5Cfg<16, 8, 3>;
using Tc5Rows32 = Tc5Cfg<32, 8, 2>;
using Tc5Rows64 = Tc5Cfg<64, 6, 2>;

template <class C>
cudaError_t launch_tc5(const MulParams& p, cudaStream_t stream) {
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(w46_gemm_tc5_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  w46_gemm_tc5_kernel<C><<<p.sched.ctas, kThreads, C::kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

int tc5_rows_per_pass() { return 64; }

// CTAs per SM the kernel is sized for, for `rows` rows of A in one pass.
int tc5_ctas_per_sm(int rows) { return rows <= 16 ? Tc5Rows16::kCtasPerSm : (rows <= 32 ? Tc5Rows32::kCtasPerSm : Tc5Rows64::kCtasPerSm); }

size_t tc5_scratch_bytes(int ctas, int rows) {
  const int nt = rows <= 16 ? 16 : (rows <= 32 ? 32 : 64);
  return (size_t)2 * ctas * nt * kStripCols * sizeof(float);
}

// Runs the GEMM for rows [0, p.M) with p.M <= 64; the host dispatcher loops over larger M.
cudaError_t launch_gemm_tc5(const MulParams& p, cudaStream_t stream) {
  if (p.M <= 16) return launch_tc5<Tc5Rows16>(p, stream);
  if (p.M <= 32) return launch_tc5<Tc5Rows32>(p, stream);
  return launch_tc5<Tc5Rows64>(p, stream);
}

}  // namespace fp6m
