// W(4&6)A16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for up to 128 rows of A (instances for
// 16, 32, 64 and 128 rows; the description below is that of the 16-row instance, the others differ in the
// numbers of teams, stages and tiles - see the configurations at the end of the file).
//
// The product is computed transposed, D[n, m] = sum_k W[k, n] * A[m, k]: the 128 weight columns of
// a strip are the M dimension of tcgen05.mma (one TMEM lane per weight column), the rows of A are
// its N dimension (16), and the dequantised weights are the A operand read from TENSOR MEMORY, so
// they never travel through shared memory.  Legacy mma.sync costs about 32 cycles per m16n8k16
// tile on B200 and cannot keep up with HBM; tcgen05 can: one 128 x 16 x 16 MMA occupies the tensor
// pipe for about 32 cycles whatever its N, i.e. 256 cycles per 8 KB of INT4 weights.
//
// Work unit: a SEGMENT = one 128-row block of one 128-column strip (two 64-row units, 8 KB of INT4
// or 12 KB of FP6 words); the host hands every CTA a contiguous range of blocks in strip-major,
// K-fastest order (fp6m_layout.h, boundaries on whole blocks).  One CTA per SM, five roles that
// only meet at mbarriers:
//   warp 0      weights producer: one bulk TMA copy (cp.async.bulk) per segment into a ring of
//               shared-memory stages.  The first round of copies is issued by fifteen other warps, one
//               stage each, before the rest of the CTA has finished its set-up.
//   warp 1      activations producer: one tiled TMA copy per segment (2 units x 16 rows x 64 halves,
//               128-byte swizzle = the K-major swizzled B operand of the MMA; rows beyond M and
//               units beyond K read as zero).
//   warps 2-7   MMA issuers, two per dequantiser team (one per 64-row unit): four tcgen05.mma
//               (kind::f16, fp32 accumulators in TMEM) per segment each, all accumulating into a tile
//               the team zeroed, then a commit.  A thread needs ~140 cycles per MMA it issues while
//               the tensor pipe needs ~32, so several threads have to issue side by side.  The two
//               commits of a segment tell the epilogue warps that the accumulator tile is ready and
//               the team and the activations producer that operand slot and activation tile are free.
//               Warp 2 owns the TMEM allocation; warp 7 also reads the launch epoch.
//   warps 8-19  three dequantiser TEAMS of four warps; thread = weight column = TMEM lane.  The teams
//               take the CTA's segments in turn.  A thread reads its 2 x 32 bytes of a segment,
//               expands the sixteen words in registers and stores them with tcgen05.st into the
//               segment's TMEM operand slot.  INT4 nibbles become the exact integers q - 8 in fp16
//               (OR into 1024 + q / 64 + q, then subtract 1032 / 72) - bit for bit what the
//               reference's dequant_8int4 feeds its tensor cores (fp6_marlin_cuda_kernel.cu:249-286).
//               FP6 codes become `s 00eee mm` fp16 patterns (exact value / 4096, as dequant_8fp6
//               builds them before its multiply by 4096, :195-237).  A team never waits for an MMA of
//               its own segment: it goes straight on to its next one.
//   warps 20-27 epilogue: two sets of four warps (one warp per TMEM lane quarter); set e takes the
//               segments n = e, e + 2, ...  Every segment has its own accumulator tile; an epilogue warp
//               reads the tile back (tcgen05.ld), multiplies by the column's group scale in fp32 and
//               adds to registers.  At the end of a slice (the CTA's blocks of one strip) set 1 hands its
//               sums to set 0 through shared memory, and set 0 writes C (column scale in fp32, one
//               rounding to fp16) or a split-K partial.  (One set alone needs ~700 cycles per segment:
//               its chain wait - load - wait - add is serial.)
// Rings: 15 weight stages, 6 {operand slot, activation tile, accumulator tile} entries.  Both ring sizes
// are multiples of the number of teams, so a stage or an entry always belongs to the same team and every
// waiter of an mbarrier observes each of its phases in turn (a parity wait that skipped a phase would
// pass early).  Instances whose tiles are too wide to have one per entry keep fewer tiles than entries: the
// epilogue zeroes a tile after reading it and hands it to the issuers of the segment that uses it next.
// The INT4 and the FP6 strips run through separate instantiations of the team loop, so that the
// hot loop holds the instructions of one format only.
// Strips shared by several CTAs are reduced without atomics or fences on the data path: partials are
// stored as {value, tag} 64-bit words, the tag being a per-launch epoch, and the strip's last
// contributor (in CTA order) sums the slots at its end - it only ever waits, with a bound, for
// lower-numbered CTAs.
//
// Programmatic dependent launch: everything up to and including the first round of weight copies runs
// before griddepcontrol.wait; every role passes that wait before its first bounded wait, so a
// long-running predecessor cannot run the bounds out.
//
// Replaces the reference's fp6_kernel_marlin (fp6_marlin/fp6_marlin_cuda_kernel.cu:288-837).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <type_traits>

#include "device_utils.cuh"
#include "fp6m_layout.h"
#include "gemm_params.h"
#include "tc5_common.cuh"
#include "trace.cuh"

namespace fp6m {

namespace {

template <int NT_, int STAGES_, int RING_, int TEAMS_, bool SPLIT_ISSUE_, int DRING_ = RING_>
struct Tc5Cfg {
  static constexpr int kTeams = TEAMS_;
  // Two issuers per team.  kSplitIssue: both work on every segment of the team, one 64-row unit each, adding to
  // a tile the team zeroed - the order in which the tensor core retires the two units is not fixed, so the last
  // bit of a sum may differ from run to run.  Otherwise they take the team's segments in turn, eight MMAs each:
  // one issuing thread per tile, a fixed order of additions, bit-identical results from run to run.
  static constexpr bool kSplitIssue = SPLIT_ISSUE_;
  static constexpr int kIssuers = 2 * TEAMS_;
  // warp 0: weights producer, warp 1: activations producer, warps 2.. : MMA issuers, then (from a
  // multiple of four, so that warp % 4 is the TMEM lane quarter) four dequantiser warps per team and
  // the four epilogue warps
  static constexpr int kDeqBase = (2 + kIssuers + 3) & ~3;
  static constexpr int kEpiBase = kDeqBase + 4 * kTeams;
  static constexpr int kEpiSets = NT_ > 64 ? 4 : 2;       // a thread of an epilogue set accumulates at most 32 rows
  static constexpr int kThreads = 32 * (kEpiBase + 4 * kEpiSets);
  // Groups of 128 threads that share the reduction of a strip at the CTA's end.  Four: the epilogue sets, with
  // the first two teams where there are only two sets.  Eight (128-row tiles, where a strip's partials are 128 KB
  // per contributor and the reduction is a chain of round trips to L2): the four sets, the two teams and the
  // eight warps in front of them (producers, issuers, two spare warps), sixteen rows each.
  // (measured at 128 rows, K = N = 8192: 32.0 -> 27.7 us per GEMM; K = N = 4096: 26.0 -> 19.9.  Unequal shares -
  // fewer rows for the epilogue sets, which get there last - measured: 128 rows, sets x 8 + the others x 24: 30.0 us;
  // 64 rows, sets x 8 + teams and front warps x 12: the same as four groups; 32 rows, sets x 4 + three teams x 8:
  // -1.7 %, but the 16-row instance compiled from that source ran 0.7 % slower.)
  static constexpr int kReduceGroups = (kEpiSets == 4 && kTeams == 2 && kDeqBase == 8) ? 8 : 4;
  static_assert(kTeams >= 2 && STAGES_ <= 4 * kTeams + 4 * kEpiSets, "the first round of weight copies is issued by one warp per stage");
  static constexpr int kEpochWarp = 2 + kIssuers - 1;
  static constexpr int NT = NT_;                       // rows of A per pass = N of the MMA
  static constexpr int kStages = STAGES_;              // shared-memory stages of packed words (one segment each)
  static constexpr int kRing = RING_;                  // ring of {activation tile, TMEM operand slot}
  // Accumulator tiles.  kDRing == kRing: every ring entry has its own tile, the team that fills the entry
  // zeroes it.  Fewer tiles (wide tiles do not fit six times): segment n uses tile n % kDRing, the epilogue
  // zeroes a tile after reading it and hands it to the issuers of segment n + kDRing.
  static constexpr int kDRing = DRING_;
  static constexpr bool kDecoupled = kDRing != kRing;
  static_assert(kDRing <= kRing && kDRing % 2 == 0, "accumulator tiles");
  static_assert(!kDecoupled || NT_ > 16, "with fewer tiles than entries both epilogue sets read every segment");
  static constexpr int kActUnitBytes = NT * 128;       // NT rows x 64 halves
  static constexpr int kActBytes = 2 * kActUnitBytes;
  static constexpr int kNumBars = 2 * kStages + 4 * kRing + 1;
  // A stage and a ring entry must always belong to the same team: then every waiter of a barrier sees
  // each of its phases (a team that came back to a barrier two phases later would pass a parity wait early).
  static_assert(kStages % kTeams == 0 && kRing % kTeams == 0, "ring sizes must be multiples of the number of teams");

  static_assert(kRing <= kIssuers, "the first round of activation copies is issued by one issuer warp per entry");
  static_assert(kRing == 2 * kTeams, "each team owns two ring entries (one per issuer when the issuers take turns)");
  // the group scale (fp16 bits in a word) of every column of the segment in a ring entry; with fewer
  // accumulator tiles than entries a team may be a whole round ahead of the epilogue: two sets of scales
  static constexpr int kScaleRingBytes = (kDecoupled ? 2 : 1) * kRing * kStripCols * 4;
  // Up to 16 rows the two epilogue sets take the segments in turn and pool their sums at the end of a slice;
  // with more rows each set reads its half of the rows of every segment (the sums would not fit in registers).
  static constexpr bool kRowSplit = NT > 16;
  static constexpr int kEpiRows = kRowSplit ? NT / kEpiSets : NT;     // rows a thread of an epilogue set accumulates
  static constexpr int kXchBytes = kRowSplit ? 0 : NT * kStripCols * 4;   // the second epilogue set's sums of a slice
  static_assert(kRowSplit || kRing % kEpiSets == 0, "a ring entry always belongs to the same epilogue set");
  static constexpr int kSmemBytes = kStages * kStageW + kRing * kActBytes + kScaleRingBytes + kXchBytes + kNumBars * 8 + 64 + 1024;   // + alignment slack
  static constexpr int kTmemD = 0, kTmemA = kDRing * NT;  // accumulator tiles, then operand slots of 64 columns
  static constexpr int kTmemUsed = kTmemA + kRing * 64;
  static constexpr int kTmemCols = kTmemUsed <= 128 ? 128 : (kTmemUsed <= 256 ? 256 : 512);
  static_assert(kTmemUsed <= 512, "tensor memory has 512 columns");
  static constexpr int kSlotFloats = NT * kStripCols;
  static constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
};

// activations of one segment: the box {64 halves, NT rows, 2 units} at unit `unit` of K
__device__ __forceinline__ void tma_load_act_segment(uint32_t dst, const CUtensorMap* map, int unit, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(0), "r"(0), "r"(unit), "r"(bar) : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// Bytes of one segment of (linear) strip `s`.
__device__ __forceinline__ uint32_t segment_bytes(const Geometry& geo, int s) {
  return s < geo.strips4 ? 2u * strip_quads(geo.n4, s) * kInt4UnitQuadBytes
                         : 2u * strip_quads(geo.n6, s - geo.strips4) * kFp6UnitQuadBytes;
}
// Byte offset of block `blk` of strip `s` in the packed weights (blocks of a strip, and strips, follow
// one another without gaps).
__device__ __forceinline__ int64_t segment_offset(const Geometry& geo, int s, int blk) {
  return s < geo.strips4 ? int4_unit_offset(geo, s, 2 * blk) : fp6_unit_offset(geo, s - geo.strips4, 2 * blk);
}

// Group scales of one segment: nq * 64 bytes behind the packed words of its stage (FP6 and per-channel strips
// have none).  Offset of the scales inside a stage: INT4 segments fill at most 8192 of the kStageW bytes.
constexpr uint32_t kStageScaleOff = 8192;
__device__ __forceinline__ uint32_t segment_scale_bytes(const Geometry& geo, int s) {
  return (s < geo.strips4 && geo.groups > 1) ? (uint32_t)strip_quads(geo.n4, s) * kQuadCols * 2u : 0u;
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }
__device__ __forceinline__ void sts_u32(uint32_t addr, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
  unsigned short v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}

// Expands one 64-row unit of this thread's column (eight packed words, plus four two-bit words for FP6)
// into 32 TMEM columns at a_tmem.
template <bool IS6>
__device__ __forceinline__ void expand_words(const uint4& lo, const uint4& hi, const uint4& two, uint32_t a_tmem) {
  const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  if constexpr (IS6) {
    const uint32_t twos[4] = {two.x, two.y, two.z, two.w};
#pragma unroll
    for (int step = 0; step < 4; ++step) {
      uint32_t regs[8];
      expand_fp6(words[2 * step], twos[step], 0, regs);
      expand_fp6(words[2 * step + 1], twos[step], 4, regs + 4);
      tc_st8(a_tmem + step * 8, regs);
    }
  } else {
#pragma unroll
    for (int step = 0; step < 4; ++step) {
      uint32_t regs[8];
      expand_int4(words[2 * step], regs);
      expand_int4(words[2 * step + 1], regs + 4);
      tc_st8(a_tmem + step * 8, regs);
    }
  }
}

template <class C>
__global__ void __launch_bounds__(C::kThreads, 1) w46_gemm_tc5_kernel(const __grid_constant__ MulParams p, const __grid_constant__ CUtensorMap amap) {
  constexpr int NT = C::NT, S = C::kStages, R = C::kRing, T = C::kTeams;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // the swizzled activation stages must start on 1024-byte boundaries
  const uint32_t smem0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t act_base = smem0 + S * kStageW;
  const uint32_t scale_ring = act_base + R * C::kActBytes;      // [entry][column] fp32
  const uint32_t xch = scale_ring + C::kScaleRingBytes;         // [row][column] fp32
  const uint32_t bars0 = xch + C::kXchBytes;
  const uint32_t w_full = bars0, w_empty = w_full + 8 * S;
  const uint32_t act_full = w_empty + 8 * S, ready = act_full + 8 * R, done = ready + 8 * R;
  const uint32_t d_free = done + 8 * R;        // the accumulator tile has been read back
  const uint32_t epoch_bar = d_free + 8 * R;   // misc[1] holds the launch epoch
  uint32_t* misc = reinterpret_cast<uint32_t*>(smem_raw + (bars0 - smem_u32(smem_raw)) + 8 * C::kNumBars);   // [0] TMEM base, [1] launch epoch

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x;
  const Geometry& geo = p.geo;
  const int kb = geo.k128;                       // blocks (segments) per strip
  // the CTA's range of blocks (the host rounds the unit boundaries of this kernel to whole blocks)
  const int B0 = p.sched.bound[cta] >> 1, B1 = p.sched.bound[cta + 1] >> 1;
  const int nseg = B1 - B0;
  FP6M_TRACE_DECL(trace);
  FP6M_TRACE_INIT(trace, cta, warp, lane);
#ifdef FP6M_TRACE
  const unsigned long long t_launch = global_ns();
#endif
  launch_dependents();
  if (nseg <= 0) {                     // no work: still counted, see read_epoch_and_count
    if (tid == 0) {
      grid_dependency_wait();
      read_epoch_and_count(p.epochs, gridDim.x);
    }
    return;
  }
  WaitState ws;
  const int s_first = B0 / kb, blk_first = B0 - s_first * kb;
  const uint64_t policy = make_evict_first_policy();
  FP6M_TRACE_EVENT(trace, 30, 0);              // the CTA's range is known (first reads of the kernel parameters)

  // ---- set-up.  Lane 0 of warp kDeqBase + i initialises the barriers of weight stage i and issues the
  // stage's first copy at once (segment i); other threads initialise the remaining barriers, warp 2
  // allocates tensor memory meanwhile.
  if (warp >= C::kDeqBase && warp < C::kDeqBase + S) {
    const int st = warp - C::kDeqBase;
    if (lane == 0) {
      mbar_init(w_full + 8 * st, 1);       // the expect_tx arrival of the weights producer
      mbar_init(w_empty + 8 * st, 128);    // every thread of the team that read the stage has used its words
      mbar_fence_init();
      FP6M_TRACE_EVENT(trace, 31, st);         // the stage's barriers exist
      if (st < nseg) {
        int s = s_first, blk = blk_first + st;
        while (blk >= kb) { blk -= kb; ++s; }
        const uint32_t bytes = segment_bytes(geo, s), sbytes = segment_scale_bytes(geo, s);
        const uint8_t* src = p.B + segment_offset(geo, s, blk);
        FP6M_TRACE_EVENT(trace, 32, st);       // source address and size computed
        (void)src;
        mbar_arrive_expect_tx(w_full + 8 * st, bytes + sbytes);
        tma_load_1d_stream(smem0 + st * kStageW, p.B + segment_offset(geo, s, blk), bytes, w_full + 8 * st, policy);
        if (sbytes)
          tma_load_1d_stream(smem0 + st * kStageW + kStageScaleOff, p.S + int4_scale_offset(geo, s, blk), sbytes, w_full + 8 * st, policy);
      }
      FP6M_TRACE_EVENT(trace, 1, st);
    }
  }
  if (tid < 4 * R + 1) {
    const int i = tid;
    // act_full: expect_tx arrival of the activations producer; ready: every thread of the segment's team
    // stored its operands into TMEM; done: the commit(s) of the segment's issuer(s); d_free: every thread of
    // the entry's epilogue set has read the tile.  (All lanes arrive: no election, no branch.)
    const uint32_t count = i < R ? 1u : (i < 2 * R ? 128u : (i < 3 * R ? (C::kSplitIssue ? 2u : 1u) : (i < 4 * R ? (C::kRowSplit ? 128u * C::kEpiSets : 128u) : 1u)));
    mbar_init(act_full + 8 * i, count);
    mbar_fence_init();
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(misc)), "r"(C::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  FP6M_TRACE_EVENT(trace, 2, 0);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = misc[0];
  // Everything below depends, directly or through the MMAs, on the activations, which the previous
  // kernel of the stream may still be writing: all bounded waits that depend on them start after it has
  // completed.  With p.expand_early the dequantiser teams go ahead: their first two segments each need the
  // (static) weights and fresh ring entries only, so their operands are in tensor memory when the activations
  // arrive (the host switches it on where a CTA's main loop is short against its set-up).
  const bool is_team_warp = p.expand_early && warp >= C::kDeqBase && warp < C::kEpiBase;
  if (!is_team_warp) grid_dependency_wait();
  FP6M_TRACE_EVENT(trace, 4, 0);

  if (warp == C::kEpochWarp && lane == 0) {
    // the tag of this launch's split-K partials is epoch + 1
    const uint32_t e = read_epoch_and_count(p.epochs, gridDim.x);
    misc[1] = e;
    mbar_arrive(epoch_bar);
  }
  const bool act3d = (p.K & 63) == 0;        // the host encoded the three-dimensional map
  // activations of the block `blk` of K into ring entry r
  auto load_activations = [&](int blk, int r) {
    const uint32_t dst = act_base + r * C::kActBytes;
    mbar_arrive_expect_tx(act_full + 8 * r, C::kActBytes);
    if (act3d) {
      // both units of the block in one copy (a unit beyond K reads as zero)
      tma_load_act_segment(dst, &amap, 2 * blk, act_full + 8 * r);
    } else {
      tma_load_act(dst, &amap, 2 * blk * kUnitRows, act_full + 8 * r);
      tma_load_act(dst + C::kActUnitBytes, &amap, (2 * blk + 1) * kUnitRows, act_full + 8 * r);
    }
  };

  // ---- pieces shared by the epilogue sets and the dequantiser teams (thread = weight column c of a strip)
  const int quarter = warp & 3;                    // the TMEM lanes this warp may touch
  const int c = quarter * 32 + lane;               // weight column inside the strip = TMEM lane
  struct Slice {
    int strip_lin, strip, b0, b1;       // blocks [b0, b1) of the strip belong to this CTA
    bool is6, group;
  };
  auto open_slice = [&](int strip_lin, int b0, int b1) {
    Slice sl;
    sl.strip_lin = strip_lin;
    sl.is6 = strip_lin >= geo.strips4;
    sl.strip = sl.is6 ? strip_lin - geo.strips4 : strip_lin;
    sl.group = !sl.is6 && geo.groups > 1;
    sl.b0 = b0;
    sl.b1 = b1;
    return sl;
  };
  auto column_scale = [&](const Slice& sl, bool writes) {
    float col_scale = 1.f;      // per-channel INT4: s; FP6: s * 4096; group INT4: already applied
    if (writes && !sl.group) {
      const half* sp = p.S + (sl.is6 ? fp6_scale_offset(geo, sl.strip) : int4_scale_offset(geo, sl.strip, 0));
      col_scale = __half2float(__ldg(sp + c)) * (sl.is6 ? 4096.f : 1.f);
    }
    return col_scale;
  };
  // Split-K without atomics or fences: a partial is stored as 64-bit words {fp32 value, tag}, the
  // tag being the launch epoch + 1 (the epoch word lives in the scratch header and is advanced once
  // per launch, see read_epoch_and_count, so every launch - also a replay of a captured graph - uses
  // fresh tags and stale slots of earlier launches never match).
  // The reducer of a strip is its LAST contributor in CTA order, i.e. the CTA whose slice reaches
  // the end of the strip; that slice is the first one of the CTA, and the reduction is postponed to
  // the CTA's end, when the other contributors have normally finished.  It then reads the slots of
  // the lower-numbered contributors, spinning (bounded) on words whose tag has not arrived, sums in
  // CTA order (deterministic) and writes C.  Only lower-numbered CTAs are waited for, and those were
  // dispatched earlier.  Only the first and the last slice of a CTA can be partial; the caller's
  // workspace is not touched.
  auto slot_of = [&](int cc, int strip_lin) {
    // slot 0 holds the partial of a CTA's first strip, slot 1 that of its last strip
    const int cc_first = (p.sched.bound[cc] >> 1) / kb;
    return p.partials + (size_t)(2 * cc + (strip_lin != cc_first ? 1 : 0)) * C::kSlotFloats + c;
  };
  // After its last segment: the strip whose LAST contributor (in CTA order) this CTA is - the strip its range
  // starts inside of and runs to the end of.  kReduceGroups groups of 128 threads take part, each with its share
  // of the rows: the epilogue sets, dequantiser teams (which have nothing else left to do) and, with eight
  // groups, the warps in front of them, so that many tagged words travel together.  A
  // value is added in CTA order, so the sum does not depend on the timing.  (Measured and dropped: giving
  // all of it to the warps that run out of work first - teams, issuers - ends the reducing CTAs earlier but
  // lengthened the step of the square layer by 4 %.)
  auto reduce_shared_strip = [&](int group) {
    if (!(blk_first > 0 && nseg >= kb - blk_first)) return;         // this CTA is no strip's last contributor
    constexpr int RR = NT / C::kReduceGroups;                        // rows of this thread
    // 64-bit loads in flight per thread: the 128-row instance runs 1024 threads of 64 registers (16 in flight spill
    // there and are 3 % slower)
    constexpr int kInFlight = NT > 64 ? 8 : 16;
    constexpr int kChunk = RR < kInFlight ? RR : kInFlight;          // rows per round
    constexpr int kBatch = kInFlight / kChunk;                       // contributors per round
    const int rr0 = group * RR;
    const int reduce_strip = s_first;
    mbar_wait(epoch_bar, 0, ws);                                     // completed long ago: orders the read of misc[1]
    const uint32_t reduce_tag = misc[1] + 1;
    const Slice sl = open_slice(reduce_strip, 0, kb);
    const int s_begin = reduce_strip * kb;         // first block of the strip
    int c_lo = cta;
    while (c_lo > 0 && (p.sched.bound[c_lo] >> 1) > s_begin) --c_lo;
    float sum[RR];
#pragma unroll
    for (int m = 0; m < RR; ++m) sum[m] = 0.f;
    FP6M_TRACE_EVENT(trace, 25, group);
#pragma unroll 1
    for (int cbase = c_lo; cbase <= cta; cbase += kBatch) {
      bool live[kBatch];
      const unsigned long long* src[kBatch];
#pragma unroll
      for (int i = 0; i < kBatch; ++i) {
        const int cc = cbase + i;
        live[i] = cc <= cta && p.sched.bound[cc] < p.sched.bound[cc + 1];       // a CTA without work stored nothing
        src[i] = slot_of(live[i] ? cc : cta, reduce_strip) + rr0 * kStripCols;
      }
#pragma unroll
      for (int m0 = 0; m0 < RR; m0 += kChunk) {
        unsigned long long v[kBatch][kChunk];
        bool all_here = false;
#pragma unroll 1
        for (int spin = 0; spin < (1 << 20) && !all_here; ++spin) {
#pragma unroll
          for (int i = 0; i < kBatch; ++i)
#pragma unroll
            for (int m = 0; m < kChunk; ++m) v[i][m] = ld_relaxed_u64(src[i] + (m0 + m) * kStripCols);
          all_here = true;
#pragma unroll
          for (int i = 0; i < kBatch; ++i)
#pragma unroll
            for (int m = 0; m < kChunk; ++m) all_here = all_here && (!live[i] || (uint32_t)(v[i][m] >> 32) == reduce_tag);
          if (ws.failed) break;                       // a wait of this thread ran out before: do not wait again
          if (!all_here) __nanosleep(64);             // the teams arrive here early: leave the issue slots to the others
        }
        if (!all_here) ws.failed = 1;
        FP6M_TRACE_EVENT(trace, 26, group);
#pragma unroll
        for (int i = 0; i < kBatch; ++i)
#pragma unroll
          for (int m = 0; m < kChunk; ++m) sum[m0 + m] += live[i] ? __uint_as_float((uint32_t)v[i][m]) : 0.f;
      }
    }
    const int ncols = strip_cols(sl.is6 ? geo.n6 : geo.n4, sl.strip);
    const bool writes = c < ncols;
    const float col_scale = column_scale(sl, writes);
#pragma unroll
    for (int m = 0; m < RR; ++m) sum[m] *= col_scale;
    store_column_rows<RR>(p, rr0, sl.is6, sl.strip * kStripCols + c, sum, writes);
    FP6M_TRACE_EVENT(trace, 27, group);
  };

  if (warp == 0) {
    // ================================================================== weights producer, segments S..
    if (lane == 0 && nseg > S) {
      int s = s_first, blk = blk_first + S;
      while (blk >= kb) { blk -= kb; ++s; }
      const uint8_t* src = p.B + segment_offset(geo, s, blk);
      uint32_t bytes = segment_bytes(geo, s), sbytes = segment_scale_bytes(geo, s);
      const uint8_t* ssrc = reinterpret_cast<const uint8_t*>(p.S + (sbytes ? int4_scale_offset(geo, s, blk) : 0));
      int stage = 0;
      uint32_t phase = 0;                      // parity of the stage's previous use
      for (int n = S; n < nseg; ++n) {
        mbar_wait<200>(w_empty + 8 * stage, phase, ws);
        mbar_arrive_expect_tx(w_full + 8 * stage, bytes + sbytes);
        tma_load_1d_stream(smem0 + stage * kStageW, src, bytes, w_full + 8 * stage, policy);
        if (sbytes) tma_load_1d_stream(smem0 + stage * kStageW + kStageScaleOff, ssrc, sbytes, w_full + 8 * stage, policy);
        FP6M_TRACE_EVENT(trace, 1, n);
        src += bytes;                          // blocks and strips follow one another without gaps
        ssrc += sbytes;                        // and so do the groups of a strip
        if (++blk == kb) {
          blk = 0; ++s;
          bytes = segment_bytes(geo, s);
          sbytes = segment_scale_bytes(geo, s);
          if (sbytes) ssrc = reinterpret_cast<const uint8_t*>(p.S + int4_scale_offset(geo, s, 0));
        }
        if (++stage == S) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ================================================================== activations producer, segments R..
    if (lane == 0 && nseg > R) {
      int blk = (blk_first + R) % kb;
      int r = 0;
      uint32_t phase = 0;                      // parity of the entry's previous use
      for (int n = R; n < nseg; ++n) {
        mbar_wait<200>(done + 8 * r, phase, ws);     // the MMAs that read this tile are done
        load_activations(blk, r);
        FP6M_TRACE_EVENT(trace, 5, n);
        if (++blk == kb) blk = 0;
        if (++r == R) { r = 0; phase ^= 1; }
      }
    }
  } else if (warp >= 2 && warp < 2 + C::kIssuers) {
    // ================================================================== MMA issuers
    // Split issue: issuer i serves team i / 2 and unit i % 2 of its segments n = team, team + T, ... (ring
    // entry n % R): four MMAs that add to the tile the team zeroed, then a commit.  Otherwise issuer r owns
    // ring entry r and issues all eight MMAs of its segments.  The whole warp waits (warp-uniform control
    // flow); one fixed lane issues the tcgen05 instructions, so that the commit tracks the MMAs before it.
    // First of all, issuer i loads the activations of segment i.
    const int mine = warp - 2;
    if (lane == 0 && mine < R && mine < nseg) {
      load_activations((blk_first + mine) % kb, mine);
      FP6M_TRACE_EVENT(trace, 5, mine);
    }
    __syncwarp();
    constexpr uint32_t kStepDesc = 32 >> 4;            // 16 halves along a 128-byte row
    if constexpr (C::kSplitIssue) {
      const int team = mine >> 1, unit = mine & 1;
      int r = team;
      uint32_t rphase = 0;
      const uint64_t desc0 = wide_act_desc(act_base) + (uint64_t)(unit * (C::kActUnitBytes >> 4));
      for (int n = team; n < nseg; n += T) {
        mbar_wait<32>(ready + 8 * r, rphase, ws);
        mbar_wait<32>(act_full + 8 * r, rphase, ws);
        if constexpr (C::kDecoupled) mbar_wait<32>(d_free + 8 * r, rphase, ws);      // the entry's accumulator tile is free and zero
        tc_fence_after();
        FP6M_TRACE_EVENT(trace, 6, n);
        const uint32_t d_tmem = tmem + C::kTmemD + (C::kDecoupled ? n % C::kDRing : r) * NT;
        const uint32_t a_tmem = tmem + C::kTmemA + r * 64 + unit * 32;
        // the descriptor's low 14 bits hold the address / 16: adding an offset never carries out of them
        const uint64_t desc = desc0 + (uint64_t)(r * (C::kActBytes >> 4));
        if (lane == 0) {
          tc_mma_unit<kStepDesc>(d_tmem, a_tmem, desc, C::kIdesc, 1u);
          tc_commit(done + 8 * r);
        }
        __syncwarp();
        FP6M_TRACE_EVENT(trace, 7, n);
        r += T;
        if (r >= R) { r -= R; rphase ^= 1; }
      }
    } else {
      // issuer r owns ring entry r: the segments n = r, r + R, ...; the first MMA overwrites the tile
      const int r = mine;
      uint32_t rphase = 0;
      const uint64_t desc = wide_act_desc(act_base) + (uint64_t)(r * (C::kActBytes >> 4));
      const uint32_t a_tmem = tmem + C::kTmemA + r * 64;
      for (int n = r; n < nseg; n += R) {
        const uint32_t d_tmem = tmem + C::kTmemD + (C::kDecoupled ? n % C::kDRing : r) * NT;
        mbar_wait<32>(ready + 8 * r, rphase, ws);
        mbar_wait<32>(act_full + 8 * r, rphase, ws);
        if constexpr (C::kDecoupled) mbar_wait<32>(d_free + 8 * r, rphase, ws);      // the entry's accumulator tile is free
        tc_fence_after();
        FP6M_TRACE_EVENT(trace, 6, n);
        if (lane == 0) {
          tc_mma_unit<kStepDesc>(d_tmem, a_tmem, desc, C::kIdesc, 0u);
          tc_mma_unit<kStepDesc>(d_tmem, a_tmem + 32, desc + (C::kActUnitBytes >> 4), C::kIdesc, 1u);
          tc_commit(done + 8 * r);
        }
        __syncwarp();
        FP6M_TRACE_EVENT(trace, 7, n);
        rphase ^= 1;
      }
    }
  } else if (warp >= C::kDeqBase && warp < C::kEpiBase) {
    // ================================================================== dequantisers
    // thread = weight column = TMEM lane; team t expands the segments n = t, t + T, ...
    const int team = (warp - C::kDeqBase) >> 2;
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t a_base = lane_base + C::kTmemA;       // + r * 64
    const uint32_t d_base = lane_base + C::kTmemD;       // + r * NT
    const uint32_t lds_lo = c * 32 + 16 * ((c >> 2) & 1);          // words 0..3 of the column; words 4..7 at ^ 16
    const uint32_t lds_hi = lds_lo ^ 16;

    // The packed words of a segment are loaded one iteration ahead: while the TMEM stores of segment n drain,
    // the team already waits for and loads segment n + T.
    struct Words {
      uint4 lo0, hi0, lo1, hi1;      // unit 0 and unit 1: words 0..3, 4..7 of this thread's column
      uint4 two0, two1;              // FP6: the two-bit words of the units
      uint32_t scale_raw;            // fp16 bits of the column's group scale (1.0 where the strip has none)
    };
    struct Strip {
      int n_end;                     // first segment (of the CTA) beyond the strip
      bool is6, scaled;
      uint32_t unit_bytes, two_off;
    };
    auto open_strip = [&](int s) {
      Strip sp;
      sp.n_end = min(nseg, (s + 1) * kb - B0);
      sp.is6 = s >= geo.strips4;
      const int nq = sp.is6 ? strip_quads(geo.n6, s - geo.strips4) : strip_quads(geo.n4, s);
      sp.unit_bytes = nq * (sp.is6 ? kFp6UnitQuadBytes : kInt4UnitQuadBytes);
      sp.two_off = nq * kInt4UnitQuadBytes + c * 16;
      sp.scaled = !sp.is6 && geo.groups > 1;       // the group scales came with the packed words
      return sp;
    };
    // Columns of padded quads read stale bytes of the stage and produce values nobody stores.
    auto load_words = [&](const Strip& sp, int stage, Words& w) {
      const uint32_t st = smem0 + stage * kStageW;
      w.lo0 = lds128(st + lds_lo);
      w.hi0 = lds128(st + lds_hi);
      w.lo1 = lds128(st + sp.unit_bytes + lds_lo);
      w.hi1 = lds128(st + sp.unit_bytes + lds_hi);
      if (sp.is6) {
        w.two0 = lds128(st + sp.two_off);
        w.two1 = lds128(st + sp.unit_bytes + sp.two_off);
      }
      w.scale_raw = sp.scaled ? lds_u16(st + kStageScaleOff + 2 * c) : 0x3C00u;
    };

    int n = team, stage = team, r = team, s = s_first;
    uint32_t wphase = 0, rphase = 1;                 // rphase: parity of the entry's previous use (a fresh barrier passes parity 1)
    Strip sp = open_strip(s);
    while (n >= sp.n_end && sp.n_end < nseg) sp = open_strip(++s);
    Words w;
    if (n < nseg) {
      mbar_wait(w_full + 8 * stage, wphase, ws);
      load_words(sp, stage, w);
    }
    bool after_grid_wait = !p.expand_early;
#pragma unroll 1
    while (n < nseg) {
      FP6M_TRACE_EVENT(trace, 10, n);
      if (n >= R && !after_grid_wait) {
        // from the team's third segment on its waits depend on the MMAs, hence on the previous kernel
        grid_dependency_wait();
        after_grid_wait = true;
      }
      if constexpr (C::kDecoupled) {
        // the MMAs of the segment that used this ring entry before are done
        mbar_wait(done + 8 * r, rphase, ws);
      } else {
        // the epilogue has read the sums of the segment that used this ring entry before (so its MMAs are done too)
        mbar_wait(d_free + 8 * r, rphase, ws);
      }
      tc_fence_after();
      FP6M_TRACE_EVENT(trace, 12, n);
      const uint32_t a_tmem = a_base + r * 64;
      // this column's scale of the block goes on to the epilogue warps
      if constexpr (C::kDecoupled) {
        sts_u32(scale_ring + (((rphase ^ 1) * R + r) * kStripCols + c) * 4, w.scale_raw);     // rphase ^ 1: parity of this use
      } else {
        sts_u32(scale_ring + (r * kStripCols + c) * 4, w.scale_raw);
        if constexpr (C::kSplitIssue) tc_st_zero<NT>(d_base + r * NT);       // both issuers' MMAs accumulate
      }
      if (sp.is6) {
        expand_words<true>(w.lo0, w.hi0, w.two0, a_tmem);
        expand_words<true>(w.lo1, w.hi1, w.two1, a_tmem + 32);
      } else {
        expand_words<false>(w.lo0, w.hi0, w.two0, a_tmem);
        expand_words<false>(w.lo1, w.hi1, w.two1, a_tmem + 32);
      }
      FP6M_TRACE_EVENT(trace, 17, n);
      mbar_arrive(w_empty + 8 * stage);                         // this thread has used its words of the stage
      // the team's next segment: wait for it and load its words while the stores above drain
      const int n_next = n + T;
      stage += T;
      if (stage >= S) { stage -= S; wphase ^= 1; }
      bool was6 = sp.is6;
      while (n_next >= sp.n_end && sp.n_end < nseg) sp = open_strip(++s);
      if (n_next < nseg) {
        mbar_wait(w_full + 8 * stage, wphase, ws);
        load_words(sp, stage, w);
      }
      (void)was6;
      FP6M_TRACE_EVENT(trace, 18, n);
      tc_wait_st();
      FP6M_TRACE_EVENT(trace, 19, n);
      tc_fence_before();
      mbar_arrive(ready + 8 * r);
      FP6M_TRACE_EVENT(trace, 13, n);
      r += T;
      if (r >= R) { r -= R; rphase ^= 1; }
      n = n_next;
    }
    if (!after_grid_wait) grid_dependency_wait();
    // groups 0.. are the epilogue sets
    if (C::kReduceGroups == 8) reduce_shared_strip(4 + team);
    else if (C::kEpiSets == 2 && team < 2) reduce_shared_strip(2 + team);
  } else if (warp >= C::kEpiBase) {
    // ================================================================== epilogue
    // Two sets of one warp per lane quarter; thread = weight column.  Set e reads the accumulator tiles of
    // the segments n = e, e + 2, ... back, scales and accumulates; at the end of a slice set 1 passes its
    // sums to set 0, which writes the slice out (sums added in the order set 0 + set 1: fixed).
    constexpr int kEpiThreads = 128 * C::kEpiSets;
    const int eset = (warp - C::kEpiBase) >> 2;
    const uint32_t d_base = tmem + ((uint32_t)(quarter * 32) << 16) + C::kTmemD;       // + r * NT

    constexpr int ROWS = C::kEpiRows;
    const int row0 = C::kRowSplit ? eset * ROWS : 0;          // this set's rows of A and C (all of them when the sets take turns)
    auto write_strip = [&](const Slice& sl, const float (&v)[ROWS]) {
      const int ncols = strip_cols(sl.is6 ? geo.n6 : geo.n4, sl.strip);
      const bool writes = c < ncols;
      const float col_scale = column_scale(sl, writes);
      float out[ROWS];
#pragma unroll
      for (int m = 0; m < ROWS; ++m) out[m] = v[m] * col_scale;
      store_column_rows<ROWS>(p, row0, sl.is6, sl.strip * kStripCols + c, out, writes);
    };
    auto finish_slice = [&](const Slice& sl, const float (&out)[ROWS]) {
      if (sl.b0 == 0 && sl.b1 == kb) {               // the whole strip was ours
        write_strip(sl, out);
        return;
      }
      mbar_wait(epoch_bar, 0, ws);   // completed long ago: orders the read of misc[1]
      const uint32_t tag = misc[1] + 1;
      unsigned long long* slot = slot_of(cta, sl.strip_lin) + row0 * kStripCols;
#pragma unroll
      for (int m = 0; m < ROWS; ++m)
        st_relaxed_u64(slot + m * kStripCols, ((unsigned long long)tag << 32) | __float_as_uint(out[m]));
    };
    float acc[ROWS];
#pragma unroll
    for (int m = 0; m < ROWS; ++m) acc[m] = 0.f;
    constexpr int kStep = C::kRowSplit ? 1 : C::kEpiSets;      // segments from one of this set's to its next
    if (!C::kRowSplit && eset == 0) named_bar_arrive(2, kEpiThreads);       // the exchange buffer starts out free
    int n = C::kRowSplit ? 0 : eset, r = n, n_first = 0;    // n_first: first segment of the current slice
    uint32_t rphase = 0;
    if constexpr (C::kDecoupled) {
      // the accumulator tiles start out free; when two issuers add to a tile it must start out zero
      if constexpr (C::kSplitIssue) {
#pragma unroll
        for (int d = 0; d < C::kDRing; ++d) tc_st_zero<ROWS>(d_base + d * NT + row0);
        tc_wait_st();
        tc_fence_before();
      }
#pragma unroll
      for (int d = 0; d < C::kDRing; ++d) mbar_arrive(d_free + 8 * d);
    }
    for (int s = s_first; n_first < nseg; ++s) {
      const int b0 = s == s_first ? blk_first : 0;
      const int n_end = min(nseg, (s + 1) * kb - B0);
      const Slice sl = open_slice(s, b0, b0 + (n_end - n_first));
#pragma unroll 1
      for (; n < n_end; n += kStep) {
        float scale;
        uint32_t d_tile;
        if constexpr (C::kDecoupled) {
          // (No wait on `ready`: the team may complete the entry's next phase of it before this thread gets here;
          // `done` cannot run ahead, the next MMAs into this tile wait for this thread.)
          mbar_wait(done + 8 * r, rphase, ws);
          scale = __half2float(__ushort_as_half((unsigned short)lds_u32(scale_ring + ((rphase * R + r) * kStripCols + c) * 4)));
          d_tile = d_base + (n % C::kDRing) * NT + row0;
        } else {
          // the team's arrival on `ready` published the column scales of this entry
          mbar_wait(ready + 8 * r, rphase, ws);
          scale = __half2float(__ushort_as_half((unsigned short)lds_u32(scale_ring + (r * kStripCols + c) * 4)));
          mbar_wait(done + 8 * r, rphase, ws);
          d_tile = d_base + r * NT + row0;
        }
        tc_fence_after();
        FP6M_TRACE_EVENT(trace, 15, n);
#pragma unroll
        for (int m0 = 0; m0 < ROWS; m0 += 16) {
          float d[16];
          tc_ld16(d_tile + m0, d);
#pragma unroll
          for (int i = 0; i < 16; ++i) acc[m0 + i] = fmaf(scale, d[i], acc[m0 + i]);
        }
        if constexpr (C::kDecoupled) {
          if constexpr (C::kSplitIssue) {
            tc_st_zero<ROWS>(d_tile);
            tc_wait_st();
          }
          tc_fence_before();
          // the tile goes to the issuers of segment n + kDRing (ring entry (r + kDRing) % R)
          mbar_arrive(d_free + 8 * ((r + C::kDRing) % R));
        } else {
          tc_fence_before();
          mbar_arrive(d_free + 8 * r);                  // the team may zero the tile for its next segment
        }
        FP6M_TRACE_EVENT(trace, 16, n);
        r += kStep;
        if (r >= R) { r -= R; rphase ^= 1; }
      }
      n_first = n_end;
      FP6M_TRACE_EVENT(trace, 20, s);
      if constexpr (C::kRowSplit) {
        finish_slice(sl, acc);
      } else if (eset == 1) {
        // set 0 has read the previous slice's sums out of the exchange buffer (barrier 2); publish (barrier 1)
        named_bar_sync(2, kEpiThreads);
#pragma unroll
        for (int m = 0; m < ROWS; ++m) sts_f32(xch + (m * kStripCols + c) * 4, acc[m]);
        named_bar_arrive(1, kEpiThreads);
      } else {
        named_bar_sync(1, kEpiThreads);
#pragma unroll
        for (int m = 0; m < ROWS; ++m) acc[m] += lds_f32(xch + (m * kStripCols + c) * 4);
        named_bar_arrive(2, kEpiThreads);
        finish_slice(sl, acc);
      }
      FP6M_TRACE_EVENT(trace, 22, s);
#pragma unroll
      for (int m = 0; m < ROWS; ++m) acc[m] = 0.f;
    }
    reduce_shared_strip(eset);
    FP6M_TRACE_EVENT(trace, 23, 0);
  }

  if (C::kReduceGroups == 8 && warp < 8) {
    // producers, issuers and the spare warps: the four warps of a group go in together, when its issuers are done
    __syncwarp();
    named_bar_sync(6 + (warp >> 2), 128);
    reduce_shared_strip(6 + (warp >> 2));
  }
  report_waits(ws, p.status);
  // ---- all roles are done with tensor memory: give it back
  tc_fence_before();
  __syncthreads();
  FP6M_TRACE_EVENT(trace, 24, 0);
#ifdef FP6M_TRACE
  if (tid == 0 && cta < 160) {
    g_launch_times[misc[1] & 63][cta][0] = t_launch;
    g_launch_times[misc[1] & 63][cta][1] = global_ns();
  }
#endif
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::kTmemCols) : "memory");
  }
}

#ifndef FP6M_TC5_TEAMS
#define FP6M_TC5_TEAMS 3
#define FP6M_TC5_STAGES 15
#endif
using Tc5Rows16 = Tc5Cfg<16, FP6M_TC5_STAGES, 2 * FP6M_TC5_TEAMS, FP6M_TC5_TEAMS, true>;          // 3 teams: 6 x 16 + 6 x 64 = 480 TMEM columns
using Tc5Rows16Ordered = Tc5Cfg<16, FP6M_TC5_STAGES, 2 * FP6M_TC5_TEAMS, FP6M_TC5_TEAMS, false>;  // one issuing thread per accumulator tile: run-to-run bit-identical
// 17 to 32 rows: three teams and six operand slots as above, four accumulator tiles of 32 TMEM columns.
// 33 to 64 rows: two teams, four operand slots and four accumulator tiles of 64 columns (with six slots only two
// tiles fit, and the chain MMA -> read-back -> next MMA on two tiles is as slow as two teams).
// The activation tiles grow with the rows, the weight stages give way.
using Tc5Rows32 = Tc5Cfg<32, 12, 6, 3, true, 4>;
using Tc5Rows32Ordered = Tc5Cfg<32, 12, 6, 3, false, 4>;
using Tc5Rows64 = Tc5Cfg<64, 10, 4, 2, true>;
using Tc5Rows64Ordered = Tc5Cfg<64, 10, 4, 2, false>;

// 65 to 128 rows: two teams, four operand slots (256 TMEM columns) beside two accumulator tiles of 128 columns;
// four epilogue sets of 32 rows each
using Tc5Rows128 = Tc5Cfg<128, 6, 4, 2, true, 2>;
using Tc5Rows128Ordered = Tc5Cfg<128, 6, 4, 2, false, 2>;

bool g_overlap_launches = false;
bool g_ordered_sums = false;

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
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.sched.ctas);
  cfg.blockDim = dim3(C::kThreads);
  cfg.dynamicSmemBytes = C::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_overlap_launches ? 1 : 0;
  alignas(64) CUtensorMap amap;
  // K a multiple of 64: one copy per segment through a {64 halves, rows, units} map; else one copy per unit
  cudaError_t me = (p.K & 63) == 0 ? encode_activation_segment_map(p.A, p.M, p.K, C::NT, &amap)
                                   : encode_activation_map(p.A, p.M, p.K, C::NT, &amap);
  if (me != cudaSuccess) return me;
  return cudaLaunchKernelEx(&cfg, w46_gemm_tc5_kernel<C>, p, amap);
}

}  // namespace

#ifdef FP6M_TRACE
extern "C" int fp6m_launch_times_read(unsigned long long* out, size_t bytes) {
  if (bytes < sizeof(g_launch_times)) return -1;
  return (int)cudaMemcpyFromSymbol(out, g_launch_times, sizeof(g_launch_times));
}
extern "C" int fp6m_trace_read(unsigned long long* out, size_t bytes) {
  if (bytes < sizeof(g_trace)) return -1;
  return (int)cudaMemcpyFromSymbol(out, g_trace, sizeof(g_trace));
}
#endif

void tc5_set_overlap(bool on) { g_overlap_launches = on; }
void tc5_set_ordered_sums(bool on) { g_ordered_sums = on; }
bool tc5_get_ordered_sums() { return g_ordered_sums; }
bool tc5_get_overlap() { return g_overlap_launches; }

// CTAs per SM the kernel is sized for, for `rows` rows of A in one pass.
int tc5_ctas_per_sm(int rows) { (void)rows; return 1; }

// rows of the MMA tile used for `rows` (<= kTc5MaxRows) rows of A
int tc5_tile_rows(int rows) { return rows <= 16 ? 16 : (rows <= 32 ? 32 : (rows <= 64 ? 64 : 128)); }

size_t tc5_scratch_bytes(int ctas, int rows) {
  return kEpochWords * sizeof(unsigned int) + (size_t)2 * ctas * tc5_tile_rows(rows) * kStripCols * sizeof(unsigned long long);
}

// Runs the GEMM for rows [0, p.M) with p.M <= kTc5MaxRows.  The schedule's unit boundaries must be even (whole blocks).
cudaError_t launch_gemm_tc5(const MulParams& p, cudaStream_t stream) {
  switch (tc5_tile_rows(p.M)) {
    case 16: return g_ordered_sums ? launch_tc5<Tc5Rows16Ordered>(p, stream) : launch_tc5<Tc5Rows16>(p, stream);
    case 32: return g_ordered_sums ? launch_tc5<Tc5Rows32Ordered>(p, stream) : launch_tc5<Tc5Rows32>(p, stream);
    case 64: return g_ordered_sums ? launch_tc5<Tc5Rows64Ordered>(p, stream) : launch_tc5<Tc5Rows64>(p, stream);
    default: return g_ordered_sums ? launch_tc5<Tc5Rows128Ordered>(p, stream) : launch_tc5<Tc5Rows128>(p, stream);
  }
}

}  // namespace fp6m
