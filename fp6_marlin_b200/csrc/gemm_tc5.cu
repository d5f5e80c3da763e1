// W(4&6)A16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM) for up to 16 rows of A.
//
// The product is computed transposed, D[n, m] = sum_k W[k, n] * A[m, k]: the 128 weight columns of
// a strip are the M dimension of tcgen05.mma (one TMEM lane per weight column), the rows of A are
// its N dimension (16), and the dequantised weights are the A operand read from TENSOR MEMORY, so
// they never travel through shared memory.  Legacy mma.sync costs about 32 cycles per m16n8k16
// tile on B200 and cannot keep up with HBM (profiles/w46_gemm_mma_*); tcgen05 can.
//
// One CTA per SM, 24 warps:
//   warp 0, 6, 7  weights producers: one bulk TMA copy (cp.async.bulk, mbarrier completion) per
//               SEGMENT = the one or two 64-row units of a 128-row block that belong to the CTA;
//               a single lane needs ~500 cycles per copy, so the segments are dealt round robin.
//   warp 1      activations producer: one tiled TMA copy per unit (16 rows x 64 halves, 128-byte
//               swizzle = the K-major swizzled B operand of the MMA; rows beyond M read as zero).
//   warps 2-5   MMA issuers, one per dequantiser team: one lane issues tcgen05.mma (kind::f16, fp32
//               accumulators in TMEM) for its team's segments and commits completion to mbarriers.
//               A thread sustains one small MMA per 75-120 cycles, the tensor core one per 32.
//               Warp 2 owns the TMEM allocation; warp 5 also reads the launch epoch.
//   warps 8-23  four dequantiser TEAMS of four warps; thread = weight column = TMEM lane.  The teams
//               take the CTA's segments in turn (independent chains that hide each other's
//               latencies).  A thread reads its 32 bytes of a unit, expands the eight words in
//               registers and stores them with tcgen05.st into the segment's TMEM operand slot.  INT4
//               nibbles become the exact integers q - 8 in fp16 (OR into 1024 + q / 64 + q, then
//               subtract 1032 / 72) - bit for bit what the reference's dequant_8int4 feeds its tensor
//               cores (fp6_marlin_cuda_kernel.cu:249-286).  FP6 codes become `s 00eee mm` fp16 patterns
//               (exact value / 4096, as dequant_8fp6 builds them before its multiply by 4096,
//               :195-237).  Every segment has its own accumulator tile; after storing its next
//               segment a team reads the previous one's tile back (tcgen05.ld), multiplies by the
//               column's group scale in fp32 and adds to registers.  At the end of a slice (the CTA's
//               units of one strip) the teams pool their sums through shared memory.
// Work comes from the cost-weighted stripe schedule (fp6m_layout.h).  Strips shared by several CTAs
// are reduced without atomics or fences on the data path: partials are stored as {value, tag} 64-bit
// words, the tag being a per-launch epoch, and the strip's last contributor (in CTA order) sums the
// slots at its end - it only ever waits, with a bound, for lower-numbered CTAs.
//
// Replaces the reference's fp6_kernel_marlin (fp6_marlin/fp6_marlin_cuda_kernel.cu:288-837).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "device_utils.cuh"
#include "fp6m_layout.h"
#include "gemm_params.h"
#include "tc5_common.cuh"

namespace fp6m {

namespace {

template <int NT_, int STAGES_, int RING_, int CTAS_PER_SM_, int TEAMS_>
struct Tc5Cfg {
  // TEAMS dequantiser teams take the segments in turn (independent chains, each with its own MMA
  // issuer) and keep all NT rows in registers
  static constexpr int kTeams = TEAMS_;
  static constexpr int kIssuers = TEAMS_;
  // warp 0: weights producer, warp 1: activations producer, warps 2.. : MMA issuers, then (from a
  // multiple of four, so that warp % 4 is the TMEM lane quarter) four dequantiser warps per team
  static constexpr int kDeqBase = (2 + kIssuers + 3) & ~3;
  static constexpr int kThreads = 32 * (kDeqBase + 4 * kTeams);
  static constexpr int kDequantThreads = 128 * kTeams;
  // the helper warps left over below kDeqBase are further weights producers (one lane needs some 500
  // cycles per copy it issues); the last MMA issuer, whose first MMA comes latest, also reads the epoch
  static constexpr int kProducers = 1 + (kDeqBase - 2 - kIssuers);
  static constexpr int kEpochWarp = 2 + kIssuers - 1;
  static constexpr int NT = NT_;                       // rows of A per pass = N of the MMA
  static constexpr int kStages = STAGES_;              // shared-memory stages of packed words (one block each)
  static constexpr int kRing = RING_;                  // ring of {activation tile, TMEM operand slot, accumulator tile}
  static constexpr int kCtasPerSm = CTAS_PER_SM_;
  static constexpr int kActUnitBytes = NT * 128;       // NT rows x 64 halves
  static constexpr int kActBytes = 2 * kActUnitBytes;
  static constexpr int kNumBars = 2 * kStages + 4 * kRing + 1;
  static_assert(kStages >= kTeams && kRing >= kTeams, "every team needs a stage and a ring entry of its own");
  static constexpr int kXchBytes = kTeams * NT * 128 * 4;   // the teams pool their partial sums at the end of a slice
  static constexpr int kSmemBytes = kStages * kStageW + kRing * kActBytes + kXchBytes + kNumBars * 8 + 64 + 1024;   // + alignment slack
  static constexpr int kTmemD = 0, kTmemA = kRing * NT;  // accumulator tiles, then operand slots of 64 columns
  static constexpr int kTmemUsed = kTmemA + kRing * 64;
  static constexpr int kTmemCols = kTmemUsed <= 128 ? 128 : (kTmemUsed <= 256 ? 256 : 512);
  static constexpr int kSlotFloats = NT * kStripCols;
  static constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
};

template <class C>
__global__ void __launch_bounds__(C::kThreads, C::kCtasPerSm) w46_gemm_tc5_kernel(const __grid_constant__ MulParams p, const __grid_constant__ CUtensorMap amap) {
  constexpr int NT = C::NT, S = C::kStages, R = C::kRing;
  constexpr int kDequantThreads = C::kDequantThreads;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // the swizzled activation stages must start on 1024-byte boundaries
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* act_base = smem + S * kStageW;
  float* xch = reinterpret_cast<float*>(smem + S * kStageW + R * C::kActBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * kStageW + R * C::kActBytes + C::kXchBytes);
  uint32_t* misc = reinterpret_cast<uint32_t*>(bars + C::kNumBars);   // [0] TMEM base, [1] flag
  const uint32_t w_full = smem_u32(bars), w_empty = w_full + 8 * S;
  const uint32_t act_full = w_empty + 8 * S, ready = act_full + 8 * R, done = ready + 8 * R;
  const uint32_t d_free = done + 8 * R;    // the accumulator tile has been read back
  const uint32_t epoch_bar = smem_u32(bars + C::kNumBars - 1);   // misc[1] holds the launch epoch

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x;
  const Geometry& geo = p.geo;
  const int ups = units_per_strip(geo);
  const int U0 = p.sched.bound[cta], U1 = p.sched.bound[cta + 1];
  launch_dependents();
  if (U0 >= U1) {                      // no work: still counted, see read_epoch_and_count
    if (tid == 0) {
      grid_dependency_wait();
      read_epoch_and_count(p.epochs, gridDim.x);
    }
    return;
  }

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(w_full + 8 * s, 1);      // the expect_tx arrival of the weights producer
      mbar_init(w_empty + 8 * s, 4);     // the team that read the stage has its words in registers
    }
    for (int r = 0; r < R; ++r) {
      mbar_init(act_full + 8 * r, 1);    // the expect_tx arrival of the activations producer
      mbar_init(ready + 8 * r, 4);       // the segment's team stored the operands into TMEM
      mbar_init(d_free + 8 * r, 4);          // the team that owns the segment has read the accumulator tile back
      mbar_init(done + 8 * r, 1);        // tcgen05.commit: every MMA of the segment has finished
    }
    mbar_init(epoch_bar, 1);
    mbar_fence_init();
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(misc)), "r"(C::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = misc[0];
  bool dead = false;

  if (warp == C::kEpochWarp && lane == 0) {
    // the tag of this launch's split-K partials is epoch + 1
    grid_dependency_wait();
    const uint32_t e = read_epoch_and_count(p.epochs, gridDim.x);
    misc[1] = e;
    mbar_arrive(epoch_bar);
  }

  if (warp == 0 || (warp >= 2 + C::kIssuers && warp < C::kDeqBase)) {
    // ================================================================== weights producer(s)
    // producer q of P copies the segments n = q, q + P, ... (each into stage n % S)
    if (lane == 0) {
      constexpr int P = C::kProducers;
      const int mine = warp == 0 ? 0 : warp - (2 + C::kIssuers) + 1;
      int turn = 0;
      const uint64_t policy = make_evict_first_policy();
      Walk it;
      it.init(U0, U1, ups);
      bool new_strip = true;
      int strip_lin = U0 / ups;
      const uint8_t* wsrc = nullptr;
      uint32_t unit_bytes = 0;
      uint32_t dst = smem_u32(smem), full = w_full, empty = w_empty;
      int stage = 0;
      uint32_t phase = 0;
      while (it.valid()) {
        if (new_strip) {
          if (strip_lin < geo.strips4) {
            unit_bytes = strip_quads(geo.n4, strip_lin) * kInt4UnitQuadBytes;
            wsrc = p.B + int4_unit_offset(geo, strip_lin, 0) + (size_t)it.unit * unit_bytes;
          } else {
            unit_bytes = strip_quads(geo.n6, strip_lin - geo.strips4) * kFp6UnitQuadBytes;
            wsrc = p.B + fp6_unit_offset(geo, strip_lin - geo.strips4, 0) + (size_t)it.unit * unit_bytes;
          }
        }
        const int cnt = it.count();
        const uint32_t bytes = cnt * unit_bytes;            // consecutive units are contiguous in HBM
        if (P == 1 || turn == mine) {
          mbar_wait_bounded<200>(empty, phase ^ 1, p.status, dead);
          mbar_arrive_expect_tx(full, bytes);
          tma_load_1d_stream(dst, wsrc, bytes, full, policy);
        }
        if (++turn == P) turn = 0;
        wsrc += bytes;
        dst += kStageW; full += 8; empty += 8;
        if (++stage == S) { stage = 0; phase ^= 1; dst = smem_u32(smem); full = w_full; empty = w_empty; }
        new_strip = it.next(cnt);
        strip_lin += new_strip;
      }
    }
  } else if (warp == 1) {
    // ================================================================== activations producer
    if (lane == 0) {
      Walk it;
      it.init(U0, U1, ups);
      int r = 0;
      uint32_t rphase = 0;
      grid_dependency_wait();                           // A may come from the previous kernel
      while (it.valid()) {
        const int cnt = it.count();
        mbar_wait_bounded<200>(done + 8 * r, rphase ^ 1, p.status, dead);     // the MMAs that read this tile are done
        mbar_arrive_expect_tx(act_full + 8 * r, cnt * C::kActUnitBytes);
        const uint32_t dst = smem_u32(act_base) + r * C::kActBytes;
        for (int h = 0; h < cnt; ++h)
          tma_load_act(dst + h * C::kActUnitBytes, &amap, (it.unit + h) * kUnitRows, act_full + 8 * r);
        if (++r == R) { r = 0; rphase ^= 1; }
        it.next(cnt);
      }
    }
  } else if (warp >= 2 && warp < 2 + C::kIssuers) {
    // ================================================================== MMA issuer(s)
    // The whole warp walks the segments and waits (warp-uniform control flow and operands); one
    // fixed lane issues the tcgen05 instructions, so that the commit tracks the MMAs before it.
    // A single thread sustains about one small MMA per 75-120 cycles, the tensor core one per 32:
    // with alternating teams each team has its own issuer (warp 1: even segments, warp 3: odd).
    {
      constexpr int kIssuers = C::kIssuers;
      const int mine = warp - 2;
      Walk it;
      it.init(U0, U1, ups);
      int r = 0, n = 0;
      uint32_t rphase = 0;
      const uint64_t desc0 = wide_act_desc(smem_u32(act_base));
      constexpr uint32_t kStepDesc = 32 >> 4;            // 16 halves along a 128-byte row
      while (it.valid()) {
        const int cnt = it.count();
        if (kIssuers == 1 || n == mine) {
          mbar_wait_bounded<40>(act_full + 8 * r, rphase, p.status, dead);
          mbar_wait_bounded<40>(ready + 8 * r, rphase, p.status, dead);
          mbar_wait_bounded(d_free + 8 * r, rphase ^ 1, p.status, dead);   // previous tile of this entry was read
          tc_fence_after();
          const uint32_t d_tmem = tmem + C::kTmemD + r * NT;
          const uint32_t a_tmem = tmem + C::kTmemA + r * 64;
          // the descriptor's low 14 bits hold the address / 16: adding an offset never carries out of them
          const uint64_t desc = desc0 + (uint64_t)(r * (C::kActBytes >> 4));
          if (lane == 0) {
            tc_mma_unit<kStepDesc>(d_tmem, a_tmem, desc, C::kIdesc, 0u);
            if (cnt == 2) tc_mma_unit<kStepDesc>(d_tmem, a_tmem + 32, desc + (C::kActUnitBytes >> 4), C::kIdesc, 1u);
            tc_commit(done + 8 * r);
          }
          __syncwarp();
        }
        if (++n == kIssuers) n = 0;
        if (++r == R) { r = 0; rphase ^= 1; }
        it.next(cnt);
      }
    }
  } else if (warp >= C::kDeqBase) {
    // ================================================================== dequantisers (warps 4..11)
    // Two teams of four warps; thread = weight column = TMEM lane.  A thread owns half of the rows of
    // A (rows [team NT/2, (team+1) NT/2)) when a slice is written out.
    constexpr int HN = NT / C::kTeams;                // rows of A that a thread writes out
    const int team = (warp - C::kDeqBase) >> 2;
    const int quarter = warp & 3;                    // the TMEM lanes this warp may touch
    const int c = quarter * 32 + lane;               // weight column inside the strip = TMEM lane
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const int dtid = tid - 32 * C::kDeqBase;         // index among the dequantiser threads
    const uint32_t lds_lo = c * 32 + 16 * ((c >> 2) & 1);          // words 0..3 of the column; words 4..7 at ^ 16
    const int strip_first = U0 / ups;
    const int row0 = team * HN;                      // this thread's rows of A and C

    struct Slice {
      int strip_lin, strip, nq, u0, u1, s_begin;
      bool is6, group;
    };
    auto open_slice = [&](int strip_lin, int u) {
      Slice sl;
      sl.strip_lin = strip_lin;
      sl.is6 = strip_lin >= geo.strips4;
      sl.strip = sl.is6 ? strip_lin - geo.strips4 : strip_lin;
      sl.nq = strip_quads(sl.is6 ? geo.n6 : geo.n4, sl.strip);
      sl.group = !sl.is6 && geo.groups > 1;
      sl.s_begin = strip_lin * ups;
      sl.u0 = u;
      sl.u1 = min(U1, sl.s_begin + ups);
      return sl;
    };

    // ---------------- the strip is finished for this CTA: write C, or store a partial sum
    // Split-K without atomics or fences: a partial is stored as 64-bit words {fp32 value, tag}, the
    // tag being the launch epoch + 1 (the epoch word lives in the scratch header and is advanced once
    // per launch, see read_epoch_and_count, so every launch - also a replay of a captured graph - uses
    // fresh tags and stale slots of earlier launches never match).
    // The reducer of a strip is its LAST contributor in CTA order, i.e. the CTA whose slice reaches
    // the end of the strip; that slice is the first one of the CTA, and the reduction is postponed to
    // the CTA's end (finish_cta), when the other contributors have normally finished.  It then
    // reads the slots of the lower-numbered contributors, spinning (bounded) on words whose tag has
    // not arrived, sums in CTA order (deterministic) and writes C.  Only lower-numbered CTAs are
    // waited for, and those were dispatched earlier.  Only the first and the last slice of a CTA can
    // be partial; the caller's workspace is not touched.
    int reduce_strip = -1;                           // strip this CTA must reduce at its end
    uint32_t reduce_tag = 0;
    auto column_scale = [&](const Slice& sl, bool writes) {
      float col_scale = 1.f;      // per-channel INT4: s; FP6: s * 4096; group INT4: already applied
      if (writes && !sl.group) {
        const half* sp = p.S + (sl.is6 ? fp6_scale_offset(geo, sl.strip) : int4_scale_offset(geo, sl.strip, 0));
        col_scale = __half2float(__ldg(sp + c)) * (sl.is6 ? 4096.f : 1.f);
      }
      return col_scale;
    };
    auto slot_of = [&](int cc, int strip_lin) {
      // slot 0 holds the partial of a CTA's first strip, slot 1 that of its last strip
      const int cc_first = p.sched.bound[cc] / ups;
      return p.partials + (size_t)(2 * cc + (strip_lin != cc_first ? 1 : 0)) * C::kSlotFloats + row0 * kStripCols + c;
    };
    auto finish_slice = [&](const Slice& sl, float (&out)[HN]) {
      grid_dependency_wait();                        // C and the scratch may still be in use by the previous kernel
      const int s_begin = sl.s_begin, s_end = s_begin + ups;
      if (sl.u0 == s_begin && sl.u1 == s_end) {      // the whole strip was ours
        const int ncols = strip_cols(sl.is6 ? geo.n6 : geo.n4, sl.strip);
        const bool writes = c < ncols;
        const float col_scale = column_scale(sl, writes);
        if (writes) {
#pragma unroll
          for (int m = 0; m < HN; ++m)
            if (row0 + m < p.M) store_result(p, row0 + m, sl.is6, sl.strip * kStripCols + c, out[m] * col_scale);
        }
        return;
      }
      mbar_wait_bounded(epoch_bar, 0, p.status, dead);   // completed long ago: orders the read of misc[1]
      const uint32_t tag = misc[1] + 1;
      unsigned long long* slot = slot_of(cta, sl.strip_lin);
#pragma unroll
      for (int m = 0; m < HN; ++m)
        st_relaxed_u64(slot + m * kStripCols, ((unsigned long long)tag << 32) | __float_as_uint(out[m]));
      if (sl.u1 == s_end) {                          // last contributor of the strip: reduce it at the end
        reduce_strip = sl.strip_lin;
        reduce_tag = tag;
      }
    };

    // ---------------- after the last slice: reduce the strip whose last contributor this CTA is
    auto finish_cta = [&]() {
      if (reduce_strip < 0) return;
      const Slice sl = open_slice(reduce_strip, 0);
      int c_lo = cta;
      while (c_lo > 0 && p.sched.bound[c_lo] > sl.s_begin) --c_lo;
      float sum[HN];
#pragma unroll
      for (int m = 0; m < HN; ++m) sum[m] = 0.f;
      // 16 tagged words are in flight together: kBatch contributors x kRows rows
      constexpr int kRows = HN < 16 ? HN : 16;
      constexpr int kBatch = 16 / kRows;
      for (int cbase = c_lo; cbase <= cta; cbase += kBatch) {
        bool live[kBatch];
        const unsigned long long* src[kBatch];
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
          const int cc = cbase + i;
          live[i] = cc <= cta && p.sched.bound[cc] < p.sched.bound[cc + 1];
          src[i] = slot_of(live[i] ? cc : cta, reduce_strip);
        }
#pragma unroll
        for (int m0 = 0; m0 < HN; m0 += kRows) {
          unsigned long long v[kBatch][kRows];
          bool all_here = false;
#pragma unroll 1
          for (int spin = 0; spin < (1 << 20) && !all_here; ++spin) {
#pragma unroll
            for (int i = 0; i < kBatch; ++i)
#pragma unroll
              for (int m = 0; m < kRows; ++m) v[i][m] = ld_relaxed_u64(src[i] + (m0 + m) * kStripCols);
            all_here = true;
#pragma unroll
            for (int i = 0; i < kBatch; ++i)
#pragma unroll
              for (int m = 0; m < kRows; ++m) all_here = all_here && (!live[i] || (uint32_t)(v[i][m] >> 32) == reduce_tag);
            if (dead) break;
          }
          if (!all_here && !dead) {
            dead = true;
            if (p.status) atomicExch(p.status, kStatusTimeout);
          }
#pragma unroll
          for (int i = 0; i < kBatch; ++i)
#pragma unroll
            for (int m = 0; m < kRows; ++m) sum[m0 + m] += live[i] ? __uint_as_float((uint32_t)v[i][m]) : 0.f;
        }
      }
      const int ncols = strip_cols(sl.is6 ? geo.n6 : geo.n4, sl.strip);
      const bool writes = c < ncols;
      const float col_scale = column_scale(sl, writes);
      if (writes) {
#pragma unroll
        for (int m = 0; m < HN; ++m)
          if (row0 + m < p.M) store_result(p, row0 + m, sl.is6, sl.strip * kStripCols + c, sum[m] * col_scale);
      }
    };

    // expands one unit (eight words of this thread's column, plus the two-bit part for FP6) into the
    // operand slot at a_tmem (32 TMEM columns)
    auto expand_unit = [&](bool is6, const uint4& lo, const uint4& hi, const uint4& two, uint32_t a_tmem) {
      const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
      const uint32_t twos[4] = {two.x, two.y, two.z, two.w};
#pragma unroll
      for (int step = 0; step < 4; ++step) {
        uint32_t regs[8];
        if (is6) {
          expand_fp6(words[2 * step], twos[step], 0, regs);
          expand_fp6(words[2 * step + 1], twos[step], 4, regs + 4);
        } else {
          expand_int4(words[2 * step], regs);
          expand_int4(words[2 * step + 1], regs + 4);
        }
        tc_st8(a_tmem + step * 8, regs);
      }
    };

    {
      // ---------------------------------------------------------------- the teams take alternate segments
      // Team t owns the segments with global index n = t, t + 2, ...: it expands both units, and after
      // storing segment n it reads back all NT rows of segment n - 2.  Two independent chains per CTA
      // hide each other's latencies; the partial sums of the teams are swapped through shared memory
      // at the end of a slice so that each thread finishes with its own half of the rows.
      const uint32_t d_base = lane_base + C::kTmemD;       // + r * NT
      const uint32_t a_base = lane_base + C::kTmemA;       // + r * 64
      float acc[NT];
#pragma unroll
      for (int m = 0; m < NT; ++m) acc[m] = 0.f;
      constexpr int T = C::kTeams;
      int n = team;                                  // global index of this team's next segment
      int stage = team, r = team;                    // n % S, n % R (T <= S, R)
      uint32_t wphase = 0, rphase = 0;               // (n / S) & 1, (n / R) & 1
      int n0 = 0;                                    // global index of the slice's first segment
      int strip_lin = strip_first;
      int u = U0;
      while (u < U1) {
        const Slice sl = open_slice(strip_lin, u);
        const bool is6 = sl.is6;
        const bool col_live = c < sl.nq * kQuadCols;     // padded quads of a ragged strip hold no data
        const uint32_t unit_bytes = sl.nq * (is6 ? kFp6UnitQuadBytes : kInt4UnitQuadBytes);
        const int unit0 = u - sl.s_begin, unit1 = sl.u1 - sl.s_begin;
        const int b0 = unit0 >> 1;                        // first 128-row block of the slice
        const int nseg = ((unit1 + 1) >> 1) - b0;         // one segment per block that the slice touches
        const uint32_t two_off = sl.nq * kInt4UnitQuadBytes + c * 16;
        const int scale_stride = sl.nq * kQuadCols;
        const unsigned short* sp0 = reinterpret_cast<const unsigned short*>(p.S) +
                                    (sl.group ? int4_scale_offset(geo, sl.strip, 0) + c : 0);
        bool pending = false;                            // a segment of this team is not read back yet
        int pr = 0;
        uint32_t prphase = 0;
        float pscale = 1.f;

        auto read_back = [&]() {
          mbar_wait_bounded(done + 8 * pr, prphase, p.status, dead);
          tc_fence_after();
          const uint32_t d_tmem = d_base + pr * NT;
#pragma unroll
          for (int m0 = 0; m0 < NT; m0 += 16) {
            float d[16];
            tc_ld16(d_tmem + m0, d);
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[m0 + i] = fmaf(pscale, d[i], acc[m0 + i]);
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(d_free + 8 * pr);    // the MMA issuer may overwrite the tile
          pending = false;
        };

        for (int j = n - n0; j < nseg; j += T) {
          const int b = b0 + j;
          const int cnt = min(unit1, 2 * b + 2) - max(unit0, 2 * b);
          // 1.0 unless the strip has group scales; converted only when queued, so the load's latency is hidden
          unsigned short scale_raw = 0x3C00;
          if (sl.group && col_live) scale_raw = __ldg(sp0 + (size_t)b * scale_stride);
          mbar_wait_bounded(w_full + 8 * stage, wphase, p.status, dead);
          // Columns of padded quads read stale bytes of the stage and produce values nobody stores.
          const uint8_t* st = smem + stage * kStageW;
          const uint4 lo0 = *reinterpret_cast<const uint4*>(st + lds_lo);          // words 0..3
          const uint4 hi0 = *reinterpret_cast<const uint4*>(st + (lds_lo ^ 16));   // words 4..7
          uint4 two0 = make_uint4(0, 0, 0, 0);
          if (is6) two0 = *reinterpret_cast<const uint4*>(st + two_off);
          // the MMAs that read this ring entry's operand slot R segments ago have finished
          mbar_wait_bounded(done + 8 * r, rphase ^ 1, p.status, dead);
          tc_fence_after();
          const uint32_t a_tmem = a_base + r * 64;
          expand_unit(is6, lo0, hi0, two0, a_tmem);
          if (cnt == 2) {
            const uint8_t* st1 = st + unit_bytes;
            const uint4 lo1 = *reinterpret_cast<const uint4*>(st1 + lds_lo);
            const uint4 hi1 = *reinterpret_cast<const uint4*>(st1 + (lds_lo ^ 16));
            uint4 two1 = make_uint4(0, 0, 0, 0);
            if (is6) two1 = *reinterpret_cast<const uint4*>(st1 + two_off);
            expand_unit(is6, lo1, hi1, two1, a_tmem + 32);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(w_empty + 8 * stage);          // the stage's words are in registers
          tc_wait_st();
          tc_fence_before();
          if (lane == 0) mbar_arrive(ready + 8 * r);
          if (pending) read_back();                      // this team's previous segment: its MMAs finished long ago
          pending = true;
          pr = r;
          prphase = rphase;
          pscale = __half2float(__ushort_as_half(scale_raw));
          n += T;
          stage += T;
          if (stage >= S) { stage -= S; wphase ^= 1; }
          r += T;
          if (r >= R) { r -= R; rphase ^= 1; }
        }
        if (pending) read_back();
        n0 += nseg;
        u = sl.u1;

        // pool the teams' partial sums: every thread publishes its NT rows, then sums its own HN rows
        // over the teams in team order
        float out[HN];
#pragma unroll
        for (int m = 0; m < NT; ++m) xch[(team * NT + m) * kStripCols + c] = acc[m];
        named_bar_sync(1, kDequantThreads);
#pragma unroll
        for (int i = 0; i < HN; ++i) {
          float v = 0.f;
#pragma unroll
          for (int t = 0; t < T; ++t) v += xch[(t * NT + row0 + i) * kStripCols + c];
          out[i] = v;
        }
        named_bar_sync(1, kDequantThreads);              // the buffer may be rewritten by the next slice
        finish_slice(sl, out);
#pragma unroll
        for (int m = 0; m < NT; ++m) acc[m] = 0.f;
        ++strip_lin;
      }
      finish_cta();
    }
  }

  // ---- all roles are done with tensor memory: give it back
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::kTmemCols) : "memory");
  }
}

using Tc5Rows16 = Tc5Cfg<16, 12, 6, 1, 4>;

bool g_overlap_launches = false;

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
  cudaError_t me = encode_activation_map(p.A, p.M, p.K, C::NT, &amap);
  if (me != cudaSuccess) return me;
  return cudaLaunchKernelEx(&cfg, w46_gemm_tc5_kernel<C>, p, amap);
}

}  // namespace

void tc5_set_overlap(bool on) { g_overlap_launches = on; }
bool tc5_get_overlap() { return g_overlap_launches; }

// CTAs per SM the kernel is sized for, for `rows` rows of A in one pass.
int tc5_ctas_per_sm(int rows) { (void)rows; return Tc5Rows16::kCtasPerSm; }

size_t tc5_scratch_bytes(int ctas, int rows) {
  (void)rows;
  const int nt = 16;
  return kEpochWords * sizeof(unsigned int) + (size_t)2 * ctas * nt * kStripCols * sizeof(unsigned long long);
}

// Runs the GEMM for rows [0, p.M) with p.M <= 16.
cudaError_t launch_gemm_tc5(const MulParams& p, cudaStream_t stream) { return launch_tc5<Tc5Rows16>(p, stream); }

}  // namespace fp6m
