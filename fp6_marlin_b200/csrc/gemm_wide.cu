// W(4&6)A16 GEMM on tcgen05 + TMEM for 129 to 256 rows of A per pass (up to 128 rows: gemm_tc5.cu).
//
// As in the kernel for up to 128 rows (gemm_tc5.cu) the product is computed transposed: the 128 weight
// columns of a strip are the M dimension of tcgen05.mma (one TMEM lane per column), the rows of A its
// N dimension (128 or 256), the dequantised weights the A operand in TENSOR MEMORY.  Differences:
//   * The INT4 group scale is multiplied into the operand - fp16(q - 8) * s_g with one fp16 rounding,
//     bit for bit the dequantised weight of the reference's rule (test.py:98) - so ONE accumulator
//     tile collects a whole slice of K and is read back once per slice, not once per scale group.
//     Per-channel INT4 scales and FP6 scales (times 4096) are applied to the fp32 sums, as before.
//   * The activations come by tiled TMA: one copy per 64-row unit brings NT rows x 64 halves (128-byte
//     rows, 128-byte swizzle) - the K-major swizzled operand layout of tcgen05 with 1024 bytes between
//     8-row groups; a K step of 16 advances the descriptor by 32 bytes.  Rows beyond M are zero-filled
//     by the copy engine.
//   * 256-row tiles have one MMA issuer.  Narrower tiles, whose MMAs are shorter than the ~100 cycles
//     one thread needs to issue one, have 2 or 4 issuers: issuer i takes the segments n = i, i + I, ...
//     into its own accumulator tile and the tiles are added, in issuer order, when a slice is written
//     out - the summation order is fixed either way.
// One CTA per SM: warp 0 weights producer, warp 1 activations producer, warps 2.. MMA issuers (warp 2
// owns TMEM, the last one reads the launch epoch), then four dequantiser warps per team; teams take the
// segments in turn.
// Split-K between CTAs uses the tagged slots of gemm_tc5.cu (the strip's last contributor reduces).
//
// Replaces the reference's large-tile path (thread_m_blocks 2..4 and its `parallel` batches,
// fp6_marlin/fp6_marlin_cuda_kernel.cu:864-951).
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "device_utils.cuh"
#include "fp6m_layout.h"
#include "gemm_params.h"
#include "tc5_common.cuh"

namespace fp6m {

namespace {

template <int NT_, int TEAMS_, int ISSUERS_, int STAGES_, int ACT_STAGES_, int RING_>
struct WideCfg {
  static constexpr int kIssuers = ISSUERS_;            // MMA issuers = accumulator tiles
  static constexpr int NT = NT_;                       // rows of A per pass = N of the MMA
  static constexpr int kTeams = TEAMS_;
  static constexpr int kStages = STAGES_;              // weight stages (one segment = up to two units each)
  static constexpr int kActStages = ACT_STAGES_;       // activation stages (one unit each)
  static constexpr int kRing = RING_;                  // TMEM operand slots (one segment each)
  static constexpr int kDeqBase = (2 + kIssuers + 3) & ~3;
  static constexpr int kThreads = 32 * (kDeqBase + 4 * kTeams);
  static constexpr int kDequantThreads = 128 * kTeams;
  static constexpr int kActUnitBytes = NT * 128;       // NT rows x 64 halves, 1024-byte aligned stages
  static constexpr int kNumBars = 2 * kStages + 2 * kActStages + 2 * kRing + 3;
  static constexpr int kOutStageBytes = 2 * 16 * kStripCols * 2;  // per team: two buffers of 16 finished rows of a strip in fp16
  static constexpr int kSmemBytes = kStages * kStageW + kActStages * kActUnitBytes + kTeams * kOutStageBytes + kNumBars * 8 + 64 + 1024;
  static constexpr int kTmemD = 0, kTmemA = kIssuers * NT;   // the accumulator tiles, then operand slots of 64 columns
  static constexpr int kTmemUsed = kTmemA + kRing * 64;
  static constexpr int kTmemCols = kTmemUsed <= 128 ? 128 : (kTmemUsed <= 256 ? 256 : 512);
  static constexpr int kSlotWords = NT * kStripCols;
  static constexpr int kRowsPerTeam = NT / kTeams;     // rows of the accumulator tile a team writes out
  static constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  static constexpr int kChunk = kRowsPerTeam < 16 ? kRowsPerTeam : 16;   // rows read back per tcgen05.ld
  static_assert(kTmemUsed <= 512 && (kRowsPerTeam % 16 == 0 || kRowsPerTeam == 8) && kStages >= kTeams && kRing % kTeams == 0, "configuration");
};

// coordinates {k0, row0}: k0 is a multiple of 64 halves = 128 bytes, so the copy starts on a 16-byte boundary
__device__ __forceinline__ void tma_load_act_rows(uint32_t dst, const CUtensorMap* map, int k0, int row0, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(k0), "r"(row0), "r"(bar) : "memory");
}

// Tensor maps of the outputs (C, or every rank's full-width output) for the asynchronous row stores; box = 128
// columns x 16 rows.  Only read when p.vec_rows == 2.
struct OutMaps {
  CUtensorMap m[8];
};

// 16 rows x 128 columns of fp16 from shared memory (row-major, 256 bytes per row) to the output behind `map` at
// column x (a multiple of 8), row y; rows beyond the output's last row are clipped by the copy engine.
__device__ __forceinline__ void tma_store_rows(const CUtensorMap* map, uint32_t src_smem, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(map), "r"(x), "r"(y), "r"(src_smem) : "memory");
}

template <class C>
__global__ void __launch_bounds__(C::kThreads, 1)
w46_gemm_wide_kernel(const __grid_constant__ MulParams p, const __grid_constant__ CUtensorMap amap, const __grid_constant__ OutMaps omaps) {
  constexpr int NT = C::NT, S = C::kStages, RA = C::kActStages, R = C::kRing, T = C::kTeams;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* act_base = smem + S * kStageW;
  uint8_t* out_stage = act_base + RA * C::kActUnitBytes;            // [team][16 rows][128 columns] fp16
  uint64_t* bars = reinterpret_cast<uint64_t*>(out_stage + T * C::kOutStageBytes);
  uint32_t* misc = reinterpret_cast<uint32_t*>(bars + C::kNumBars);   // [0] TMEM base, [1] launch epoch
  const uint32_t w_full = smem_u32(bars), w_empty = w_full + 8 * S;
  const uint32_t a_full = w_empty + 8 * S, a_empty = a_full + 8 * RA;
  const uint32_t ready = a_empty + 8 * RA, slot_free = ready + 8 * R;
  const uint32_t slice_done = slot_free + 8 * R, d_read = slice_done + 8, epoch_bar = d_read + 8;

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
    for (int s = 0; s < RA; ++s) {
      mbar_init(a_full + 8 * s, 1);      // the expect_tx arrival of the activations producer
      mbar_init(a_empty + 8 * s, 1);     // tcgen05.commit: the MMAs that read the stage have finished
    }
    for (int r = 0; r < R; ++r) {
      mbar_init(ready + 8 * r, 4);       // the segment's team stored the operands into TMEM
      mbar_init(slot_free + 8 * r, 1);   // tcgen05.commit: the MMAs that read the slot have finished
    }
    mbar_init(slice_done, C::kIssuers);  // tcgen05.commit of every issuer: the accumulator tiles hold the whole slice
    mbar_init(d_read, 4 * T);            // every dequantiser warp has read its part of the tile back
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

  if (warp == 0) {
    // ================================================================== weights producer
    if (lane == 0) {
      const uint64_t policy = make_evict_first_policy();
      Walk it;
      it.init(U0, U1, ups);
      bool new_strip = true;
      const int nstrips = geo.strips4 + geo.strips6;
      int strip_lin = (U0 / ups) % nstrips;            // the strip of the virtual strip (row tile x strip)
      const uint8_t* wsrc = nullptr;
      uint32_t unit_bytes = 0;
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
        if (phase == 1 && stage == 0) grid_dependency_wait();   // the first S copies need nobody; from here on the teams must have made room
        mbar_wait_bounded<200>(w_empty + 8 * stage, phase ^ 1, p.status, dead);
        mbar_arrive_expect_tx(w_full + 8 * stage, bytes);
        tma_load_1d_stream(smem_u32(smem) + stage * kStageW, wsrc, bytes, w_full + 8 * stage, policy);
        wsrc += bytes;
        if (++stage == S) { stage = 0; phase ^= 1; }
        new_strip = it.next(cnt);
        strip_lin += new_strip;
        if (strip_lin == nstrips) strip_lin = 0;
      }
    }
  } else if (warp == 1) {
    // ================================================================== activations producer
    if (lane == 0) {
      Walk it;
      it.init(U0, U1, ups);
      int sa = 0;
      uint32_t aphase = 0;
      const int nstrips = geo.strips4 + geo.strips6;
      int vstrip = U0 / ups;
      grid_dependency_wait();                           // A may come from the previous kernel
      while (it.valid()) {
        const int cnt = it.count();
        const int tile_row0 = (vstrip / nstrips) * NT;
        for (int h = 0; h < cnt; ++h) {
          mbar_wait_bounded<100>(a_empty + 8 * sa, aphase ^ 1, p.status, dead);
          mbar_arrive_expect_tx(a_full + 8 * sa, C::kActUnitBytes);
          tma_load_act_rows(smem_u32(act_base) + sa * C::kActUnitBytes, &amap, (it.unit + h) * kUnitRows, tile_row0, a_full + 8 * sa);
          if (++sa == RA) { sa = 0; aphase ^= 1; }
        }
        vstrip += it.next(cnt);
      }
    }
  } else if (warp >= 2 && warp < 2 + C::kIssuers) {
    // ================================================================== MMA issuers
    // The whole warp walks the segments and waits; one fixed lane issues, so the commits track its MMAs.
    constexpr int I = C::kIssuers;
    const int mine = warp - 2;
    // every bounded wait below depends on the activations, which the previous kernel of the stream may still be
    // writing: start them only when it has completed
    grid_dependency_wait();
    if (mine == I - 1 && lane == 0) {
      // the tag of this launch's split-K partials is epoch + 1
      const uint32_t e = read_epoch_and_count(p.epochs, gridDim.x);
      misc[1] = e;
      mbar_arrive(epoch_bar);
    }
    __syncwarp();
    Walk it;
    it.init(U0, U1, ups);
    int r = 0, sa = 0, slices = 0, turn = 0;
    uint32_t rphase = 0, aphase = 0;
    bool first = true;                                // my next MMA is my first of the slice: it overwrites my tile
    constexpr uint32_t kStepDesc = 32 >> 4;            // 16 halves along a 128-byte row
    const uint64_t desc0 = wide_act_desc(smem_u32(act_base));
    const uint32_t d_tmem = tmem + C::kTmemD + mine * NT;
    while (it.valid()) {
      const int cnt = it.count();
      const bool my_turn = I == 1 || turn == mine;
      if (my_turn) {
        mbar_wait_bounded<40>(ready + 8 * r, rphase, p.status, dead);
        if (first && slices > 0) mbar_wait_bounded<40>(d_read, (slices - 1) & 1, p.status, dead);   // previous slice was read back
      }
      const uint32_t a_tmem = tmem + C::kTmemA + r * 64;
      for (int h = 0; h < cnt; ++h) {
        if (my_turn) {
          mbar_wait_bounded<40>(a_full + 8 * sa, aphase, p.status, dead);
          tc_fence_after();
          // the descriptor's low 14 bits hold the address / 16: adding an offset never carries out of them
          const uint64_t desc = desc0 + (uint64_t)(sa * (C::kActUnitBytes >> 4));
          if (lane == 0) {
            tc_mma_unit<kStepDesc>(d_tmem, a_tmem + h * 32, desc, C::kIdesc, first ? 0u : 1u);
            tc_commit(a_empty + 8 * sa);                  // the stage may be refilled when these MMAs are done
          }
          __syncwarp();
          first = false;
        }
        if (++sa == RA) { sa = 0; aphase ^= 1; }
      }
      const bool slice_ends = it.next(cnt) || !it.valid();
      // An issuer without work in a slice runs ahead; its arrival for slice k must not be counted
      // towards slice k - 1, so it first sees that phase complete.
      if (slice_ends && I > 1 && slices > 0) mbar_wait_bounded<40>(slice_done, (slices - 1) & 1, p.status, dead);
      if (lane == 0) {
        if (my_turn) tc_commit(slot_free + 8 * r);
        if (slice_ends) tc_commit(slice_done);          // completes when all my MMAs so far have finished
      }
      __syncwarp();
      if (slice_ends) { first = true; ++slices; }
      if (++turn == I) turn = 0;
      if (++r == R) { r = 0; rphase ^= 1; }
    }
  } else if (warp >= C::kDeqBase) {
    // ================================================================== dequantisers (warps kDeqBase..)
    // thread = weight column = TMEM lane; team t expands the segments n = t, t + T, ... of the CTA
    // and writes out rows [t NT/T, (t+1) NT/T) of every slice's accumulator tile
    constexpr int RPT = C::kRowsPerTeam, CH = C::kChunk;
    auto tc_ld_chunk = [](uint32_t taddr, float (&v)[CH]) {
      if constexpr (CH == 8) tc_ld8(taddr, v); else tc_ld16(taddr, v);
    };
    const int team = (warp - C::kDeqBase) >> 2;
    const int quarter = warp & 3;                    // the TMEM lanes this warp may touch
    const int c = quarter * 32 + lane;               // weight column inside the strip
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    grid_dependency_wait();                          // the waits below depend, through the MMAs, on the previous kernel's output
    const uint32_t a_base = lane_base + C::kTmemA;
    const uint32_t d_base = lane_base + C::kTmemD + team * RPT;
    const uint32_t lds_lo = c * 32 + 16 * ((c >> 2) & 1);          // words 0..3 of the column; words 4..7 at ^ 16
    const int strip_first = U0 / ups;
    const int row0 = team * RPT;

    struct Slice {
      int strip_lin, strip, nq, u0, u1, s_begin, tile_row0;   // strip_lin: the VIRTUAL strip (row tile x strip)
      bool is6, group;
    };
    auto open_slice = [&](int strip_lin, int u) {
      Slice sl;
      const int nstrips = geo.strips4 + geo.strips6;
      const int real = strip_lin % nstrips;
      sl.strip_lin = strip_lin;
      sl.tile_row0 = (strip_lin / nstrips) * NT;
      sl.is6 = real >= geo.strips4;
      sl.strip = sl.is6 ? real - geo.strips4 : real;
      sl.nq = strip_quads(sl.is6 ? geo.n6 : geo.n4, sl.strip);
      sl.group = !sl.is6 && geo.groups > 1;
      sl.s_begin = strip_lin * ups;
      sl.u0 = u;
      sl.u1 = min(U1, sl.s_begin + ups);
      return sl;
    };
    auto column_scale = [&](const Slice& sl, bool writes) {
      float col_scale = 1.f;      // per-channel INT4: s; FP6: s * 4096; group INT4: already in the operands
      if (writes && !sl.group) {
        const half* sp = p.S + (sl.is6 ? fp6_scale_offset(geo, sl.strip) : int4_scale_offset(geo, sl.strip, 0));
        col_scale = __half2float(__ldg(sp + c)) * (sl.is6 ? 4096.f : 1.f);
      }
      return col_scale;
    };
    auto slot_of = [&](int cc, int strip_lin) {
      // slot 0 holds the partial of a CTA's first strip, slot 1 that of its last strip
      const int cc_first = p.sched.bound[cc] / ups;
      return p.partials + (size_t)(2 * cc + (strip_lin != cc_first ? 1 : 0)) * C::kSlotWords + row0 * kStripCols + c;
    };
    // CH finished rows of this thread's column.  Plain path: one 2-byte store per value (a warp writes 64
    // bytes of a row).  With p.vec_rows the team turns the CH x 128 block round through shared memory and
    // every thread stores 16 bytes of a row - to C, or to every rank's output over NVLink, where the size of
    // a write matters most.  All 128 threads of the team call this together.
    const uint32_t my_stage = smem_u32(out_stage) + team * C::kOutStageBytes;
    const int team_tid = (warp - C::kDeqBase - 4 * team) * 32 + lane;
    int stage_turn = 0;                                // which of the team's two buffers the next block of rows uses
    auto store_rows = [&](const Slice& sl, int m0, const float (&v)[CH], float col_scale, bool writes) {
      float out[CH];
#pragma unroll
      for (int i = 0; i < CH; ++i) out[i] = v[i] * col_scale;
      if (!p.vec_rows || CH != 16) {
        store_column_rows<CH>(p, sl.tile_row0 + row0 + m0, sl.is6, sl.strip * kStripCols + c, out, writes);
        return;
      }
      const uint32_t buf = my_stage + (uint32_t)(stage_turn & 1) * (16 * kStripCols * 2);
      ++stage_turn;
      // the copy engine has read the rows this buffer held two blocks ago (only team thread 0 issues copies)
      if (team_tid == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      named_bar_sync(1 + team, 128);
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const unsigned short hbits = __half_as_ushort(__float2half_rn(out[i]));
        asm volatile("st.shared.u16 [%0], %1;" ::"r"(buf + (uint32_t)(i * kStripCols + c) * 2), "h"(hbits) : "memory");
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // the copy engine reads what this thread wrote
      named_bar_sync(1 + team, 128);
      const int ncols = strip_cols(sl.is6 ? geo.n6 : geo.n4, sl.strip);
      const int row_first = sl.tile_row0 + row0 + m0;
      if (row_first >= p.M) return;                    // uniform over the team
      const int col_strip = (p.out.n_out == 0 ? (sl.is6 ? geo.n4 : 0) : (sl.is6 ? p.out.col6 : p.out.col4)) + sl.strip * kStripCols;
      if (p.vec_rows == 2 && ncols == kStripCols) {
        // a full strip: one asynchronous tensor store per output; the team goes on at once
        if (team_tid == 0) {
          const int n_maps = p.out.n_out == 0 ? 1 : p.out.n_out;
#pragma unroll 1
          for (int q = 0; q < n_maps; ++q) tma_store_rows(&omaps.m[q], buf, col_strip, row_first);
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        return;
      }
      const int g = team_tid & 15;                     // eight columns of the strip
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const int i = (team_tid >> 4) + 8 * rr;
        const int row = row_first + i;
        if (row < p.M && g * 8 < ncols) {
          uint4 val;
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                       : "r"(buf + (uint32_t)(i * kStripCols + g * 8) * 2));
          if (p.out.n_out == 0) {
            *reinterpret_cast<uint4*>(p.C + (size_t)row * p.N + col_strip + g * 8) = val;
          } else {
            const size_t at = (size_t)row * p.out.ld + col_strip + g * 8;
#pragma unroll 1
            for (int q = 0; q < p.out.n_out; ++q) *reinterpret_cast<uint4*>(p.out.peer[q] + at) = val;
          }
        }
      }
      // (the buffer is not written again before the barrier at the top of the block after next)
    };
    // before the team leaves: its asynchronous stores have been performed
    auto drain_stores = [&]() {
      if (team_tid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    };

    int reduce_strip = -1;                           // strip this CTA must reduce at its end
    uint32_t reduce_tag = 0;
    int n = team, stage = team, r = team;            // this team's next segment, its weight stage and operand slot
    uint32_t wphase = 0, rphase = 0;
    int n0 = 0, slices = 0;
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
      const half* sp0 = p.S + (sl.group ? int4_scale_offset(geo, sl.strip, 0) + c : 0);
      const bool scaled = sl.group && col_live;
      half next_scale = __float2half(1.f);
      if (scaled && n - n0 < nseg) next_scale = __ldg(sp0 + (size_t)(b0 + n - n0) * scale_stride);

      for (int j = n - n0; j < nseg; j += T) {
        const int b = b0 + j;
        const int cnt = min(unit1, 2 * b + 2) - max(unit0, 2 * b);
        const half2 s2 = __half2half2(next_scale);
        if (scaled && j + T < nseg) next_scale = __ldg(sp0 + (size_t)(b + T) * scale_stride);   // used one iteration later
        mbar_wait_bounded(w_full + 8 * stage, wphase, p.status, dead);
        const uint8_t* st = smem + stage * kStageW;
        // the MMAs that read this operand slot R segments ago have finished
        mbar_wait_bounded(slot_free + 8 * r, rphase ^ 1, p.status, dead);
        tc_fence_after();
        const uint32_t a_tmem = a_base + r * 64;
#pragma unroll 1
        for (int h = 0; h < cnt; ++h) {
          // Columns of padded quads read stale bytes of the stage and produce values nobody stores.
          const uint8_t* su = st + h * unit_bytes;
          const uint4 lo = *reinterpret_cast<const uint4*>(su + lds_lo);          // words 0..3
          const uint4 hi = *reinterpret_cast<const uint4*>(su + (lds_lo ^ 16));   // words 4..7
          uint4 two = make_uint4(0, 0, 0, 0);
          if (is6) two = *reinterpret_cast<const uint4*>(su + two_off);
          const uint32_t words[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
          const uint32_t twos[4] = {two.x, two.y, two.z, two.w};
#pragma unroll
          for (int step = 0; step < 4; ++step) {
            uint32_t regs[8];
            if (is6) {
              expand_fp6(words[2 * step], twos[step], 0, regs);
              expand_fp6(words[2 * step + 1], twos[step], 4, regs + 4);
            } else if (sl.group) {
              expand_int4_scaled(words[2 * step], s2, regs);
              expand_int4_scaled(words[2 * step + 1], s2, regs + 4);
            } else {
              expand_int4(words[2 * step], regs);
              expand_int4(words[2 * step + 1], regs + 4);
            }
            tc_st8(a_tmem + h * 32 + step * 8, regs);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(w_empty + 8 * stage);          // the stage's words are in registers
        tc_wait_st();
        tc_fence_before();
        if (lane == 0) mbar_arrive(ready + 8 * r);
        n += T;
        stage += T;
        if (stage >= S) { stage -= S; wphase ^= 1; }
        r += T;
        if (r >= R) { r -= R; rphase ^= 1; }
      }
      const int n0_slice = n0;
      n0 += nseg;
      u = sl.u1;

      // ---------------- the slice is in the accumulator tile: write C, or store a tagged partial
      mbar_wait_bounded(slice_done, slices & 1, p.status, dead);
      tc_fence_after();
      grid_dependency_wait();                        // C and the scratch may still be in use by the previous kernel
      const bool whole = sl.u0 == sl.s_begin && sl.u1 == sl.s_begin + ups;
      const bool writes = c < strip_cols(is6 ? geo.n6 : geo.n4, sl.strip);
      const float col_scale = whole ? column_scale(sl, writes) : 1.f;
      uint32_t tag = 0;
      unsigned long long* slot = nullptr;
      if (!whole) {
        mbar_wait_bounded(epoch_bar, 0, p.status, dead);   // completed long ago: orders the read of misc[1]
        tag = misc[1] + 1;
        slot = slot_of(cta, sl.strip_lin);
      }
#pragma unroll 1
      for (int m0 = 0; m0 < RPT; m0 += CH) {
        // add the issuers' tiles in issuer order; issuer i took the slice's segments j with
        // (n0_slice + j) % I == i - one that had none keeps a stale tile, which is skipped
        float v[CH];
#pragma unroll
        for (int q = 0; q < CH; ++q) v[q] = 0.f;
#pragma unroll
        for (int i = 0; i < C::kIssuers; ++i) {
          const int first_j = (i - n0_slice % C::kIssuers + C::kIssuers) % C::kIssuers;
          if (first_j < nseg) {
            float t[CH];
            tc_ld_chunk(d_base + i * NT + m0, t);
#pragma unroll
            for (int q = 0; q < CH; ++q) v[q] += t[q];
          }
        }
        if (whole) {
          store_rows(sl, m0, v, col_scale, writes);
        } else {
#pragma unroll
          for (int i = 0; i < CH; ++i)
            st_relaxed_u64(slot + (m0 + i) * kStripCols, ((unsigned long long)tag << 32) | __float_as_uint(v[i]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(d_read);            // the MMA issuer may start the next slice in the tile
      if (!whole && sl.u1 == sl.s_begin + ups) {     // last contributor of the strip: reduce it at the end
        reduce_strip = sl.strip_lin;
        reduce_tag = tag;
      }
      ++slices;
      ++strip_lin;
    }

    // ---------------- after the last slice: reduce the strip whose last contributor this CTA is, by
    // reading the tagged slots of the lower-numbered contributors (bounded spin) in CTA order
    if (reduce_strip >= 0) {
      const Slice sl = open_slice(reduce_strip, 0);
      int c_lo = cta;
      while (c_lo > 0 && p.sched.bound[c_lo] > sl.s_begin) --c_lo;
      const bool writes = c < strip_cols(sl.is6 ? geo.n6 : geo.n4, sl.strip);
      const float col_scale = column_scale(sl, writes);
#pragma unroll 1
      for (int m0 = 0; m0 < RPT; m0 += CH) {
        float sum[CH];
#pragma unroll
        for (int i = 0; i < CH; ++i) sum[i] = 0.f;
        // two contributors per round trip to L2 (32 tagged words in flight per thread); added in CTA order
#pragma unroll 1
        for (int cc = c_lo; cc <= cta; cc += 2) {
          // a CTA without work stored nothing; this CTA's own slot (present for sure) stands in for it
          const bool live0 = p.sched.bound[cc] < p.sched.bound[cc + 1];
          const bool live1 = cc + 1 <= cta && p.sched.bound[cc + 1] < p.sched.bound[cc + 2];
          const unsigned long long* src0 = slot_of(live0 ? cc : cta, reduce_strip) + m0 * kStripCols;
          const unsigned long long* src1 = slot_of(live1 ? cc + 1 : cta, reduce_strip) + m0 * kStripCols;
          unsigned long long v0[CH], v1[CH];
          bool all_here = false;
#pragma unroll 1
          for (int spin = 0; spin < (1 << 20) && !all_here; ++spin) {
#pragma unroll
            for (int i = 0; i < CH; ++i) v0[i] = ld_relaxed_u64(src0 + i * kStripCols);
#pragma unroll
            for (int i = 0; i < CH; ++i) v1[i] = ld_relaxed_u64(src1 + i * kStripCols);
            all_here = true;
#pragma unroll
            for (int i = 0; i < CH; ++i)
              all_here = all_here && (uint32_t)(v0[i] >> 32) == reduce_tag && (uint32_t)(v1[i] >> 32) == reduce_tag;
            if (dead) break;
          }
          if (!all_here && !dead) {
            dead = true;
            if (p.status) atomicExch(p.status, kStatusTimeout);
          }
#pragma unroll
          for (int i = 0; i < CH; ++i) {
            sum[i] += live0 ? __uint_as_float((uint32_t)v0[i]) : 0.f;
            sum[i] += live1 ? __uint_as_float((uint32_t)v1[i]) : 0.f;
          }
        }
        store_rows(sl, m0, sum, col_scale, writes);
      }
    }
    drain_stores();
  }

  // ---- all roles are done with tensor memory: give it back
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(C::kTmemCols) : "memory");
  }
}

// The number of operand slots is a multiple of the number of teams, so a slot always belongs to the same team
// and every waiter of a barrier sees each of its phases (a parity wait that skipped a phase would pass early).
using Wide256 = WideCfg<256, 2, 1, 4, 4, 4>;    // 256 + 4 x 64 = 512 TMEM columns

template <class C>
cudaError_t launch_wide(const MulParams& p_in, cudaStream_t stream, bool overlap) {
  alignas(64) CUtensorMap amap;
  cudaError_t me = encode_activation_map(p_in.A, p_in.M, p_in.K, C::NT, &amap);
  if (me != cudaSuccess) return me;
  MulParams p = p_in;
  alignas(64) OutMaps omaps = {};
  if (p.vec_rows) {
    // asynchronous tensor stores of the finished rows: one map per output; without them the 16-byte stores stay
    bool ok = true;
    if (p.out.n_out == 0) {
      ok = encode_output_map(p.C, p.M, p.N, &omaps.m[0]) == cudaSuccess;
    } else {
      for (int q = 0; q < p.out.n_out && ok; ++q) ok = encode_output_map(p.out.peer[q], p.M, p.out.ld, &omaps.m[q]) == cudaSuccess;
    }
    if (ok) p.vec_rows = 2;
  }

  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(w46_gemm_wide_kernel<C>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
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
  cfg.numAttrs = overlap ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, w46_gemm_wide_kernel<C>, p, amap, omaps);
}

}  // namespace

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver's tensor-map encoder, looked up once through the runtime (no link against libcuda).
static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult res;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &res) == cudaSuccess &&
        res == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// The last few tensor maps of the calling thread: a decode loop calls with the same activation buffer again
// and again, and encoding a map costs a driver call.  (A map depends on the pointer and the shape only.)
namespace {
struct MapKey {
  const void* A;
  int M, K, box_rows, dims;
};
struct MapCache {
  static constexpr int kEntries = 96;      // a GEMM of many launches onto eight outputs has 64 output maps
  MapKey key[kEntries] = {};
  CUtensorMap map[kEntries];
  int next = 0;
  bool find(const MapKey& k, CUtensorMap* out) const {
    for (int i = 0; i < kEntries; ++i)
      if (key[i].A == k.A && key[i].M == k.M && key[i].K == k.K && key[i].box_rows == k.box_rows && key[i].dims == k.dims) {
        *out = map[i];
        return true;
      }
    return false;
  }
  void put(const MapKey& k, const CUtensorMap& m) {
    key[next] = k;
    map[next] = m;
    next = (next + 1) % kEntries;
  }
};
thread_local MapCache g_map_cache;
}  // namespace

// A as a K x M tensor (K contiguous): one box = 64 halves x `box_rows` rows = the activations of one
// 64-row unit, written to shared memory with the 128-byte swizzle; rows beyond M read as zero.
cudaError_t encode_activation_map(const half* A, int M, int K, int box_rows, CUtensorMap* map) {
  const MapKey mk = {A, M, K, box_rows, 2};
  if (g_map_cache.find(mk, map)) return cudaSuccess;
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return cudaErrorNotSupported;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t elem[2] = {1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<half*>(A), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;
  g_map_cache.put(mk, *map);
  return cudaSuccess;
}

// An output (C, or a rank's full-width output) as an `ld` x `rows` fp16 tensor; one box = 128 columns x 16 rows,
// row-major in shared memory (no swizzle).  Stores beyond the last row are clipped.
cudaError_t encode_output_map(const half* base, int rows, int ld, CUtensorMap* map) {
  const MapKey mk = {base, rows, ld, 16, 4};
  if (g_map_cache.find(mk, map)) return cudaSuccess;
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return cudaErrorNotSupported;
  const cuuint64_t dims[2] = {(cuuint64_t)ld, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kStripCols, 16};
  const cuuint32_t elem[2] = {1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<half*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;
  g_map_cache.put(mk, *map);
  return cudaSuccess;
}

// A as a 64 x M x K/64 tensor (K a multiple of 64): one box = 64 halves x `box_rows` rows x 2 units = the
// activations of one 128-row block as two swizzled tiles, one behind the other; units beyond K and rows
// beyond M read as zero.
cudaError_t encode_activation_segment_map(const half* A, int M, int K, int box_rows, CUtensorMap* map) {
  const MapKey mk = {A, M, K, box_rows, 3};
  if (g_map_cache.find(mk, map)) return cudaSuccess;
  EncodeTiledFn encode = encode_tiled();
  if (!encode) return cudaErrorNotSupported;
  const cuuint64_t dims[3] = {64, (cuuint64_t)M, (cuuint64_t)(K / 64)};
  const cuuint64_t strides[2] = {(cuuint64_t)K * 2, 128};
  const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 2};
  const cuuint32_t elem[3] = {1, 1, 1};
  if (encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<half*>(A), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;
  g_map_cache.put(mk, *map);
  return cudaSuccess;
}

int wide_rows_per_pass() { return 256; }   // the widest tile

// rows of the MMA tile used for `rows` rows of A
int wide_tile_rows(int rows) { (void)rows; return 256; }

size_t wide_scratch_bytes(int ctas, int rows) {
  return kEpochWords * sizeof(unsigned int) + (size_t)2 * ctas * wide_tile_rows(rows) * kStripCols * sizeof(unsigned long long);
}

// Runs the GEMM for rows [0, p.M) in p.row_tiles tiles of `tile_rows` rows; the host dispatcher loops over larger M.
cudaError_t launch_gemm_wide(const MulParams& p, int tile_rows, cudaStream_t stream) {
  const bool overlap = tc5_get_overlap();
  (void)tile_rows;                     // always 256: up to 128 rows go to the kernel of gemm_tc5.cu
  return launch_wide<Wide256>(p, stream, overlap);
}

}  // namespace fp6m
