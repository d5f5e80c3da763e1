// Device-side pieces shared by the tcgen05 GEMM kernels: programmatic-dependent-launch controls,
// tcgen05 / TMEM wrappers, gpu-scope relaxed accesses for the tagged split-K slots, the launch
// epoch, the in-register expanders and the walk over a CTA's units.
#pragma once
#ifndef FP6M_PARTIAL_STORE_MODE
#define FP6M_PARTIAL_STORE_MODE 0
#endif

#include <cuda.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "device_utils.cuh"
#include "fp6m_layout.h"

namespace fp6m {

constexpr int kStageW = 12288;          // packed words of one block: up to 2 x (4096 four-bit + 2048 two-bit)

// ---- programmatic dependent launch ---------------------------------------------------------------
// launch_dependents: the next kernel of the stream may start launching (it runs its set-up and
// prefetches weights while this one finishes).  grid_dependency_wait: returns once every kernel this
// one depends on has completed and its writes are visible; without a programmatic dependency both
// are no-ops.  Everything that earlier kernels may have written (A, C, the scratch) is only touched
// after the wait; the weights and scales are read before it.
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- tcgen05 wrappers -------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// The four MMAs of one 64-row unit, D[128 x N] (+)= A[128 x 16] (TMEM) * B[N x 16]^T (shared memory
// descriptor) for K steps 0..3: the operand slot advances by 8 TMEM columns and the descriptor by
// `step_desc` (16-byte units) per step.  `accumulate` = 0 makes the first MMA overwrite D.
template <uint32_t kStepDesc>
__device__ __forceinline__ void tc_mma_unit(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p, t;\n"
      ".reg .b32 a1, a2, a3;\n"
      ".reg .b64 d1, d2, d3;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "setp.eq.b32 t, 0, 0;\n"
      "add.u32 a1, %1, 8;\n"
      "add.u32 a2, %1, 16;\n"
      "add.u32 a3, %1, 24;\n"
      "add.u64 d1, %2, %5;\n"
      "add.u64 d2, %2, %6;\n"
      "add.u64 d3, %2, %7;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], d1, %3, t;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], d2, %3, t;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], d3, %3, t;\n"
      "}\n"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate),
        "n"(kStepDesc), "n"(2 * kStepDesc), "n"(3 * kStepDesc)
      : "memory");
}
__device__ __forceinline__ void tc_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
// zeroes kCols (a multiple of 16) TMEM columns of this warp's 32 lanes
template <int kCols>
__device__ __forceinline__ void tc_st_zero(uint32_t taddr) {
  const uint32_t z = 0;
#pragma unroll
  for (int c0 = 0; c0 < kCols; c0 += 16)
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1};"
                 ::"r"(taddr + c0), "r"(z) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr) : "memory");
  tc_wait_ld();
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
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
__device__ __forceinline__ uint32_t ld_relaxed_u32(const unsigned int* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_u32(unsigned int* p, uint32_t v) {
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
#if FP6M_PARTIAL_STORE_MODE == 1
  asm volatile("st.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
#elif FP6M_PARTIAL_STORE_MODE == 2
  asm volatile("st.global.cg.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
#else
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
#endif
}
__device__ __forceinline__ uint32_t atomic_add_relaxed_u32(unsigned int* addr, uint32_t v) {
  uint32_t old;
  asm volatile("atom.relaxed.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(addr), "r"(v) : "memory");
  return old;
}

// ---- result stores ---------------------------------------------------------------------------------
// `col` is the column inside the shard's INT4 or FP6 region; see OutputMap.
template <class Params>
__device__ __forceinline__ void store_result(const Params& p, int row, bool is6, int col, float v) {
  const half h = __float2half_rn(v);
  if (p.out.n_out == 0) {
    p.C[(size_t)row * p.N + (is6 ? p.geo.n4 : 0) + col] = h;
  } else {
    const size_t at = (size_t)row * p.out.ld + (is6 ? p.out.col6 : p.out.col4) + col;
#pragma unroll 1
    for (int q = 0; q < p.out.n_out; ++q) p.out.peer[q][at] = h;
  }
}

// Stores kRows finished values of one weight column (this thread's; neighbouring lanes hold neighbouring
// columns), rows row0 .. row0 + kRows - 1, applying the epilogue: v[i] is the fp32 sum times the column scale.
// Every lane of the warp must call it (the gate / up pairs are exchanged between lanes); `writes` says
// whether the column exists.  The epilogues extend the reference's write_result
// (fp6_marlin_cuda_kernel.cu:698-749), which only scales and stores.
template <int kRows, class Params>
__device__ __forceinline__ void store_column_rows(const Params& p, int row0, bool is6, int col, const float (&v)[kRows], bool writes) {
  if (p.epilogue == kEpilogueSiluMul) {
    const int half_n = p.N >> 1;
    const size_t out_col = (size_t)((is6 ? p.geo.n4 : 0) + col) >> 1;
#pragma unroll
    for (int i = 0; i < kRows; ++i) {
      const float up = __shfl_xor_sync(0xffffffffu, v[i], 1);          // the odd neighbour's value
      if (writes && (col & 1) == 0 && row0 + i < p.M) {
        const float g = v[i];
        p.C[(size_t)(row0 + i) * half_n + out_col] = __float2half_rn(g / (1.f + __expf(-g)) * up);
      }
    }
    return;
  }
  if (kRows % 4 == 0 && kRows >= 8 && p.vec_rows) {
    // Four neighbouring lanes turn their 4 x kRows block round with shuffles: lane q of the quad ends up
    // with the rows q * kRows / 4 ... of all four columns and stores 8 bytes per row instead of 2 (a warp
    // store then covers four rows of 64 bytes; the host checked that every row start and both column
    // bases lie on 16-byte boundaries).  Measured on 128-row tiles, K = N = 8192: 33.9 -> 32.0 us per GEMM;
    // with four rows per thread (the strip reduction of 16-row tiles) the shuffles cost what the stores save.
    constexpr int Q = kRows / 4;
    const int lane = threadIdx.x & 31, q = lane & 3;
    const bool odd = q & 1, upper = q >> 1;
    const unsigned exists = __ballot_sync(0xffffffffu, writes);
    const bool quad_full = ((exists >> (lane & ~3)) & 0xFu) == 0xFu;
    uint2 packed[Q];
#pragma unroll
    for (int j = 0; j < Q; ++j) {
      const float a0 = v[j], a1 = v[Q + j], a2 = v[2 * Q + j], a3 = v[3 * Q + j];      // for lanes 0..3 of the quad
      // with the neighbouring column: the values for the two lanes of this lane's parity
      const float r0 = __shfl_xor_sync(0xffffffffu, odd ? a0 : a1, 1);
      const float r1 = __shfl_xor_sync(0xffffffffu, odd ? a2 : a3, 1);
      const half2 h0 = odd ? __floats2half2_rn(r0, a1) : __floats2half2_rn(a0, r0);      // (even column, odd column) for lane q & 1
      const half2 h1 = odd ? __floats2half2_rn(r1, a3) : __floats2half2_rn(a2, r1);      // ... for lane 2 + (q & 1)
      // with the other pair of columns: keep the pair for this lane, pass the other one on
      const uint32_t keep = h2_as_u32(upper ? h1 : h0);
      const uint32_t got = __shfl_xor_sync(0xffffffffu, h2_as_u32(upper ? h0 : h1), 2);
      packed[j] = upper ? make_uint2(got, keep) : make_uint2(keep, got);
    }
    if (quad_full) {
      const int first_row = row0 + q * Q;
      if (p.out.n_out == 0) {
        half* dst = p.C + (size_t)first_row * p.N + (is6 ? p.geo.n4 : 0) + (col - q);
#pragma unroll
        for (int j = 0; j < Q; ++j)
          if (first_row + j < p.M) *reinterpret_cast<uint2*>(dst + (size_t)j * p.N) = packed[j];
      } else {
        const size_t at = (size_t)first_row * p.out.ld + (is6 ? p.out.col6 : p.out.col4) + (col - q);
#pragma unroll 1
        for (int o = 0; o < p.out.n_out; ++o) {
          half* dst = p.out.peer[o] + at;
#pragma unroll
          for (int j = 0; j < Q; ++j)
            if (first_row + j < p.M) *reinterpret_cast<uint2*>(dst + (size_t)j * p.out.ld) = packed[j];
        }
      }
      return;
    }
    // a quad at the ragged end of the last strip: single values, below
  }
  if (!writes) return;
  if (p.epilogue == kEpilogueResidual) {
    const size_t at = (size_t)(is6 ? p.geo.n4 : 0) + col;
#pragma unroll
    for (int i = 0; i < kRows; ++i)
      if (row0 + i < p.M) {
        const size_t idx = (size_t)(row0 + i) * p.N + at;
        p.C[idx] = __float2half_rn(v[i] + __half2float(p.R[idx]));
      }
    return;
  }
#pragma unroll
  for (int i = 0; i < kRows; ++i)
    if (row0 + i < p.M) store_result(p, row0 + i, is6, col, v[i]);
}

// ---- activations by tiled TMA --------------------------------------------------------------------
// activations of one unit: K-major, 128-byte swizzle (layout type 2), 1024 bytes between 8-row groups;
// the leading-dimension field is not used by swizzled K-major layouts
__device__ __forceinline__ uint64_t wide_act_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// k0 is a multiple of 64 halves = 128 bytes, so the copy starts on a 16-byte boundary
__device__ __forceinline__ void tma_load_act(uint32_t dst, const CUtensorMap* map, int k0, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(k0), "r"(0), "r"(bar) : "memory");
}
// Launch epoch.  Every CTA of a launch reads the epoch word and then counts itself; the CTA that
// completes the count knows that all have read it and advances it for the next launch (also for
// the next replay of a captured graph).  The counting atomic takes its address through the loaded
// value, so it cannot be performed before the load.
__device__ __forceinline__ uint32_t read_epoch_and_count(unsigned int* words, uint32_t ctas) {
  const uint32_t e = ld_relaxed_u32(words);
  uint32_t zero;
  asm volatile("and.b32 %0, %1, 0;" : "=r"(zero) : "r"(e));
  const uint32_t arrived = atomic_add_relaxed_u32(words + 1 + zero, 1u);
  if (arrived == ctas - 1) {
    st_relaxed_u32(words + 1, 0u);
    st_relaxed_u32(words, e + 1);
  }
  return e;
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

// The same expansions times a scale, rounded once to fp16: fp16(q - 8) * s is the dequantised INT4 weight of
// the reference's rule (test.py:98); (value / 4096) * (s * 4096) equals hmul(hmul(bits, 4096), s) of
// dequantMatrix_fp6_to_fp16 (weight_prepacking.cpp:205-212) because the factor 4096 is exact.
__device__ __forceinline__ void expand_int4_scaled(uint32_t q, half2 s, uint32_t* b) {
  uint32_t e[4];
  expand_int4(q, e);
#pragma unroll
  for (int i = 0; i < 4; ++i) b[i] = h2_as_u32(__hmul2(u32_as_h2(e[i]), s));
}
__device__ __forceinline__ void expand_fp6_scaled(uint32_t four, uint32_t two, int rot, half2 s4096, uint32_t* b) {
  uint32_t e[4];
  expand_fp6(four, two, rot, e);
#pragma unroll
  for (int i = 0; i < 4; ++i) b[i] = h2_as_u32(__hmul2(u32_as_h2(e[i]), s4096));
}

// Walks the units [u0, u1) of a CTA as SEGMENTS: runs of one or two units inside one 128-row block
// of one strip (= one INT4 scale group, one TMA copy, one operand slot, one accumulator tile).
// Every role runs the same walk, so ring positions agree without communication.
struct Walk {
  int u, end, ups;
  int unit, unit1;                 // position inside the strip, end of this CTA's slice of the strip
  __device__ __forceinline__ void open_slice() { unit1 = min(ups, unit + end - u); }
  __device__ __forceinline__ void init(int u0, int u1, int ups_) {
    u = u0; end = u1; ups = ups_;
    unit = u % ups;
    open_slice();
  }
  __device__ __forceinline__ bool valid() const { return u < end; }
  __device__ __forceinline__ int count() const { return ((unit & 1) == 0 && unit + 1 < unit1) ? 2 : 1; }
  // returns true when the step left the strip
  __device__ __forceinline__ bool next(int cnt) {
    u += cnt;
    unit += cnt;
    if (unit != ups) return false;
    unit = 0;
    open_slice();
    return true;
  }
};

}  // namespace fp6m
