// W(4&6)A16 GEMM for the memory-bound regime (few rows of A): a persistent, warp-specialised
// sm_100a kernel.  One producer warp streams packed INT4 / FP6 weight blocks (and their group
// scales) from HBM into a ring of shared-memory stages with bulk TMA copies that complete on
// mbarriers; eight consumer warps dequantise the words in registers to fp16 - bit-exact against
// the reference dequantisers - and feed them to the tensor cores with mma.sync (fp32 accumulate).
// Work is split by a byte-weighted stripe schedule over all CTAs; strips shared by several CTAs
// are reduced in fp32 through a scratch buffer by whichever CTA finishes last (no CTA ever waits
// for another), followed by the fp16 epilogue.
//
// This replaces, for the b200 weight layout, the reference's fp6_kernel_marlin
// (fp6_marlin/fp6_marlin_cuda_kernel.cu:288-837): its cp.async ring (:508-546), ldmatrix path
// (:548-563), dequant + mma loop (:565-600), in-CTA and lock-ordered global reductions (:603-696)
// and its epilogue (:698-749).
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "device_utils.cuh"
#include "fp6m_layout.h"
#include "gemm_params.h"

namespace fp6m {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 128;         // + one producer warpgroup (one warp of it works)
constexpr int kStages = 6;
constexpr int kStageWeightBytes = 2 * 4 * kFp6QuadBytes;  // two blocks of a full FP6 strip
constexpr int kStageScaleBytes = 2 * kStripCols * 2;      // two groups of 128 fp16 scales
constexpr int kStageBytes = kStageWeightBytes + kStageScaleBytes;
constexpr int kRedStride = kStripCols + 8;                // floats per row of the reduction buffer
constexpr int kRedWarpFloats = 16 * kRedStride;
constexpr int kRedBytes = kConsumerWarps * kRedWarpFloats * 4;
constexpr int kSmemBytes = kStages * kStageBytes + kRedBytes + 256;

// Walks the blocks [b0, b1) of a CTA as pipeline items: up to two consecutive blocks of one strip.
struct ItemIter {
  int blk, end, k128;
  int strip, kb, nblk;
  bool valid;
  __device__ __forceinline__ void init(int b0, int b1, int k128_) {
    blk = b0; end = b1; k128 = k128_;
    load();
  }
  __device__ __forceinline__ void load() {
    valid = blk < end;
    if (valid) {
      strip = blk / k128;
      kb = blk - strip * k128;
      int slice_end = min(end, (strip + 1) * k128);
      nblk = min(2, slice_end - blk);
    }
  }
  __device__ __forceinline__ void next() { blk += nblk; load(); }
};

template <int MB>
__global__ void __launch_bounds__(kThreads, 1) w46_gemm_mma_kernel(const __grid_constant__ MulParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* stage_base = smem;
  float* red = reinterpret_cast<float*>(smem + kStages * kStageBytes);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes + kRedBytes);
  int* flag = reinterpret_cast<int*>(bars + 2 * kStages);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kStages);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x;
  const Geometry& geo = p.geo;
  const int b0 = p.sched.bound[cta], b1 = p.sched.bound[cta + 1];

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, kConsumerWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();
  if (b0 >= b1) return;

  bool dead = false;

  if (warp >= kConsumerWarps) {
    // ------------------------------------------------------------------ producer warpgroup
    // gives most of its registers to the consumers; only lane 0 of its first warp issues copies
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    if (warp == kConsumerWarps && lane == 0) {
      const uint64_t policy = make_evict_first_policy();
      ItemIter it;
      it.init(b0, b1, geo.k128);
      int n = 0;
      for (; it.valid; it.next(), ++n) {
        const int s = n % kStages;
        const uint32_t round = n / kStages;
        mbar_wait_bounded(empty0 + 8 * s, (round & 1) ^ 1, p.status, dead);
        const bool is6 = it.strip >= geo.strips4;
        const int strip = is6 ? it.strip - geo.strips4 : it.strip;
        const int nq = strip_quads(is6 ? geo.n6 : geo.n4, strip);
        const uint32_t wbytes = it.nblk * nq * (is6 ? kFp6QuadBytes : kInt4QuadBytes);
        const uint8_t* wsrc = p.B + (is6 ? fp6_block_offset(geo, strip, it.kb) : int4_block_offset(geo, strip, it.kb));
        const bool group_scales = !is6 && geo.groups > 1;
        const uint32_t sbytes = group_scales ? it.nblk * nq * kQuadCols * 2 : 0;
        const uint32_t dst = smem_u32(stage_base + s * kStageBytes);
        mbar_arrive_expect_tx(full0 + 8 * s, wbytes + sbytes);
        tma_load_1d_stream(dst, wsrc, wbytes, full0 + 8 * s, policy);
        if (group_scales)
          tma_load_1d(dst + kStageWeightBytes, p.S + int4_scale_offset(geo, strip, it.kb), sbytes, full0 + 8 * s);
      }
      // Do not leave while copies may still be landing in this CTA's shared memory.
      const int issued = n;
      for (int k = max(0, issued - kStages); k < issued; ++k)
        mbar_wait_bounded(full0 + 8 * (k % kStages), (k / kStages) & 1, p.status, dead);
    }
    return;
  }

  // -------------------------------------------------------------------- consumer warps
  asm volatile("setmaxnreg.inc.sync.aligned.u32 232;");
  const int g = lane >> 2, t = lane & 3;
  const int bh = warp >> 2;      // which of the item's two blocks this warp works on
  const int win = warp & 3;      // 32-row window inside the block
  const half2 k4096 = __float2half2_rn(4096.0f);

  float acc[MB][16][4];
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int j = 0; j < 16; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[mb][j][e] = 0.f;

  // A fragments for one item: rows g and g+8 of each 16-row block, 8 consecutive halves each.
  uint4 a_cur[MB][2], a_nxt[MB][2];
  auto load_a = [&](const ItemIter& it, uint4 (&dst)[MB][2]) {
    const int k0 = (it.kb + bh) * kBlockRows + 32 * win + 8 * t;
    const bool k_ok = it.valid && bh < it.nblk && k0 < p.K;
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int row = mb * 16 + g + 8 * h;
        if (k_ok && row < p.M)
          dst[mb][h] = __ldg(reinterpret_cast<const uint4*>(p.A + (size_t)row * p.K + k0));
        else
          dst[mb][h] = make_uint4(0, 0, 0, 0);
      }
  };

  ItemIter it;
  it.init(b0, b1, geo.k128);
  load_a(it, a_cur);
  int n = 0;
  const int first_strip = it.strip;

  while (it.valid) {
    // ---- one slice = this CTA's share of one strip
    const int strip_lin = it.strip;
    const bool is6 = strip_lin >= geo.strips4;
    const int strip = is6 ? strip_lin - geo.strips4 : strip_lin;
    const int nq = strip_quads(is6 ? geo.n6 : geo.n4, strip);
    const bool group_scales = !is6 && geo.groups > 1;
    const int slice_kb0 = it.kb;

    // Per-slice scales (per-channel INT4, FP6): four fp16 per quad for this lane's column g.
    uint2 sc[4];
    if (!group_scales) {
      const half* sp = p.S + (is6 ? fp6_scale_offset(geo, strip) : int4_scale_offset(geo, strip, 0)) + g * 4 * nq;
#pragma unroll
      for (int jq = 0; jq < 4; ++jq)
        if (jq < nq) {
          sc[jq] = __ldg(reinterpret_cast<const uint2*>(sp) + jq);
          if (is6) {
            sc[jq].x = h2_as_u32(__hmul2(u32_as_h2(sc[jq].x), k4096));
            sc[jq].y = h2_as_u32(__hmul2(u32_as_h2(sc[jq].y), k4096));
          }
        }
    }

    int slice_blocks = 0;
    while (it.valid && it.strip == strip_lin) {
      ItemIter nx = it;
      nx.next();
      load_a(nx, a_nxt);

      const int s = n % kStages;
      mbar_wait_bounded(full0 + 8 * s, (n / kStages) & 1, p.status, dead);

      if (bh < it.nblk) {
        const uint8_t* st = stage_base + s * kStageBytes;
        const uint8_t* blk = st + bh * nq * (is6 ? kFp6QuadBytes : kInt4QuadBytes);
        const uint4* w4 = reinterpret_cast<const uint4*>(blk) + (win * nq) * 32 + lane;
        const uint2* w2 = reinterpret_cast<const uint2*>(blk + nq * kInt4QuadBytes) + (win * nq) * 32 + lane;
        const uint2* ss = reinterpret_cast<const uint2*>(st + kStageWeightBytes + bh * nq * kQuadCols * 2) + g * nq;
#pragma unroll
        for (int jq = 0; jq < 4; ++jq) {
          if (jq < nq) {
            const uint4 q = w4[jq * 32];
            uint2 two = make_uint2(0, 0);
            if (is6) two = w2[jq * 32];
            if (group_scales) sc[jq] = ss[jq];
            const uint32_t qs[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int jr = 0; jr < 4; ++jr) {
              const uint32_t spair = (jr < 2) ? sc[jq].x : sc[jq].y;
              const half2 s2 = u32_as_h2(prmt(spair, spair, (jr & 1) ? 0x3232u : 0x1010u));
              uint32_t b[4];
              if (is6)
                dequant_fp6_word(qs[jr], (jr < 2) ? two.x : two.y, 4 * (jr & 1), s2, b);
              else
                dequant_int4_word(qs[jr], s2, b);
#pragma unroll
              for (int mb = 0; mb < MB; ++mb) {
                mma_16816(acc[mb][jq * 4 + jr], a_cur[mb][0].x, a_cur[mb][1].x, a_cur[mb][0].y, a_cur[mb][1].y, b[0], b[1]);
                mma_16816(acc[mb][jq * 4 + jr], a_cur[mb][0].z, a_cur[mb][1].z, a_cur[mb][0].w, a_cur[mb][1].w, b[2], b[3]);
              }
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty0 + 8 * s);

      slice_blocks += it.nblk;
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) { a_cur[mb][0] = a_nxt[mb][0]; a_cur[mb][1] = a_nxt[mb][1]; }
      it = nx;
      ++n;
    }

    // ---- slice finished: reduce the eight warps, then either write C or hand over a partial
    const bool full_strip = (slice_kb0 == 0) && (slice_blocks == geo.k128);
    const int ncols = strip_cols(is6 ? geo.n6 : geo.n4, strip);
    const int col0 = (is6 ? geo.n4 : 0) + strip * kStripCols;
    const int r = tid >> 4, c8 = (tid & 15) * 8;       // this thread's output row and 8 columns

    int contributors = 1, c_lo = cta, c_hi = cta;
    if (!full_strip) {
      const int s_begin = strip_lin * geo.k128, s_end = s_begin + geo.k128;
      while (c_lo > 0 && p.sched.bound[c_lo] > s_begin) --c_lo;
      while (c_hi + 1 < p.sched.ctas && p.sched.bound[c_hi + 1] < s_end) ++c_hi;
      contributors = 0;
      for (int c = c_lo; c <= c_hi; ++c) contributors += p.sched.bound[c] < p.sched.bound[c + 1];
    }
    const size_t slot_floats = (size_t)MB * 16 * kStripCols;
    float* my_slot = p.partials + (size_t)(2 * cta + (strip_lin != first_strip ? 1 : 0)) * slot_floats;

#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
      float* mine = red + warp * kRedWarpFloats;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        *reinterpret_cast<float2*>(mine + g * kRedStride + 8 * j + 2 * t) = make_float2(acc[mb][j][0], acc[mb][j][1]);
        *reinterpret_cast<float2*>(mine + (g + 8) * kRedStride + 8 * j + 2 * t) = make_float2(acc[mb][j][2], acc[mb][j][3]);
        acc[mb][j][0] = acc[mb][j][1] = acc[mb][j][2] = acc[mb][j][3] = 0.f;
      }
      named_bar_sync(1, kConsumerThreads);
      float v[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) {
        const float4 x = *reinterpret_cast<const float4*>(red + w * kRedWarpFloats + r * kRedStride + c8);
        const float4 y = *reinterpret_cast<const float4*>(red + w * kRedWarpFloats + r * kRedStride + c8 + 4);
        v[0] += x.x; v[1] += x.y; v[2] += x.z; v[3] += x.w;
        v[4] += y.x; v[5] += y.y; v[6] += y.z; v[7] += y.w;
      }
      const int row = mb * 16 + r;
      if (full_strip) {
        if (row < p.M && c8 < ncols) {
          uint4 o;
          o.x = h2_as_u32(__floats2half2_rn(v[0], v[1]));
          o.y = h2_as_u32(__floats2half2_rn(v[2], v[3]));
          o.z = h2_as_u32(__floats2half2_rn(v[4], v[5]));
          o.w = h2_as_u32(__floats2half2_rn(v[6], v[7]));
          *reinterpret_cast<uint4*>(p.C + (size_t)row * p.N + col0 + c8) = o;
        }
      } else {
        float4* dst = reinterpret_cast<float4*>(my_slot + (size_t)row * kStripCols + c8);
        __stcg(dst, make_float4(v[0], v[1], v[2], v[3]));
        __stcg(dst + 1, make_float4(v[4], v[5], v[6], v[7]));
      }
      named_bar_sync(1, kConsumerThreads);   // red is free again
    }

    if (!full_strip) {
      __threadfence();
      named_bar_sync(1, kConsumerThreads);
      if (tid == 0) {
        const int prev = atomicAdd(p.counters + strip_lin, 1);
        const int last = prev == contributors - 1;
        if (last) p.counters[strip_lin] = 0;   // leave the workspace zeroed, as the reference does
        *flag = last;
      }
      named_bar_sync(1, kConsumerThreads);
      const bool last = *flag != 0;
      if (last) {
        __threadfence();
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          const int row = mb * 16 + r;
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = 0.f;
          for (int c = c_lo; c <= c_hi; ++c) {
            if (p.sched.bound[c] >= p.sched.bound[c + 1]) continue;
            const int c_first_strip = p.sched.bound[c] / geo.k128;
            const float* src = p.partials + (size_t)(2 * c + (strip_lin != c_first_strip ? 1 : 0)) * slot_floats +
                               (size_t)row * kStripCols + c8;
            const float4 x = __ldcg(reinterpret_cast<const float4*>(src));
            const float4 y = __ldcg(reinterpret_cast<const float4*>(src) + 1);
            v[0] += x.x; v[1] += x.y; v[2] += x.z; v[3] += x.w;
            v[4] += y.x; v[5] += y.y; v[6] += y.z; v[7] += y.w;
          }
          if (row < p.M && c8 < ncols) {
            uint4 o;
            o.x = h2_as_u32(__floats2half2_rn(v[0], v[1]));
            o.y = h2_as_u32(__floats2half2_rn(v[2], v[3]));
            o.z = h2_as_u32(__floats2half2_rn(v[4], v[5]));
            o.w = h2_as_u32(__floats2half2_rn(v[6], v[7]));
            *reinterpret_cast<uint4*>(p.C + (size_t)row * p.N + col0 + c8) = o;
          }
        }
      }
      named_bar_sync(1, kConsumerThreads);     // flag may be rewritten by the next slice
    }
  }
}

template <int MB>
cudaError_t launch_one(const MulParams& p, cudaStream_t stream) {
  static bool configured[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 16 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(w46_gemm_mma_kernel<MB>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  w46_gemm_mma_kernel<MB><<<p.sched.ctas, kThreads, kSmemBytes, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace

int mma_rows_per_pass() { return 32; }

size_t mma_scratch_bytes(int ctas, int rows_per_pass) {
  return (size_t)2 * ctas * rows_per_pass * kStripCols * sizeof(float);
}

// Runs the GEMM for rows [0, p.M) with p.M <= 32; the host dispatcher loops over larger M.
cudaError_t launch_gemm_mma(const MulParams& p, cudaStream_t stream) {
  if (p.M <= 16) return launch_one<1>(p, stream);
  return launch_one<2>(p, stream);
}

}  // namespace fp6m
