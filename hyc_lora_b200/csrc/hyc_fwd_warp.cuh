// Warp-per-row forward kernel for the channel-outlier mode (bf16 rows of up to 16 register
// groups per lane, i.e. 4096 channels): compress-only and fused norm + compress.
//
// Every warp walks its own rows.  A row is staged in the warp's own shared-memory slot by one
// bulk asynchronous copy (completion on the warp's own mbarrier), its outlier channels are saved,
// written out and zeroed in the slot, and the lane's share -- units lane, lane+32, ... (see
// hyc_rows.cuh for the unit mapping) -- moves into registers as raw bf16.  The slot is then handed
// straight back to the copy engine, so the next row travels while this one is computed from
// registers: pass 1 accumulates the row statistics (sum of squares in fp32, absmax with packed
// bf16 min/max), warp shuffles reduce them, pass 2 writes the norm output and the packed codes.
// There is no CTA barrier in the row loop and no thread waits for another warp: the per-row scalar
// work (reductions, the two divisions, ring bookkeeping) is paid once per 128 elements of a lane
// instead of once per 32 as in the CTA-per-row kernel, which is what takes the kernel from
// instruction-issue-bound towards memory-bound.
//
// Arithmetic is that of fwd_n_fast_kernel: codes, scales and outlier values are bit-identical.
#pragma once
#include "hyc_fwd_fast.cuh"

namespace hyc {

constexpr int kWarpKernelThreads = 256;
constexpr int kWarpKernelCtasPerSm = 2;
constexpr int kWarpRotThreads = 384;           // rotating variant: one CTA per SM, the rotated row lives in registers
constexpr int kWarpOutPerLane = 4;          // outlier channels a lane looks after: k <= 128

struct WarpFwdArgs {
  PackedDev p;
  PackedDev p2;          // two-record variant: the record of the norm output
  const __nv_bfloat16* x;
  long long row_stride;  // elements
  int kind;
  float eps;
  const void* weight;
  const void* bias;
  int param_bf16;
  __nv_bfloat16* y;
  float* rstd;
  float* mean;
  uint32_t off_chan, off_chan2, off_wsm, off_bsm, off_slots, slot_bytes;
  long long wait_cycles;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// |.| maximum of the eight bf16 values of a 16-byte group, kept as packed bf16 pairs
__device__ __forceinline__ __nv_bfloat162 absmax_acc(__nv_bfloat162 m, const uint4& w) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
  m = __hmax2(m, __habs2(h[0]));
  m = __hmax2(m, __habs2(h[1]));
  m = __hmax2(m, __habs2(h[2]));
  return __hmax2(m, __habs2(h[3]));
}
// Tells the compiler that the register group may have changed: values unpacked from it before are not
// carried across (the passes unpack again, one instruction per element, instead of holding the whole
// row in fp32 next to the raw copy).
__device__ __forceinline__ void forget_unpacked(uint4& w) {
  asm volatile("" : "+r"(w.x), "+r"(w.y), "+r"(w.z), "+r"(w.w));
}
__device__ __forceinline__ void forget_unpacked2(uint2& w) { asm volatile("" : "+r"(w.x), "+r"(w.y)); }
__device__ __forceinline__ float pair_max(__nv_bfloat162 m) {
  return fmaxf(__bfloat162float(__low2bfloat16(m)), __bfloat162float(__high2bfloat16(m)));
}

// Group scales of one row.  On entry v[r] is the absmax of the 128-channel group that register group r of
// this half-warp belongs to (the same value on its 16 lanes); on exit v[r] is the group's reciprocal scale.
// The two divisions per group are shared out: lane i of the half-warp divides for register group i, stores
// that group's scale and hands the reciprocal to the other lanes by shuffle (one shuffle instead of a
// division sequence per lane and group).
template <int BITS, int NG>
__device__ __forceinline__ void group_scales(float (&v)[NG], float* scales_row, int segw, int U, int lane) {
  constexpr int NSEG = 8 / BITS;
  const float qmax = static_cast<float>(CodeTraits<BITS>::kHi);
  const int i = lane & 15;
  float mine = 0.f;
#pragma unroll
  for (int r = 0; r < NG; ++r) mine = (i == r) ? v[r] : mine;
  const bool live = mine > 0.f;
  const float inv = live ? __fdiv_rn(qmax, mine) : 1.f;
  const int u0 = (lane & 16) + 32 * (i / NSEG);             // first unit of this half-warp in register group i
  if (i < NG && u0 < U) scales_row[((i % NSEG) * segw + (u0 << 3)) >> 7] = live ? __fdiv_rn(mine, qmax) : 1.f;
#pragma unroll
  for (int r = 0; r < NG; ++r) v[r] = __shfl_sync(0xffffffffu, inv, (lane & 16) | (r & 15));
}

// One row of the walk above, staged in `xs`: outlier channels, statistics, norm output, codes.
// `next_src`: the row to bring into the slot once this one is in registers (nullptr: none).  TO_SLOT (the
// first stage of the two-record variant): the slot is not handed back; instead the norm output, complete
// with its outlier channels, takes the row's place in it, for a second call that compresses it.
template <int BITS, int NK, int NG, bool GROUP, bool TO_SLOT>
__device__ __forceinline__ void warp_row_plain(const WarpFwdArgs& a, const PackedDev& p, const int (&oc)[kWarpOutPerLane],
                                               __nv_bfloat16* xs, uint64_t* bar, long long row,
                                               const __nv_bfloat16* next_src, const float* wsm, const float* bsm) {
  using C = CodeTraits<BITS>;
  constexpr int NSEG = C::kSeg;
  constexpr int UPL = NG / NSEG;
  constexpr bool NORM = NK != 0;
  constexpr bool ln = NK == 2;
  const int D = p.cols;
  const int segw = D / NSEG;
  const int U = segw >> 3;
  const int k = p.n_channels;
  const int lane = threadIdx.x & 31;
  const int G = GROUP ? (D >> 7) : 1;
  const float qmax = static_cast<float>(C::kHi);
  const float inv_d = 1.0f / static_cast<float>(D);
  const uint32_t row_bytes = static_cast<uint32_t>(D) * 2u;
  {
    // ---- outlier channels: keep the original, write it out, zero it in the staged row
    float ov[kWarpOutPerLane];
#pragma unroll
    for (int q = 0; q < kWarpOutPerLane; ++q) {
      ov[q] = 0.f;
      if (oc[q] >= 0) {
        const __nv_bfloat16 o = xs[oc[q]];
        p.out_value[row * k + lane + 32 * q] = o;
        ov[q] = __bfloat162float(o);
        xs[oc[q]] = __float2bfloat16_rn(0.f);
      }
    }
    __syncwarp();
    // ---- the lane's share of the row, raw
    uint4 raw[NG];
#pragma unroll
    for (int r = 0; r < NG; ++r) {
      const int u = lane + 32 * (r / NSEG);
      raw[r] = u < U ? *reinterpret_cast<const uint4*>(xs + (r % NSEG) * segw + (u << 3)) : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncwarp();
    // every lane has what it needs: hand the slot back to the copy engine
    if (!TO_SLOT && lane == 0 && next_src) {
      fence_proxy_async();
      mbar_expect_tx(bar, row_bytes);
      bulk_g2s(xs, next_src, row_bytes, bar);
    }
    // ---- statistics
    float mean = 0.f;
    if (ln) {
      float s1 = 0.f;
#pragma unroll
      for (int r = 0; r < NG; ++r) {
        float f[8];
        unpack_bf16x8(raw[r], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) s1 += f[e];
      }
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q) s1 += ov[q];
      mean = warp_sum(s1) * inv_d;
#pragma unroll
      for (int r = 0; r < NG; ++r) forget_unpacked(raw[r]);
    }
    float ss = 0.f;
    __nv_bfloat162 am2 = __float2bfloat162_rn(0.f);
    float ginv[GROUP ? NG : 1];
#pragma unroll
    for (int r = 0; r < NG; ++r) {
      if (NORM) {
        float f[8];
        unpack_bf16x8(raw[r], f);
        if (ln) {
          const bool live = (lane + 32 * (r / NSEG)) < U;
#pragma unroll
          for (int e = 0; e < 8; ++e) { const float c = f[e] - mean; ss = live ? fmaf(c, c, ss) : ss; }
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
        }
      }
      if (GROUP) {
        // 16 consecutive lanes hold one 128-channel group of this register group
        float a8 = pair_max(absmax_acc(__float2bfloat162_rn(0.f), raw[r]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) a8 = fmaxf(a8, __shfl_xor_sync(0xffffffffu, a8, o));
        ginv[r] = a8;
      } else {
        am2 = absmax_acc(am2, raw[r]);
      }
    }
    if constexpr (GROUP) group_scales<BITS, NG>(ginv, p.scales + row * G, segw, U, lane);
    float rstd = 0.f;
    if (NORM) {
      // the zeroed outlier channels still belong to the row statistics
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q)
        if (oc[q] >= 0) ss += ln ? ((ov[q] - mean) * (ov[q] - mean) - mean * mean) : ov[q] * ov[q];
      ss = warp_sum(ss);
      rstd = 1.0f / sqrtf(ss * inv_d + a.eps);
      if (lane == 0) {
        a.rstd[row] = rstd;
        if (ln) a.mean[row] = mean;
      }
    }
    float inv_row = 1.f;
    if (!GROUP) {
      const float amax = warp_max(pair_max(am2));
      const bool live = amax > 0.f;
      inv_row = live ? __fdiv_rn(qmax, amax) : 1.f;
      if (lane == 0) p.scales[row] = live ? __fdiv_rn(amax, qmax) : 1.f;
    }
    // ---- pass 2: norm output and packed codes from the registers
#pragma unroll
    for (int r = 0; r < NG; ++r) forget_unpacked(raw[r]);
    unsigned char* codes_row = p.codes + row * (static_cast<long long>(D) * BITS / 8);
    __nv_bfloat16* yrow = NORM ? a.y + row * a.row_stride : nullptr;
#pragma unroll
    for (int iu = 0; iu < UPL; ++iu) {
      const int u = lane + 32 * iu;
      if (u < U) {
        PackAcc<BITS> acc;
#pragma unroll
        for (int s = 0; s < NSEG; ++s) {
          const int col = s * segw + (u << 3);
          float f[8];
          unpack_bf16x8(raw[iu * NSEG + s], f);
          if (NORM) {
            float y[8], wv[8];
            load8_split(wsm, D, col, wv);
            if (ln) {
              float bv[8];
              load8_split(bsm, D, col, bv);
#pragma unroll
              for (int e = 0; e < 8; ++e) y[e] = (f[e] - mean) * rstd * wv[e] + bv[e];
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) y[e] = f[e] * rstd * wv[e];
            }
            store8<__nv_bfloat16>(yrow, col, y);
            if (TO_SLOT) store8<__nv_bfloat16>(xs, col, y);    // the norm output takes the row's place in the slot
          }
          acc.add(f, GROUP ? ginv[iu * NSEG + s] : inv_row, s);
        }
        *reinterpret_cast<uint2*>(codes_row + (u << 3)) = acc.done();
      }
      // keep the table loads of the next unit behind this unit's stores: hoisting all of them to the top of
      // the unrolled pass would cost more registers than the raw row itself
      if (NORM && (iu & 1)) asm volatile("" ::: "memory");
    }
    if (NORM) {
      // the vector stores above wrote the norm of the zeroed value at the outlier channels: order
      // them before the scalar stores of the real values (same warp, other lanes)
      __syncwarp();
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q) {
        if (oc[q] >= 0) {
          const int cs = split_index(oc[q], D);
          const float y = ln ? ((ov[q] - mean) * rstd * wsm[cs] + bsm[cs]) : (ov[q] * rstd * wsm[cs]);
          yrow[oc[q]] = __float2bfloat16_rn(y);
          if (TO_SLOT) xs[oc[q]] = __float2bfloat16_rn(y);
        }
      }
    }
  }
}

// NK: 0 compress only, 1 RMSNorm (plain or Gemma), 2 LayerNorm;  NG: 16-byte register groups per lane
// (units per lane x segments)
template <int BITS, int NK, int NG, bool GROUP>
__global__ void __launch_bounds__(kWarpKernelThreads, kWarpKernelCtasPerSm) fwd_n_warp_kernel(const __grid_constant__ WarpFwdArgs a) {
  using C = CodeTraits<BITS>;
  constexpr int NSEG = C::kSeg;
  constexpr int UPL = NG / NSEG;
  constexpr bool NORM = NK != 0;
  constexpr bool ln = NK == 2;
  static_assert(UPL >= 1 && UPL * NSEG == NG, "register groups must cover whole units");
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  const int D = p.cols;
  const int segw = D / NSEG;
  const int U = segw >> 3;
  const int k = p.n_channels;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
  const int G = GROUP ? (D >> 7) : 1;
  const float qmax = static_cast<float>(C::kHi);
  const float inv_d = 1.0f / static_cast<float>(D);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  int* chan = reinterpret_cast<int*>(smem + a.off_chan);
  float* wsm = reinterpret_cast<float*>(smem + a.off_wsm);
  float* bsm = reinterpret_cast<float*>(smem + a.off_bsm);
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem + a.off_slots + static_cast<size_t>(warp) * a.slot_bytes);
  uint64_t* bar = &bars[warp];
  const uint32_t row_bytes = static_cast<uint32_t>(D) * 2u;
  const long long rows = p.rows, stride = static_cast<long long>(gridDim.x) * W;
  long long row = static_cast<long long>(blockIdx.x) * W + warp;
  if (threadIdx.x == 0) {
    for (int i = 0; i < W; ++i) mbar_init(&bars[i], 1);
    fence_barrier_init();
  }
  __syncthreads();
  // the first row of every warp starts travelling before the per-CTA tables are set up
  if (lane == 0 && row < rows) {
    mbar_expect_tx(bar, row_bytes);
    bulk_g2s(xs, a.x + row * a.row_stride, row_bytes, bar);
  }
  for (int j = threadIdx.x; j < k; j += blockDim.x) chan[j] = p.channels[j];
  if (NORM) {
    const float plus = a.kind == HYC_NORM_RMS_GEMMA ? 1.f : 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      wsm[split_index(c, D)] = (a.param_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.weight)[c])
                                             : static_cast<const float*>(a.weight)[c]) + plus;
      if (ln)
        bsm[split_index(c, D)] = a.param_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.bias)[c])
                                              : static_cast<const float*>(a.bias)[c];
    }
  }
  __syncthreads();
  // the outlier channels this lane looks after (-1: none)
  int oc[kWarpOutPerLane];
#pragma unroll
  for (int q = 0; q < kWarpOutPerLane; ++q) oc[q] = (lane + 32 * q) < k ? chan[lane + 32 * q] : -1;

  uint32_t ph = 0;
  for (; row < rows; row += stride, ph ^= 1u) {
    if (!mbar_wait_bounded(bar, ph, a.wait_cycles)) {
      // the only copy this warp has in flight is the one it gave up on
      if (lane == 0 && p.status) atomicOr(p.status, kStatusWaitExpired);
      return;
    }
    // ---- outlier channels: keep the original, write it out, zero it in the staged row
    float ov[kWarpOutPerLane];
#pragma unroll
    for (int q = 0; q < kWarpOutPerLane; ++q) {
      ov[q] = 0.f;
      if (oc[q] >= 0) {
        const __nv_bfloat16 o = xs[oc[q]];
        p.out_value[row * k + lane + 32 * q] = o;
        ov[q] = __bfloat162float(o);
        xs[oc[q]] = __float2bfloat16_rn(0.f);
      }
    }
    __syncwarp();
    // ---- the lane's share of the row, raw
    uint4 raw[NG];
#pragma unroll
    for (int r = 0; r < NG; ++r) {
      const int u = lane + 32 * (r / NSEG);
      raw[r] = u < U ? *reinterpret_cast<const uint4*>(xs + (r % NSEG) * segw + (u << 3)) : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncwarp();
    // every lane has what it needs: hand the slot back to the copy engine
    const long long next = row + stride;
    if (lane == 0 && next < rows) {
      fence_proxy_async();
      mbar_expect_tx(bar, row_bytes);
      bulk_g2s(xs, a.x + next * a.row_stride, row_bytes, bar);
    }
    // ---- statistics
    float mean = 0.f;
    if (ln) {
      float s1 = 0.f;
#pragma unroll
      for (int r = 0; r < NG; ++r) {
        float f[8];
        unpack_bf16x8(raw[r], f);
#pragma unroll
        for (int e = 0; e < 8; ++e) s1 += f[e];
      }
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q) s1 += ov[q];
      mean = warp_sum(s1) * inv_d;
#pragma unroll
      for (int r = 0; r < NG; ++r) forget_unpacked(raw[r]);
    }
    float ss = 0.f;
    __nv_bfloat162 am2 = __float2bfloat162_rn(0.f);
    float ginv[GROUP ? NG : 1];
#pragma unroll
    for (int r = 0; r < NG; ++r) {
      if (NORM) {
        float f[8];
        unpack_bf16x8(raw[r], f);
        if (ln) {
          const bool live = (lane + 32 * (r / NSEG)) < U;
#pragma unroll
          for (int e = 0; e < 8; ++e) { const float c = f[e] - mean; ss = live ? fmaf(c, c, ss) : ss; }
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
        }
      }
      if (GROUP) {
        // 16 consecutive lanes hold one 128-channel group of this register group
        float a8 = pair_max(absmax_acc(__float2bfloat162_rn(0.f), raw[r]));
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) a8 = fmaxf(a8, __shfl_xor_sync(0xffffffffu, a8, o));
        ginv[r] = a8;
      } else {
        am2 = absmax_acc(am2, raw[r]);
      }
    }
    if constexpr (GROUP) group_scales<BITS, NG>(ginv, p.scales + row * G, segw, U, lane);
    float rstd = 0.f;
    if (NORM) {
      // the zeroed outlier channels still belong to the row statistics
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q)
        if (oc[q] >= 0) ss += ln ? ((ov[q] - mean) * (ov[q] - mean) - mean * mean) : ov[q] * ov[q];
      ss = warp_sum(ss);
      rstd = 1.0f / sqrtf(ss * inv_d + a.eps);
      if (lane == 0) {
        a.rstd[row] = rstd;
        if (ln) a.mean[row] = mean;
      }
    }
    float inv_row = 1.f;
    if (!GROUP) {
      const float amax = warp_max(pair_max(am2));
      const bool live = amax > 0.f;
      inv_row = live ? __fdiv_rn(qmax, amax) : 1.f;
      if (lane == 0) p.scales[row] = live ? __fdiv_rn(amax, qmax) : 1.f;
    }
    // ---- pass 2: norm output and packed codes from the registers
#pragma unroll
    for (int r = 0; r < NG; ++r) forget_unpacked(raw[r]);
    unsigned char* codes_row = p.codes + row * (static_cast<long long>(D) * BITS / 8);
    __nv_bfloat16* yrow = NORM ? a.y + row * a.row_stride : nullptr;
#pragma unroll
    for (int iu = 0; iu < UPL; ++iu) {
      const int u = lane + 32 * iu;
      if (u < U) {
        PackAcc<BITS> acc;
#pragma unroll
        for (int s = 0; s < NSEG; ++s) {
          const int col = s * segw + (u << 3);
          float f[8];
          unpack_bf16x8(raw[iu * NSEG + s], f);
          if (NORM) {
            float y[8], wv[8];
            load8_split(wsm, D, col, wv);
            if (ln) {
              float bv[8];
              load8_split(bsm, D, col, bv);
#pragma unroll
              for (int e = 0; e < 8; ++e) y[e] = (f[e] - mean) * rstd * wv[e] + bv[e];
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) y[e] = f[e] * rstd * wv[e];
            }
            store8<__nv_bfloat16>(yrow, col, y);
          }
          acc.add(f, GROUP ? ginv[iu * NSEG + s] : inv_row, s);
        }
        *reinterpret_cast<uint2*>(codes_row + (u << 3)) = acc.done();
      }
      // keep the table loads of the next unit behind this unit's stores: hoisting all of them to the top of
      // the unrolled pass would cost more registers than the raw row itself
      if (NORM && (iu & 1)) asm volatile("" ::: "memory");
    }
    if (NORM) {
      // the vector stores above wrote the norm of the zeroed value at the outlier channels: order
      // them before the scalar stores of the real values (same warp, other lanes)
      __syncwarp();
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q) {
        if (oc[q] >= 0) {
          const int cs = split_index(oc[q], D);
          const float y = ln ? ((ov[q] - mean) * rstd * wsm[cs] + bsm[cs]) : (ov[q] * rstd * wsm[cs]);
          yrow[oc[q]] = __float2bfloat16_rn(y);
        }
      }
    }
  }
}

// The two-record variant of the kernel above: a second record (a.p2, with its own outlier channels) takes the
// compressed norm OUTPUT -- the sites behind a norm save that tensor, and this way it is compressed in the pass
// that produces it.  The row body is warp_row_plain, run twice on the warp's slot.  (The one-record kernel
// keeps its own hand-scheduled body: folding both into one template cost it 15 % at 65 536 rows.)
template <int BITS, int NK, int NG, bool GROUP>
__global__ void __launch_bounds__(kWarpKernelThreads, kWarpKernelCtasPerSm) fwd_n_warp_dual_kernel(const __grid_constant__ WarpFwdArgs a) {
  constexpr bool DUAL = true;
  using C = CodeTraits<BITS>;
  constexpr int NSEG = C::kSeg;
  constexpr int UPL = NG / NSEG;
  constexpr bool NORM = NK != 0;
  constexpr bool ln = NK == 2;
  static_assert(UPL >= 1 && UPL * NSEG == NG, "register groups must cover whole units");
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  const int D = p.cols;
  const int segw = D / NSEG;
  const int U = segw >> 3;
  const int k = p.n_channels;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
  const int G = GROUP ? (D >> 7) : 1;
  const float qmax = static_cast<float>(C::kHi);
  const float inv_d = 1.0f / static_cast<float>(D);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  int* chan = reinterpret_cast<int*>(smem + a.off_chan);
  float* wsm = reinterpret_cast<float*>(smem + a.off_wsm);
  float* bsm = reinterpret_cast<float*>(smem + a.off_bsm);
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem + a.off_slots + static_cast<size_t>(warp) * a.slot_bytes);
  uint64_t* bar = &bars[warp];
  const uint32_t row_bytes = static_cast<uint32_t>(D) * 2u;
  const long long rows = p.rows, stride = static_cast<long long>(gridDim.x) * W;
  long long row = static_cast<long long>(blockIdx.x) * W + warp;
  if (threadIdx.x == 0) {
    for (int i = 0; i < W; ++i) mbar_init(&bars[i], 1);
    fence_barrier_init();
  }
  __syncthreads();
  // the first row of every warp starts travelling before the per-CTA tables are set up
  if (lane == 0 && row < rows) {
    mbar_expect_tx(bar, row_bytes);
    bulk_g2s(xs, a.x + row * a.row_stride, row_bytes, bar);
  }
  for (int j = threadIdx.x; j < k; j += blockDim.x) chan[j] = p.channels[j];
  int* chan2 = reinterpret_cast<int*>(smem + a.off_chan2);
  if (DUAL)
    for (int j = threadIdx.x; j < a.p2.n_channels; j += blockDim.x) chan2[j] = a.p2.channels[j];
  if (NORM) {
    const float plus = a.kind == HYC_NORM_RMS_GEMMA ? 1.f : 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      wsm[split_index(c, D)] = (a.param_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.weight)[c])
                                             : static_cast<const float*>(a.weight)[c]) + plus;
      if (ln)
        bsm[split_index(c, D)] = a.param_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.bias)[c])
                                              : static_cast<const float*>(a.bias)[c];
    }
  }
  __syncthreads();
  // the outlier channels this lane looks after (-1: none)
  int oc[kWarpOutPerLane];
#pragma unroll
  for (int q = 0; q < kWarpOutPerLane; ++q) oc[q] = (lane + 32 * q) < k ? chan[lane + 32 * q] : -1;
  int oc2[kWarpOutPerLane];
#pragma unroll
  for (int q = 0; q < kWarpOutPerLane; ++q) oc2[q] = (DUAL && (lane + 32 * q) < a.p2.n_channels) ? chan2[lane + 32 * q] : -1;

  uint32_t ph = 0;
  for (; row < rows; row += stride, ph ^= 1u) {
    if (!mbar_wait_bounded(bar, ph, a.wait_cycles)) {
      // the only copy this warp has in flight is the one it gave up on
      if (lane == 0 && p.status) atomicOr(p.status, kStatusWaitExpired);
      return;
    }
    const long long next = row + stride;
    const __nv_bfloat16* next_src = next < rows ? a.x + next * a.row_stride : nullptr;
    if (DUAL) {
      warp_row_plain<BITS, NK, NG, GROUP, true>(a, p, oc, xs, bar, row, nullptr, wsm, bsm);
      __syncwarp();
      warp_row_plain<BITS, 0, NG, GROUP, false>(a, a.p2, oc2, xs, bar, row, next_src, wsm, bsm);
    } else {
      warp_row_plain<BITS, NK, NG, GROUP, false>(a, p, oc, xs, bar, row, next_src, wsm, bsm);
    }
  }
}

// One row of the rotating walk, staged in `xs` (see the kernel below).  `next_src`: the row to bring into the
// slot after the second pass (nullptr: none).  TO_SLOT as in warp_row_plain: the slot is kept and the norm
// output takes the row's place in it.
template <int BITS, int NK, int NG, bool GROUP, bool TO_SLOT>
__device__ __forceinline__ void warp_row_rot(const WarpFwdArgs& a, const PackedDev& p, const int (&oc)[kWarpOutPerLane],
                                             __nv_bfloat16* xs, uint64_t* bar, long long row,
                                             const __nv_bfloat16* next_src, const float* wsm, const float* bsm) {
  using C = CodeTraits<BITS>;
  constexpr int NSEG = C::kSeg;
  constexpr int UPL = NG / NSEG;
  constexpr bool NORM = NK != 0;
  constexpr bool ln = NK == 2;
  const int D = p.cols;
  const int segw = D / NSEG;
  const int U = segw >> 3;                  // a multiple of 32 here: a warp is wholly inside or outside a unit round
  const int k = p.n_channels;
  const int nrot = p.rotate;
  const int lane = threadIdx.x & 31;
  const int G = GROUP ? (D >> 7) : 1;
  const float qmax = static_cast<float>(C::kHi);
  const float inv_d = 1.0f / static_cast<float>(D);
  const uint32_t row_bytes = static_cast<uint32_t>(D) * 2u;
  {
    float ov[kWarpOutPerLane];
#pragma unroll
    for (int q = 0; q < kWarpOutPerLane; ++q) {
      ov[q] = 0.f;
      if (oc[q] >= 0) {
        const __nv_bfloat16 o = xs[oc[q]];
        p.out_value[row * k + lane + 32 * q] = o;
        ov[q] = __bfloat162float(o);
        xs[oc[q]] = __float2bfloat16_rn(0.f);
      }
    }
    __syncwarp();
    // ---- first pass over the staged row: statistics of the norm
    float mean = 0.f, rstd = 0.f;
    if (NORM) {
      if (ln) {
        float s1 = 0.f;
#pragma unroll
        for (int r = 0; r < NG; ++r) {
          if (32 * (r / NSEG) >= U) continue;            // register groups beyond the row (uniform over the warp)
          float f[8];
          load8<__nv_bfloat16>(xs, (r % NSEG) * segw + ((lane + 32 * (r / NSEG)) << 3), f);
#pragma unroll
          for (int e = 0; e < 8; ++e) s1 += f[e];
        }
#pragma unroll
        for (int q = 0; q < kWarpOutPerLane; ++q) s1 += ov[q];
        mean = warp_sum(s1) * inv_d;
      }
      float ss = 0.f;
#pragma unroll
      for (int r = 0; r < NG; ++r) {
        if (32 * (r / NSEG) >= U) continue;
        float f[8];
        load8<__nv_bfloat16>(xs, (r % NSEG) * segw + ((lane + 32 * (r / NSEG)) << 3), f);
#pragma unroll
        for (int e = 0; e < 8; ++e) { const float c = ln ? f[e] - mean : f[e]; ss = fmaf(c, c, ss); }
      }
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q)
        if (oc[q] >= 0) ss += ln ? ((ov[q] - mean) * (ov[q] - mean) - mean * mean) : ov[q] * ov[q];
      ss = warp_sum(ss);
      rstd = 1.0f / sqrtf(ss * inv_d + a.eps);
      if (lane == 0) {
        a.rstd[row] = rstd;
        if (ln) a.mean[row] = mean;
      }
    }
    // ---- second pass: norm output, rotation
    unsigned char* codes_row = p.codes + row * (static_cast<long long>(D) * BITS / 8);
    __nv_bfloat16* yrow = NORM ? a.y + row * a.row_stride : nullptr;
    float rot[NG][8];
    float amax = 0.f;
    float ginv[GROUP ? NG : 1];
#pragma unroll
    for (int iu = 0; iu < UPL; ++iu) {
      const int u = lane + 32 * iu;
      if (32 * iu >= U) {
        // a unit round beyond the row: nothing to read, rotate or store; its registers quantise to nothing
#pragma unroll
        for (int s = 0; s < NSEG; ++s) {
          if (GROUP) ginv[GROUP ? iu * NSEG + s : 0] = 0.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) rot[iu * NSEG + s][e] = 0.f;
        }
        continue;
      }
#pragma unroll
      for (int s = 0; s < NSEG; ++s) {
        const int col = s * segw + (u << 3);
        float f[8];
        load8<__nv_bfloat16>(xs, col, f);
        if (NORM) {
          float y[8], wv[8];
          load8_split(wsm, D, col, wv);
          if (ln) {
            float bv[8];
            load8_split(bsm, D, col, bv);
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = (f[e] - mean) * rstd * wv[e] + bv[e];
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = f[e] * rstd * wv[e];
          }
          store8<__nv_bfloat16>(yrow, col, y);
          if (TO_SLOT) store8<__nv_bfloat16>(xs, col, y);      // the norm output takes the row's place in the slot
        }
        rotate_group(f, nrot, lane);
        float a8 = absmax8(f);
        if (GROUP) {
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) a8 = fmaxf(a8, __shfl_xor_sync(0xffffffffu, a8, o));
          ginv[GROUP ? iu * NSEG + s : 0] = a8;
        } else {
          amax = fmaxf(amax, a8);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) rot[iu * NSEG + s][e] = f[e];
      }
      if (NORM && (iu & 1)) asm volatile("" ::: "memory");
    }
    __syncwarp();
    if (!TO_SLOT && lane == 0 && next_src) {
      fence_proxy_async();
      mbar_expect_tx(bar, row_bytes);
      bulk_g2s(xs, next_src, row_bytes, bar);
    }
    float inv_row = 1.f;
    if constexpr (GROUP) {
      group_scales<BITS, NG>(ginv, p.scales + row * G, segw, U, lane);
    } else {
      amax = warp_max(amax);
      const bool live = amax > 0.f;
      inv_row = live ? __fdiv_rn(qmax, amax) : 1.f;
      if (lane == 0) p.scales[row] = live ? __fdiv_rn(amax, qmax) : 1.f;
    }
#pragma unroll
    for (int iu = 0; iu < UPL; ++iu) {
      if (32 * iu >= U) continue;
      PackAcc<BITS> acc;
#pragma unroll
      for (int s = 0; s < NSEG; ++s) acc.add(rot[iu * NSEG + s], GROUP ? ginv[GROUP ? iu * NSEG + s : 0] : inv_row, s);
      *reinterpret_cast<uint2*>(codes_row + ((lane + 32 * iu) << 3)) = acc.done();
    }
    if (NORM) {
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q) {
        if (oc[q] >= 0) {
          const int cs = split_index(oc[q], D);
          const float y = ln ? ((ov[q] - mean) * rstd * wsm[cs] + bsm[cs]) : (ov[q] * rstd * wsm[cs]);
          yrow[oc[q]] = __float2bfloat16_rn(y);
          if (TO_SLOT) xs[oc[q]] = __float2bfloat16_rn(y);
        }
      }
    }
  }
}

// The same walk with a block Walsh-Hadamard rotation (block <= 256) before quantisation.  A warp holds 256
// consecutive channels of every segment (lane l: channels 8l..8l+7 of the window), so the butterflies of
// strides 1, 2, 4 run inside a lane and those of strides 8..128 through shuffles (rotate_group).  The row
// statistics of the norm are taken in a first pass over the staged row; the second pass writes the norm
// output of a group, rotates the group in place and keeps it in registers as fp32 (per-token scale: the
// row's absmax has to be known before any code can be written) or quantises it at once (group scales: a
// group's absmax lives in one half-warp).  The slot is handed back after the second pass.
template <int BITS, int NK, int NG, bool GROUP, bool DUAL>
__global__ void __launch_bounds__(kWarpRotThreads, 1) fwd_n_warp_rot_kernel(const __grid_constant__ WarpFwdArgs a) {
  using C = CodeTraits<BITS>;
  constexpr int NSEG = C::kSeg;
  constexpr int UPL = NG / NSEG;
  constexpr bool NORM = NK != 0;
  constexpr bool ln = NK == 2;
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  const int D = p.cols;
  const int segw = D / NSEG;
  const int U = segw >> 3;                  // a multiple of 32 here: a warp is wholly inside or outside a unit round
  const int k = p.n_channels;
  const int nrot = p.rotate;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
  const int G = GROUP ? (D >> 7) : 1;
  const float qmax = static_cast<float>(C::kHi);
  const float inv_d = 1.0f / static_cast<float>(D);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  int* chan = reinterpret_cast<int*>(smem + a.off_chan);
  float* wsm = reinterpret_cast<float*>(smem + a.off_wsm);
  float* bsm = reinterpret_cast<float*>(smem + a.off_bsm);
  // two slots per warp: the row after this one is already travelling while this one is rotated
  unsigned char* slots = smem + a.off_slots + static_cast<size_t>(warp) * 2u * a.slot_bytes;
  uint64_t* bar2 = &bars[2 * warp];
  const uint32_t row_bytes = static_cast<uint32_t>(D) * 2u;
  const long long rows = p.rows, stride = static_cast<long long>(gridDim.x) * W;
  long long row = static_cast<long long>(blockIdx.x) * W + warp;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2 * W; ++i) mbar_init(&bars[i], 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (lane == 0) {
    for (int s = 0; s < 2; ++s) {
      const long long r = row + s * stride;
      if (r < rows) {
        mbar_expect_tx(&bar2[s], row_bytes);
        bulk_g2s(slots + s * a.slot_bytes, a.x + r * a.row_stride, row_bytes, &bar2[s]);
      }
    }
  }
  for (int j = threadIdx.x; j < k; j += blockDim.x) chan[j] = p.channels[j];
  int* chan2 = reinterpret_cast<int*>(smem + a.off_chan2);
  if (DUAL)
    for (int j = threadIdx.x; j < a.p2.n_channels; j += blockDim.x) chan2[j] = a.p2.channels[j];
  if (NORM) {
    const float plus = a.kind == HYC_NORM_RMS_GEMMA ? 1.f : 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      wsm[split_index(c, D)] = (a.param_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.weight)[c])
                                             : static_cast<const float*>(a.weight)[c]) + plus;
      if (ln)
        bsm[split_index(c, D)] = a.param_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.bias)[c])
                                              : static_cast<const float*>(a.bias)[c];
    }
  }
  __syncthreads();
  int oc[kWarpOutPerLane];
#pragma unroll
  for (int q = 0; q < kWarpOutPerLane; ++q) oc[q] = (lane + 32 * q) < k ? chan[lane + 32 * q] : -1;
  int oc2[kWarpOutPerLane];
#pragma unroll
  for (int q = 0; q < kWarpOutPerLane; ++q) oc2[q] = (DUAL && (lane + 32 * q) < a.p2.n_channels) ? chan2[lane + 32 * q] : -1;

  uint32_t ph = 0;
  int st = 0;
  for (; row < rows; row += stride) {
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(slots + st * a.slot_bytes);
    uint64_t* bar = &bar2[st];
    if (!mbar_wait_bounded(bar, ph, a.wait_cycles)) {
      if (lane == 0 && p.status) atomicOr(p.status, kStatusWaitExpired);
      // the copy into the other slot may still be in flight: give it a bounded chance to land
      if (row + stride < rows) (void)mbar_wait_bounded(&bar2[st ^ 1], st ? ph ^ 1u : ph, a.wait_cycles);
      return;
    }
    const long long next = row + 2 * stride;
    const __nv_bfloat16* next_src = next < rows ? a.x + next * a.row_stride : nullptr;
    if (DUAL) {
      warp_row_rot<BITS, NK, NG, GROUP, true>(a, p, oc, xs, bar, row, nullptr, wsm, bsm);
      __syncwarp();
      warp_row_rot<BITS, 0, NG, GROUP, false>(a, a.p2, oc2, xs, bar, row, next_src, wsm, bsm);
    } else {
      warp_row_rot<BITS, NK, NG, GROUP, false>(a, p, oc, xs, bar, row, next_src, wsm, bsm);
    }
    if (st) ph ^= 1u;
    st ^= 1;
  }
}

// ------------------------------------------------------------------ host: eligibility and launch

struct WarpPlan {
  bool ok;
  int ng;          // register groups per lane (instantiated: 2, 4, 8, 16)
  int warps, grid, threads;
  bool rot, dual;
  uint32_t off_chan2;
  uint32_t off_chan, off_wsm, off_bsm, off_slots, slot_bytes, total;
};

// bf16 rows in the plain layout, at most 16 register groups per lane and 128 outlier channels; a rotation
// block of at most 256 channels that divides the segment width, with every lane of the warp in use
// `q2`: second record for the norm output (two-record variant), or nullptr; it must share the first record's
// bit width, scale grouping and rotation
inline WarpPlan plan_warp_fwd(const hyc_packed* q, const hyc_dense* x, bool norm, bool ln, const hyc_packed* q2 = nullptr) {
  WarpPlan w;
  memset(&w, 0, sizeof(w));
  if (q2) {
    if (!norm || q2->mode != HYC_MODE_N || q2->bits != q->bits || q2->group != q->group || q2->rotate != q->rotate ||
        q2->cols != q->cols || q2->rows != q->rows || q2->n_channels > 32 * kWarpOutPerLane)
      return w;
    if (q2->rotate && q->rows > 8192) return w;      // with a rotation the pair pays off for few rows only
    w.dual = true;
  }
  if (q->mode != HYC_MODE_N || x->dtype != HYC_BF16 || x->chunks != 1) return w;
  if (q->rotate && (q->rotate > 256 || (q->cols / (8 / q->bits)) % 256 != 0)) return w;
  if (q->bits != 2 && q->bits != 4 && q->bits != 8) return w;
  if (q->n_channels > 32 * kWarpOutPerLane) return w;
  if (g_tune_threads || g_tune_stages || g_tune_ctas) return w;     // explicit tuning addresses the CTA-per-row kernels
  const int D = q->cols, nseg = 8 / q->bits;
  const int U = D / nseg / 8;
  if (q->group && (D / nseg) % 128 != 0) return w;
  const int upl = (U + 31) / 32;
  int ng = nseg;
  while (ng < upl * nseg) ng *= 2;
  if (ng > 16) return w;
  if (ng < 2) ng = 2;
  w.ng = ng;
  uint32_t off = 64 * 8;                                   // one mbarrier per warp
  auto take = [&](uint32_t bytes) { uint32_t o = off; off = align_up(off + bytes, 16); return o; };
  w.off_chan = take((q->n_channels > 0 ? q->n_channels : 1) * 4);
  w.off_chan2 = take((q2 && q2->n_channels > 0 ? q2->n_channels : 1) * 4);
  if (norm) w.off_wsm = take(D * 4);
  if (ln) w.off_bsm = take(D * 4);
  off = align_up(off, 128);
  w.off_slots = off;
  w.slot_bytes = align_up(static_cast<uint32_t>(D) * 2u, 128);
  w.rot = q->rotate != 0;
  w.threads = w.rot ? kWarpRotThreads : kWarpKernelThreads;
  const int ctas = w.rot ? 1 : kWarpKernelCtasPerSm;
  w.warps = w.threads / 32;
  w.total = off + w.slot_bytes * w.warps * (w.rot ? 2 : 1);
  if (w.total > (ctas == 1 ? kSmemPerCtaMax - 1024 : kSmemBudget / ctas)) return w;
  long long grid = static_cast<long long>(sm_count()) * ctas;
  const long long need = (q->rows + w.warps - 1) / w.warps;
  if (grid > need) grid = need;
  w.grid = static_cast<int>(grid);
  w.ok = true;
  return w;
}

template <int BITS>
int launch_fwd_warp_bits(const WarpFwdArgs& a, const WarpPlan& w, bool norm, cudaStream_t stream) {
#define HYC_WARP_LAUNCH(NK, NG, GROUP)                                                          \
  {                                                                                             \
    if constexpr (NG >= 8 / BITS) {                                                             \
      if (w.rot) {                                                                              \
        if (w.dual) {                                                                           \
          if constexpr (NK != 0) {                                                              \
            auto kern = fwd_n_warp_rot_kernel<BITS, NK, NG, GROUP, true>;                       \
            int rc = set_smem(kern, w.total);                                                   \
            if (rc) return rc;                                                                  \
            kern<<<w.grid, w.threads, w.total, stream>>>(a); HYC_LAUNCHED();                    \
          } else {                                                                              \
            return HYC_ERR_SHAPE;                                                               \
          }                                                                                     \
        } else {                                                                                \
          auto kern = fwd_n_warp_rot_kernel<BITS, NK, NG, GROUP, false>;                        \
          int rc = set_smem(kern, w.total);                                                     \
          if (rc) return rc;                                                                    \
          kern<<<w.grid, w.threads, w.total, stream>>>(a); HYC_LAUNCHED();                      \
        }                                                                                       \
      } else if (w.dual) {                                                                      \
        if constexpr (NK != 0) {                                                                \
          auto kern = fwd_n_warp_dual_kernel<BITS, NK, NG, GROUP>;                             \
          int rc = set_smem(kern, w.total);                                                     \
          if (rc) return rc;                                                                    \
          kern<<<w.grid, w.threads, w.total, stream>>>(a); HYC_LAUNCHED();                      \
        } else {                                                                                \
          return HYC_ERR_SHAPE;                                                                 \
        }                                                                                       \
      } else {                                                                                  \
        auto kern = fwd_n_warp_kernel<BITS, NK, NG, GROUP>;                              \
        int rc = set_smem(kern, w.total);                                                       \
        if (rc) return rc;                                                                      \
        kern<<<w.grid, w.threads, w.total, stream>>>(a); HYC_LAUNCHED();                        \
      }                                                                                         \
    } else {                                                                                    \
      return HYC_ERR_SHAPE;                                                                     \
    }                                                                                           \
  }
#define HYC_WARP_NG(NK, GROUP)                                                                  \
  switch (w.ng) {                                                                               \
    case 2: HYC_WARP_LAUNCH(NK, 2, GROUP) break;                                                \
    case 4: HYC_WARP_LAUNCH(NK, 4, GROUP) break;                                                \
    case 8: HYC_WARP_LAUNCH(NK, 8, GROUP) break;                                                \
    default: HYC_WARP_LAUNCH(NK, 16, GROUP) break;                                              \
  }
  const int nk = !norm ? 0 : a.kind == HYC_NORM_LAYER ? 2 : 1;
  if (nk == 2) {
    if (a.p.group) { HYC_WARP_NG(2, true) } else { HYC_WARP_NG(2, false) }
  } else if (nk == 1) {
    if (a.p.group) { HYC_WARP_NG(1, true) } else { HYC_WARP_NG(1, false) }
  } else {
    if (a.p.group) { HYC_WARP_NG(0, true) } else { HYC_WARP_NG(0, false) }
  }
#undef HYC_WARP_NG
#undef HYC_WARP_LAUNCH
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? HYC_OK : cuda_fail(e, "fwd_n_warp_kernel launch");
}

int launch_fwd_warp_b2(const WarpFwdArgs& a, const WarpPlan& w, bool norm, cudaStream_t stream);
int launch_fwd_warp_b4(const WarpFwdArgs& a, const WarpPlan& w, bool norm, cudaStream_t stream);
int launch_fwd_warp_b8(const WarpFwdArgs& a, const WarpPlan& w, bool norm, cudaStream_t stream);

}  // namespace hyc
