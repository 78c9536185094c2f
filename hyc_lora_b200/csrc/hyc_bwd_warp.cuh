// Warp-per-row consumers of a record (rows of up to 4096 channels; channel-mode records, and reference-mode
// records without a low-rank part): decompress, decompress + norm backward with a frozen norm weight and a bf16
// gradient, decompress + SiLU / GELU backward with a bf16 gradient.
//
// Same walk as the warp-per-row forward kernel: a warp owns its rows; the packed codes (and the gradient
// row) of a row land in the warp's own shared-memory slot by bulk asynchronous copies on the warp's own
// mbarrier; reductions are warp shuffles, and there is no CTA barrier in the row loop.  The decompress
// moves the codes into registers and hands the slot straight back to the copy engine; the norm backward
// makes its two passes (the two row sums, then the result) and the activation backward its one pass over the
// slot itself, in short rolled loops on packed fp32 pairs, and rebuild the values from the codes there.
// Outliers (the outlier channels of a channel-mode record, the pool entries of a reference-mode row) are
// streamed as the zero their code encodes and put right afterwards by the lanes that look after them (after the
// inverse rotation they are cleared first, the correction assumes a zero).  Arithmetic per element is that of
// the CTA-per-row kernels in hyc_bwd_fast.cuh, which keep the product backward, fp32 gradients, rotated
// records and wider rows.  (A first warp-per-row activation backward held the whole row in registers, spilled and
// measured slower than those; the rolled loop over the slot needs few registers.)
#pragma once
#include <stdlib.h>

#include <type_traits>

#include "hyc_bwd_fast.cuh"
#include "hyc_fwd_warp.cuh"

namespace hyc {

struct WarpBwdArgs {
  PackedDev p, p2;
  const __nv_bfloat16* g;     // upstream gradient rows [rows, D] (activation / norm backward)
  __nv_bfloat16* out1;        // decompress: reconstruction; activation: dx1; norm: dx
  __nv_bfloat16* out2;        // product: dx2
  long long out_stride;       // elements between rows of out1 (decompress follows the caller's layout)
  int kind, ref_compat_c2, param_bf16;
  const void* weight;
  const float* rstd;
  const float* mean;
  uint32_t off_chan, off_chan2, off_wsm, off_slots, slot_bytes, off_c2, off_g;
  uint32_t tx_pad;
  long long wait_cycles;
};

// what every consumer sets up once per CTA and per lane
template <int BITS, int NG>
struct WarpRowCtx {
  static constexpr int NSEG = 8 / BITS;
  static constexpr int UPL = NG / NSEG;
  int D, segw, U, k, lane, warp, W;
  unsigned char* slot;
  uint64_t* bar;
  int* chan;
  long long rows, stride, row;
  uint32_t ph;
  int oc[kWarpOutPerLane];

  __device__ __forceinline__ void init(const WarpBwdArgs& a, unsigned char* smem) {
    D = a.p.cols; segw = D / NSEG; U = segw >> 3; k = a.p.n_channels;
    lane = threadIdx.x & 31; warp = threadIdx.x >> 5; W = blockDim.x >> 5;
    slot = smem + a.off_slots + static_cast<size_t>(warp) * a.slot_bytes;
    bar = reinterpret_cast<uint64_t*>(smem) + warp;
    chan = reinterpret_cast<int*>(smem + a.off_chan);
    rows = a.p.rows; stride = static_cast<long long>(gridDim.x) * W;
    row = static_cast<long long>(blockIdx.x) * W + warp;
    ph = 0;
    if (threadIdx.x == 0) {
      for (int i = 0; i < W; ++i) mbar_init(reinterpret_cast<uint64_t*>(smem) + i, 1);
      fence_barrier_init();
    }
    __syncthreads();
  }
  // column of register group r of this lane
  __device__ __forceinline__ int col(int r) const { return (r % NSEG) * segw + ((lane + 32 * (r / NSEG)) << 3); }
  __device__ __forceinline__ bool live(int r) const { return (lane + 32 * (r / NSEG)) < U; }
  __device__ __forceinline__ void lanes_channels() {
#pragma unroll
    for (int q = 0; q < kWarpOutPerLane; ++q) oc[q] = (lane + 32 * q) < k ? chan[lane + 32 * q] : -1;
  }
};

// one row's bytes into the warp's slot: codes (and the second operand's), then the gradient row
__device__ __forceinline__ void warp_issue_row(const WarpBwdArgs& a, unsigned char* slot, uint64_t* bar, long long row,
                                               uint32_t cb, bool second, bool grad, int D) {
  const uint32_t total = cb + (second ? cb : 0u) + (grad ? static_cast<uint32_t>(D) * 2u : 0u);
  mbar_expect_tx(bar, total + a.tx_pad);
  bulk_g2s(slot, a.p.codes + row * cb, cb, bar);
  if (second) bulk_g2s(slot + a.off_c2, a.p2.codes + row * cb, cb, bar);
  if (grad) bulk_g2s(slot + a.off_g, a.g + row * D, static_cast<uint32_t>(D) * 2u, bar);
}

// the values of register group (iu, s): (code - offset) * scale, rotated back when the record is rotated,
// rounded to bf16 when ROUND (what a reconstruction holds)
template <int BITS, bool ROT, bool ROUND>
__device__ __forceinline__ void warp_rebuild8(const uint2& cw, int s, float sc, int nrot, int lane, float (&f)[8]) {
  dequant8<BITS>(cw, s, sc, f);
  if (ROT) rotate_group(f, nrot, lane);
  if (ROUND) round_bf16x8(f);
}

// The same values as four fp32 pairs (channels 2i, 2i + 1 of the group), not rotated, rounded to bf16: two
// channels per instruction on the packed fp32 pipe.  `sc`: the scale of each pair's channels.
template <int BITS>
__device__ __forceinline__ void warp_rebuild8_pairs(const uint2& cw, int s, const f32x2 (&sc)[4], f32x2 (&f)[4]) {
  using C = CodeTraits<BITS>;
  uint32_t w[2] = {cw.x, cw.y};
  float bias;
  if (BITS == 8) {
    w[0] ^= 0x80808080u; w[1] ^= 0x80808080u;  // two's complement -> offset 128
    bias = 8388608.f + 128.f;
  } else {
    const uint32_t m = 0x01010101u * C::kMask;
    w[0] = (w[0] >> (s * BITS)) & m;
    w[1] = (w[1] >> (s * BITS)) & m;
    bias = 8388608.f + static_cast<float>(C::kOff);
  }
  const f32x2 bias2 = f2_make(bias, bias);
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const f32x2 lo = f2_make(__uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7650)),
                             __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7651)));
    const f32x2 hi = f2_make(__uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7652)),
                             __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7653)));
    const f32x2 a = f2_mul(f2_sub(lo, bias2), sc[2 * i]), b = f2_mul(f2_sub(hi, bias2), sc[2 * i + 1]);
    float a0, a1, b0, b1;
    f2_split(a, a0, a1);
    f2_split(b, b0, b1);
    const uint32_t pa = pack_bf16x2(a0, a1), pb = pack_bf16x2(b0, b1);
    f[2 * i] = f2_make(__uint_as_float(pa << 16), __uint_as_float(pa & 0xffff0000u));
    f[2 * i + 1] = f2_make(__uint_as_float(pb << 16), __uint_as_float(pb & 0xffff0000u));
  }
}

// the 8 table entries of load8_split as four pairs
__device__ __forceinline__ void load8_split_pairs(const float* table, int D, int col, f32x2 (&f)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(table + ((col >> 3) << 2));
  const float4 b = *reinterpret_cast<const float4*>(table + (D >> 1) + ((col >> 3) << 2));
  f[0] = f2_make(a.x, a.y); f[1] = f2_make(a.z, a.w);
  f[2] = f2_make(b.x, b.y); f[3] = f2_make(b.z, b.w);
}

// ------------------------------------------------------------------ decompress

// KIND 0: channel-mode record; 1: rotated channel-mode record; 2: reference-mode record without a low-rank part
// (static scales: an fp32 table per channel, or one per row; the row's element outliers -- stored values with
// their columns in the pool -- overwrite the zeros their codes gave, as the outlier channels' originals do).
template <int BITS, int NG, int KIND>
__global__ void __launch_bounds__(kWarpKernelThreads, 2) decompress_n_warp_kernel(const __grid_constant__ WarpBwdArgs a) {
  using Ctx = WarpRowCtx<BITS, NG>;
  constexpr int NSEG = Ctx::NSEG, UPL = Ctx::UPL;
  constexpr bool ROT = KIND == 1, REF = KIND == 2;
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  Ctx c;
  c.init(a, smem);
  const uint32_t cb = static_cast<uint32_t>(c.D) * BITS / 8;
  if (c.lane == 0 && c.row < c.rows) warp_issue_row(a, c.slot, c.bar, c.row, cb, false, false, c.D);
  float* csc = reinterpret_cast<float*>(smem + a.off_chan2);   // REF, per-channel scale: fp32 table (split halves)
  const bool per_channel = REF && p.scale_kind == kScaleChannel;
  if (REF) {
    if (per_channel)
      for (int ch = threadIdx.x; ch < c.D; ch += blockDim.x) csc[split_index(ch, c.D)] = __bfloat162float(p.scale[ch]);
  } else {
    for (int j = threadIdx.x; j < c.k; j += blockDim.x) c.chan[j] = max(0, min(c.D - 1, p.channels[j]));
  }
  __syncthreads();
  if (!REF) c.lanes_channels();
  const int G = (!REF && p.group) ? (c.D >> 7) : 1;
  for (; c.row < c.rows; c.row += c.stride, c.ph ^= 1u) {
    const long long row = c.row;
    // the stored originals of the outlier channels, fetched before the wait
    __nv_bfloat16 ov[kWarpOutPerLane];
    uint2 meta = make_uint2(0u, 0u);
    const float* sc_row = p.scales + row * G;
    float sc_tok = 0.f;
    if (REF) {
      meta = p.row_meta[row];
      if (!per_channel) sc_tok = __bfloat162float(p.scale[p.scale_kind == kScaleToken ? row % p.seq : 0]);
    } else {
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q)
        ov[q] = c.oc[q] >= 0 ? p.out_value[row * c.k + c.lane + 32 * q] : __float2bfloat16_rn(0.f);
      sc_tok = p.group ? 0.f : __ldg(sc_row);
    }
    if (!mbar_wait_bounded(c.bar, c.ph, a.wait_cycles)) {
      if (c.lane == 0 && p.status) atomicOr(p.status, kStatusWaitExpired);
      return;
    }
    uint2 cw[UPL];
#pragma unroll
    for (int iu = 0; iu < UPL; ++iu)
      cw[iu] = (c.lane + 32 * iu) < c.U ? *reinterpret_cast<const uint2*>(c.slot + ((c.lane + 32 * iu) << 3)) : make_uint2(0u, 0u);
    __syncwarp();
    const long long next = row + c.stride;
    if (c.lane == 0 && next < c.rows) {
      fence_proxy_async();
      warp_issue_row(a, c.slot, c.bar, next, cb, false, false, c.D);
    }
    __nv_bfloat16* orow = a.out1 + row * a.out_stride;
#pragma unroll
    for (int r = 0; r < NG; ++r) {
      const int col = c.col(r);
      float f[8];
      if (REF) {
        dequant8<BITS>(cw[r / NSEG], r % NSEG, per_channel ? 1.f : sc_tok, f);
        if (per_channel) {
          float sc[8];
          load8_split(csc, c.D, min(col, c.D - 8), sc);
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] *= sc[e];
        }
      } else {
        const float sc = p.group ? __ldg(sc_row + (min(col, c.D - 8) >> 7)) : sc_tok;
        warp_rebuild8<BITS, ROT, false>(cw[r / NSEG], r % NSEG, sc, p.rotate, c.lane, f);
      }
      if (c.live(r)) store8<__nv_bfloat16>(orow, col, f);
    }
    __syncwarp();   // the vector stores come before the stored originals (other lanes)
    if (REF) {
      for (uint32_t j = c.lane; j < meta.y; j += 32) {
        const uint32_t e = p.pool[meta.x + j];
        reinterpret_cast<uint16_t*>(orow)[e & 0xffffu] = static_cast<uint16_t>(e >> 16);
      }
    } else {
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q)
        if (c.oc[q] >= 0) orow[c.oc[q]] = ov[q];
    }
  }
}

// ------------------------------------------------------------------ norm backward (frozen weight)

constexpr int kNormBwdWarpThreads = 640;    // 20 warps, one CTA per SM: the slots of 20 rows fill the shared memory

// Two passes over the row (the two row sums, then the result) read the codes and the gradient row from
// the warp's slot both times, in short rolled loops, instead of holding them in registers: few registers,
// twenty warps per SM to cover the arithmetic latencies, and the slot goes back to the copy engine when
// the row is done (the other warps keep the memory system busy meanwhile).  Every step of both passes runs on
// packed fp32 pairs, and the loops are compiled per launch-wide fact (which kind of scale; every lane owns a
// unit in every round), so that no test of those sits between the segments of a unit.
//
// REF: a reference-mode record without a low-rank part.  Its values are (code - offset) * static scale rounded
// to bf16 (per channel: an fp32 table in shared memory; per token / per tensor: one scale per row); the row's
// element outliers (their code is the zero code, so the streamed passes see exactly 0 there) come from the pool
// and are put right by the lanes, entry by entry, after each pass -- the place the outlier channels' stored
// originals take in a channel-mode record.
template <int BITS, bool REF, bool LN>
__global__ void __launch_bounds__(kNormBwdWarpThreads, 1) norm_bwd_n_warp_kernel(const __grid_constant__ WarpBwdArgs a) {
  constexpr int NSEG = 8 / BITS;
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  WarpRowCtx<BITS, NSEG> c;
  c.init(a, smem);
  const int D = c.D;
  const int upl = (c.U + 31) >> 5;
  const bool full = (c.U & 31) == 0;
  const uint32_t cb = static_cast<uint32_t>(D) * BITS / 8;
  if (c.lane == 0 && c.row < c.rows) warp_issue_row(a, c.slot, c.bar, c.row, cb, false, true, D);
  float* wsm = reinterpret_cast<float*>(smem + a.off_wsm);
  float* csc = reinterpret_cast<float*>(smem + a.off_chan2);   // REF, per-channel scale: fp32 table (split halves)
  const bool per_channel = REF && p.scale_kind == kScaleChannel;
  const float plus = a.kind == HYC_NORM_RMS_GEMMA ? 1.f : 0.f;
  if (!REF)
    for (int j = threadIdx.x; j < c.k; j += blockDim.x) c.chan[j] = max(0, min(D - 1, p.channels[j]));
  for (int ch = threadIdx.x; ch < D; ch += blockDim.x) {
    wsm[split_index(ch, D)] = (a.param_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.weight)[ch])
                                            : static_cast<const float*>(a.weight)[ch]) + plus;
    if (per_channel) csc[split_index(ch, D)] = __bfloat162float(p.scale[ch]);
  }
  __syncthreads();
  if (!REF) c.lanes_channels();
  const int G = (!REF && p.group) ? (D >> 7) : 1;
  const float inv_d = 1.0f / static_cast<float>(D);
  const __nv_bfloat16* gs = reinterpret_cast<const __nv_bfloat16*>(c.slot + a.off_g);
  // 0: one scale per row; 1: one per 128 channels (channel mode); 2: one per channel (reference mode)
  const int scale_mode = REF ? (per_channel ? 2 : 0) : (p.group ? 1 : 0);
  for (; c.row < c.rows; c.row += c.stride, c.ph ^= 1u) {
    const long long row = c.row;
    const float rstd = __ldg(a.rstd + row);
    const float mean = LN ? __ldg(a.mean + row) : 0.f;
    float ov[kWarpOutPerLane];
    uint2 meta = make_uint2(0u, 0u);
    const float* sc_row = p.scales + row * G;
    float sc_tok = 0.f;
    if (REF) {
      meta = p.row_meta[row];
      if (!per_channel) sc_tok = __bfloat162float(p.scale[p.scale_kind == kScaleToken ? row % p.seq : 0]);
    } else {
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q)
        ov[q] = c.oc[q] >= 0 ? __bfloat162float(p.out_value[row * c.k + c.lane + 32 * q]) : 0.f;
      sc_tok = p.group ? 0.f : __ldg(sc_row);
    }
    if (!mbar_wait_bounded(c.bar, c.ph, a.wait_cycles)) {
      if (c.lane == 0 && p.status) atomicOr(p.status, kStatusWaitExpired);
      return;
    }
    float gq[kWarpOutPerLane];
    if (!REF) {
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q) gq[q] = c.oc[q] >= 0 ? __bfloat162float(gs[c.oc[q]]) : 0.f;
    }
    // the values of one register group and what goes with them: x-hat, the gradient, the norm weight
    auto group_operands = [&](auto mode_c, const uint2& cw, int s, int col, f32x2 (&f)[4], f32x2 (&gv)[4], f32x2 (&wv)[4]) {
      constexpr int kMode = decltype(mode_c)::value;
      f32x2 sc4[4];
      if (kMode == 2) {
        load8_split_pairs(csc, D, col, sc4);
      } else {
        const float sg = kMode == 1 ? __ldg(sc_row + (col >> 7)) : sc_tok;
        sc4[0] = sc4[1] = sc4[2] = sc4[3] = f2_make(sg, sg);
      }
      warp_rebuild8_pairs<BITS>(cw, s, sc4, f);
      unpack_bf16x8_pairs(*reinterpret_cast<const uint4*>(gs + col), gv);
      load8_split_pairs(wsm, D, col, wv);
    };
    // ---- pass 1: the two row sums.  With x-hat = (x - mean) * rstd the first one is
    //   c1 = mean_d(x-hat * w dy) = rstd * (S1 - mean * S2) / D,   S1 = sum x * w dy,  S2 = sum w dy,
    // so the pass accumulates S1 and S2 from the rebuilt x itself (two fused multiply-adds per element).
    float s1 = 0.f, s2 = 0.f;
    auto pass1 = [&](auto mode_c, auto full_c) {
      f32x2 s1p = 0ull, s2p = 0ull;
#pragma unroll 2
      for (int iu = 0; iu < upl; ++iu) {
        const int u = c.lane + 32 * iu;
        if (decltype(full_c)::value || u < c.U) {
          const uint2 cw = *reinterpret_cast<const uint2*>(c.slot + (u << 3));
#pragma unroll
          for (int s = 0; s < NSEG; ++s) {
            f32x2 f[4], gv[4], wv[4];
            group_operands(mode_c, cw, s, s * c.segw + (u << 3), f, gv, wv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const f32x2 wd = f2_mul(wv[e], gv[e]);
              s1p = f2_fma(f[e], wd, s1p);
              s2p = f2_add(s2p, wd);
            }
          }
        }
      }
      float lo, hi;
      f2_split(s1p, lo, hi);
      s1 = lo + hi;
      f2_split(s2p, lo, hi);
      s2 = lo + hi;
    };
    using M0 = std::integral_constant<int, 0>;
    using M1 = std::integral_constant<int, 1>;
    using M2 = std::integral_constant<int, 2>;
    using T = std::true_type;
    using F = std::false_type;
    if (scale_mode == 0) { if (full) pass1(M0(), T()); else pass1(M0(), F()); }
    else if (REF) { if (full) pass1(M2(), T()); else pass1(M2(), F()); }
    else { if (full) pass1(M1(), T()); else pass1(M1(), F()); }
    // what the streamed pass saw as the zero of its code: the outlier channels' stored originals, or the row's
    // element outliers from the pool
    if (REF) {
      for (uint32_t j = c.lane; j < meta.y; j += 32) {
        const uint32_t e = p.pool[meta.x + j];
        const int col = static_cast<int>(e & 0xffffu);
        s1 = fmaf(bf16_bits_to_float(e >> 16), wsm[split_index(col, D)] * __bfloat162float(gs[col]), s1);
      }
    } else {
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q)
        if (c.oc[q] >= 0) s1 = fmaf(ov[q], wsm[split_index(c.oc[q], D)] * gq[q], s1);
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    const float c1 = rstd * (s1 - mean * s2) * inv_d;
    const float c2 = (LN || a.ref_compat_c2) ? s2 * inv_d : 0.f;
    // ---- pass 2: dx = (w dy - (x-hat * c1 + c2)) * rstd = ka * w dy + kb * x + kc with three row constants
    const float ka = rstd, kb = -rstd * rstd * c1, kc = (mean * rstd * c1 - c2) * rstd;
    __nv_bfloat16* dxrow = a.out1 + row * D;
    auto pass2 = [&](auto mode_c, auto full_c) {
      const f32x2 ka2 = f2_make(ka, ka), kb2 = f2_make(kb, kb), kc2 = f2_make(kc, kc);
#pragma unroll 2
      for (int iu = 0; iu < upl; ++iu) {
        const int u = c.lane + 32 * iu;
        if (decltype(full_c)::value || u < c.U) {
          const uint2 cw = *reinterpret_cast<const uint2*>(c.slot + (u << 3));
#pragma unroll
          for (int s = 0; s < NSEG; ++s) {
            const int col = s * c.segw + (u << 3);
            f32x2 f[4], gv[4], wv[4];
            group_operands(mode_c, cw, s, col, f, gv, wv);
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float lo, hi;
              f2_split(f2_fma(ka2, f2_mul(wv[e], gv[e]), f2_fma(kb2, f[e], kc2)), lo, hi);
              o[e] = pack_bf16x2(lo, hi);
            }
            *reinterpret_cast<uint4*>(dxrow + col) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      }
    };
    if (scale_mode == 0) { if (full) pass2(M0(), T()); else pass2(M0(), F()); }
    else if (REF) { if (full) pass2(M2(), T()); else pass2(M2(), F()); }
    else { if (full) pass2(M1(), T()); else pass2(M1(), F()); }
    __syncwarp();   // the vector stores come before the results at the outliers (other lanes)
    if (REF) {
      for (uint32_t j = c.lane; j < meta.y; j += 32) {
        const uint32_t e = p.pool[meta.x + j];
        const int col = static_cast<int>(e & 0xffffu);
        dxrow[col] = __float2bfloat16_rn(fmaf(ka, wsm[split_index(col, D)] * __bfloat162float(gs[col]),
                                              fmaf(kb, bf16_bits_to_float(e >> 16), kc)));
      }
      __syncwarp();   // every lane is done with the slot
    }
    const long long next = row + c.stride;
    if (c.lane == 0 && next < c.rows) {
      fence_proxy_async();
      warp_issue_row(a, c.slot, c.bar, next, cb, false, true, D);
    }
    if (!REF) {
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q) {
        if (c.oc[q] >= 0)
          dxrow[c.oc[q]] = __float2bfloat16_rn(fmaf(ka, wsm[split_index(c.oc[q], D)] * gq[q], fmaf(kb, ov[q], kc)));
      }
    }
  }
}

// ------------------------------------------------------------------ activation backward (SiLU / GELU)

__device__ __forceinline__ float ex2_approx(float x) {   // what __expf evaluates after its scaling by log2(e)
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// silu'(x) * g for two channels: silu_grad_f's formula on packed fp32 pairs (the exponential and the reciprocal
// stay one channel at a time: they run on the special-function unit)
__device__ __forceinline__ f32x2 silu_grad_times_pairs(f32x2 x2, f32x2 g2) {
  const f32x2 one2 = f2_make(1.f, 1.f);
  float t0, t1;
  f2_split(f2_mul(x2, f2_make(-1.4426950408889634f, -1.4426950408889634f)), t0, t1);
  float d0, d1;
  f2_split(f2_add(f2_make(ex2_approx(t0), ex2_approx(t1)), one2), d0, d1);
  const f32x2 s2 = f2_make(__fdividef(1.f, d0), __fdividef(1.f, d1));
  return f2_mul(f2_mul(s2, f2_fma(x2, f2_sub(one2, s2), one2)), g2);
}

// dx = act'(x-hat) * g for bf16 gradients, rows of up to 4096 channels, records without rotation (channel mode)
// or reference-mode records without a low-rank part.  One pass over the warp's slot (codes + gradient row) in a
// short rolled loop, twenty warps per SM; the outliers are put right afterwards as in the norm backward.
template <int BITS, bool REF, bool GELU>
__global__ void __launch_bounds__(kNormBwdWarpThreads, 1) act_bwd_n_warp_kernel(const __grid_constant__ WarpBwdArgs a) {
  constexpr int NSEG = 8 / BITS;
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  WarpRowCtx<BITS, NSEG> c;
  c.init(a, smem);
  const int D = c.D;
  const int upl = (c.U + 31) >> 5;
  const bool full = (c.U & 31) == 0;
  const uint32_t cb = static_cast<uint32_t>(D) * BITS / 8;
  if (c.lane == 0 && c.row < c.rows) warp_issue_row(a, c.slot, c.bar, c.row, cb, false, true, D);
  float* csc = reinterpret_cast<float*>(smem + a.off_chan2);   // REF, per-channel scale: fp32 table (split halves)
  const bool per_channel = REF && p.scale_kind == kScaleChannel;
  if (REF) {
    if (per_channel)
      for (int ch = threadIdx.x; ch < D; ch += blockDim.x) csc[split_index(ch, D)] = __bfloat162float(p.scale[ch]);
  } else {
    for (int j = threadIdx.x; j < c.k; j += blockDim.x) c.chan[j] = max(0, min(D - 1, p.channels[j]));
  }
  __syncthreads();
  if (!REF) c.lanes_channels();
  const int G = (!REF && p.group) ? (D >> 7) : 1;
  const __nv_bfloat16* gs = reinterpret_cast<const __nv_bfloat16*>(c.slot + a.off_g);
  const int scale_mode = REF ? (per_channel ? 2 : 0) : (p.group ? 1 : 0);
  auto grad_of = [&](float x) { return GELU ? gelu_tanh_grad_f(x) : silu_grad_f(x); };
  for (; c.row < c.rows; c.row += c.stride, c.ph ^= 1u) {
    const long long row = c.row;
    float ov[kWarpOutPerLane];
    uint2 meta = make_uint2(0u, 0u);
    const float* sc_row = p.scales + row * G;
    float sc_tok = 0.f;
    if (REF) {
      meta = p.row_meta[row];
      if (!per_channel) sc_tok = __bfloat162float(p.scale[p.scale_kind == kScaleToken ? row % p.seq : 0]);
    } else {
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q)
        ov[q] = c.oc[q] >= 0 ? __bfloat162float(p.out_value[row * c.k + c.lane + 32 * q]) : 0.f;
      sc_tok = p.group ? 0.f : __ldg(sc_row);
    }
    if (!mbar_wait_bounded(c.bar, c.ph, a.wait_cycles)) {
      if (c.lane == 0 && p.status) atomicOr(p.status, kStatusWaitExpired);
      return;
    }
    float gq[kWarpOutPerLane];
    if (!REF) {
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q) gq[q] = c.oc[q] >= 0 ? __bfloat162float(gs[c.oc[q]]) : 0.f;
    }
    __nv_bfloat16* dxrow = a.out1 + row * D;
    auto pass = [&](auto mode_c, auto full_c) {
      constexpr int kMode = decltype(mode_c)::value;
#pragma unroll 2
      for (int iu = 0; iu < upl; ++iu) {
        const int u = c.lane + 32 * iu;
        if (decltype(full_c)::value || u < c.U) {
          const uint2 cw = *reinterpret_cast<const uint2*>(c.slot + (u << 3));
#pragma unroll
          for (int s = 0; s < NSEG; ++s) {
            const int col = s * c.segw + (u << 3);
            f32x2 sc4[4], f[4], gv[4];
            if (kMode == 2) {
              load8_split_pairs(csc, D, col, sc4);
            } else {
              const float sg = kMode == 1 ? __ldg(sc_row + (col >> 7)) : sc_tok;
              sc4[0] = sc4[1] = sc4[2] = sc4[3] = f2_make(sg, sg);
            }
            warp_rebuild8_pairs<BITS>(cw, s, sc4, f);
            unpack_bf16x8_pairs(*reinterpret_cast<const uint4*>(gs + col), gv);
            uint32_t o[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float lo, hi;
              if (GELU) {
                float x0, x1, g0, g1;
                f2_split(f[e], x0, x1);
                f2_split(gv[e], g0, g1);
                lo = gelu_tanh_grad_f(x0) * g0;
                hi = gelu_tanh_grad_f(x1) * g1;
              } else {
                f2_split(silu_grad_times_pairs(f[e], gv[e]), lo, hi);
              }
              o[e] = pack_bf16x2(lo, hi);
            }
            *reinterpret_cast<uint4*>(dxrow + col) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      }
    };
    using M0 = std::integral_constant<int, 0>;
    using M1 = std::integral_constant<int, 1>;
    using M2 = std::integral_constant<int, 2>;
    if (scale_mode == 0) { if (full) pass(M0(), std::true_type()); else pass(M0(), std::false_type()); }
    else if (REF) { if (full) pass(M2(), std::true_type()); else pass(M2(), std::false_type()); }
    else { if (full) pass(M1(), std::true_type()); else pass(M1(), std::false_type()); }
    __syncwarp();   // the vector stores come before the results at the outliers (other lanes)
    if (REF) {
      for (uint32_t j = c.lane; j < meta.y; j += 32) {
        const uint32_t e = p.pool[meta.x + j];
        const int col = static_cast<int>(e & 0xffffu);
        dxrow[col] = __float2bfloat16_rn(grad_of(bf16_bits_to_float(e >> 16)) * __bfloat162float(gs[col]));
      }
      __syncwarp();   // every lane is done with the slot
    }
    const long long next = row + c.stride;
    if (c.lane == 0 && next < c.rows) {
      fence_proxy_async();
      warp_issue_row(a, c.slot, c.bar, next, cb, false, true, D);
    }
    if (!REF) {
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q)
        if (c.oc[q] >= 0) dxrow[c.oc[q]] = __float2bfloat16_rn(grad_of(ov[q]) * gq[q]);
    }
  }
}

// ------------------------------------------------------------------ host: eligibility and launch

struct WarpBwdPlan {
  bool ok;
  int ng, grid, threads;
  uint32_t off_chan, off_chan2, off_wsm, off_slots, slot_bytes, off_c2, off_g, total;
};

// channel-mode record(s) of up to 16 register groups per lane and 128 outlier channels; a rotation block of
// at most 256 channels dividing a segment of whole 256-channel windows
// threads / ctas: CTA size and CTAs per SM of the kernel to be launched
inline WarpBwdPlan plan_warp_bwd(const hyc_packed* q, const hyc_packed* q2, bool grad, bool want_w,
                                 int threads = kWarpKernelThreads, int ctas = 2) {
  WarpBwdPlan w;
  memset(&w, 0, sizeof(w));
  static const bool off_env = getenv("HYC_BWD_WARP") && getenv("HYC_BWD_WARP")[0] == '0';
  // reference-mode records: the single-record consumers, without a low-rank part, columns that fit 16 bits
  const bool ref = q->mode == HYC_MODE_R;
  if (off_env || (ref && (q2 || q->lowrank || q->seq <= 0 || q->cols > 65535)) ||
      (!ref && q->mode != HYC_MODE_N) || (q2 && q2->mode != HYC_MODE_N))
    return w;
  if (q->bits != 2 && q->bits != 4 && q->bits != 8) return w;
  if (!ref && (q->n_channels > 32 * kWarpOutPerLane || (q2 && q2->n_channels > 32 * kWarpOutPerLane))) return w;
  if (g_tune_threads || g_tune_stages || g_tune_ctas) return w;
  const int D = q->cols, nseg = 8 / q->bits;
  if (!ref && q->rotate && (q->rotate > 256 || (D / nseg) % 256 != 0)) return w;
  if (!ref && q->group && (D / nseg) % 128 != 0) return w;
  const int U = D / nseg / 8;
  const int upl = (U + 31) / 32;
  int ng = nseg;
  while (ng < upl * nseg) ng *= 2;
  if (ng > 16) return w;
  if (ng < 2) ng = 2;
  w.ng = ng;
  uint32_t off = 64 * 8;
  auto take = [&](uint32_t bytes) { uint32_t o = off; off = align_up(off + bytes, 16); return o; };
  w.off_chan = take((!ref && q->n_channels > 0 ? q->n_channels : 1) * 4);
  // second channel list (product), or the per-channel scale table of a reference-mode record (fp32 [D])
  w.off_chan2 = take(ref ? (q->scale_kind == HYC_SCALE_CHANNEL ? static_cast<uint32_t>(D) * 4u : 16u)
                         : (q2 && q2->n_channels > 0 ? q2->n_channels : 1) * 4);
  if (want_w) w.off_wsm = take(D * 4);
  off = align_up(off, 128);
  w.off_slots = off;
  const uint32_t cb = align_up(static_cast<uint32_t>(D) * q->bits / 8, 128);
  w.off_c2 = cb;
  w.off_g = q2 ? 2 * cb : cb;
  w.slot_bytes = w.off_g + (grad ? align_up(static_cast<uint32_t>(D) * 2u, 128) : 0u);
  const int warps = threads / 32;
  w.threads = threads;
  w.total = off + w.slot_bytes * warps;
  if (w.total > (ctas == 1 ? kSmemPerCtaMax - 1024 : kSmemBudget / ctas)) return w;
  long long grid = static_cast<long long>(sm_count()) * ctas;
  const long long need = (q->rows + warps - 1) / warps;
  if (grid > need) grid = need;
  w.grid = static_cast<int>(grid);
  w.ok = true;
  return w;
}

inline void fill_warp_bwd(WarpBwdArgs* a, const WarpBwdPlan& w, const hyc_packed* q, const hyc_packed* q2) {
  memset(a, 0, sizeof(*a));
  a->p = to_dev(q);
  if (q2) a->p2 = to_dev(q2);
  a->off_chan = w.off_chan; a->off_chan2 = w.off_chan2; a->off_wsm = w.off_wsm; a->off_slots = w.off_slots;
  a->slot_bytes = w.slot_bytes; a->off_c2 = w.off_c2; a->off_g = w.off_g;
  a->tx_pad = g_debug_tx_pad;
  a->wait_cycles = g_debug_wait_cycles > 0 ? g_debug_wait_cycles : kWaitCycles;
}

// BITS x NG dispatch shared by the three launchers; LAUNCH(B, NG) launches one instantiation
#define HYC_WARP_BWD_DISPATCH(BITS_V, NG_V, LAUNCH)                         \
  switch (BITS_V) {                                                         \
    case 2:                                                                 \
      switch (NG_V) { case 4: LAUNCH(2, 4) break; case 8: LAUNCH(2, 8) break; default: LAUNCH(2, 16) break; } break; \
    case 4:                                                                 \
      switch (NG_V) { case 2: LAUNCH(4, 2) break; case 4: LAUNCH(4, 4) break; case 8: LAUNCH(4, 8) break; default: LAUNCH(4, 16) break; } break; \
    default:                                                                \
      switch (NG_V) { case 2: LAUNCH(8, 2) break; case 4: LAUNCH(8, 4) break; case 8: LAUNCH(8, 8) break; default: LAUNCH(8, 16) break; } break; \
  }

int launch_decompress_warp(const WarpBwdArgs& a, const WarpBwdPlan& w, cudaStream_t stream);
int launch_norm_bwd_warp(const WarpBwdArgs& a, const WarpBwdPlan& w, cudaStream_t stream);
int launch_act_bwd_warp(const WarpBwdArgs& a, const WarpBwdPlan& w, bool gelu, cudaStream_t stream);

}  // namespace hyc
