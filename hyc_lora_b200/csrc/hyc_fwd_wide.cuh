// Forward kernels of the sites AROUND the gated MLP, channel mode, bf16 rows of any width that is a multiple of
// 128 channels (3072, 11008, 14336, ...): one pass makes the site's output and every record the layer saves of
// the tensors the pass touches.
//
//   OP_COMPRESS   x                 -> C(x)
//   OP_SILU/GELU  x                 -> y = act(x), C(x), and (optionally) C(y)
//   OP_PRODUCT    x1, x2            -> y = x1 * x2, C(x2), and (optionally) C(y)
//
// In the reference every one of these is a separate pass: the activation (efficient_silu.py:33), the compression
// of its input (:35), the product (efficient_hadamard.py:43), the compression of both operands (:45-46) and, in
// the LoRA-A linear behind it, the compression of the product (efficient_linear.py:46).
//
// Layout: as in hyc_fwd_chunk.cuh a lane owns one chunk of CH = 128 / segments consecutive channels of every
// packed segment, so a row of D channels takes D / 128 lanes: WPR = 1..4 warps work on one row (a "row group";
// the CTA holds 12 / WPR of them), rotation blocks up to CH wide never leave the lane, wider ones cross lanes of
// one warp.  Rows are staged by tensor copies with the 128-byte swizzle; the output is written over a staged
// row and leaves through one tensor store; its record is then made from there.  The warps of a row group meet
// at a named barrier (bar.sync id, 32 * WPR) for the row's absmax and around the staged row; whether a bounded
// wait ran out is decided for the whole group at once, so no warp can be left waiting at such a barrier.
#pragma once
#include <type_traits>
#include "hyc_fwd_chunk.cuh"

namespace hyc {

constexpr int kWideWarps = 12;
enum { kWideCompress = 0, kWideSilu = 1, kWideGelu = 2, kWideProduct = 3 };

struct WideArgs {
  PackedDev p;           // record of x (OP_PRODUCT: of x2)
  PackedDev p2;          // record of the output (has_p2)
  int has_p2;
  int lanes;             // chunks per segment = lanes at work on a row (D / 128)
  uint32_t off_chan, off_chan2, off_red, off_slots, slot_stride;
  long long wait_cycles;
  uint32_t tx_pad;       // test hook: bytes announced beyond what a copy brings (0 in normal use)
};

template <int WPR>
__device__ __forceinline__ void group_sync(int group) {
  if (WPR == 1) __syncwarp();
  else asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(WPR * 32) : "memory");
}

// maximum over the lanes of a row group; `red`: WPR floats of this group and call parity
template <int WPR>
__device__ __forceinline__ float group_max(float v, float* red, int group, int wig, int lane) {
  v = warp_max(v);
  if (WPR == 1) return v;
  if (lane == 0) red[wig] = v;
  group_sync<WPR>(group);
  float m = red[0];
#pragma unroll
  for (int i = 1; i < WPR; ++i) m = fmaxf(m, red[i]);
  return m;
}

// Outlier channels of one record, looked after by the lanes of a row group (lane g: entries g, g + 32 WPR, ...).
template <int WPR, int NQ>
__device__ __forceinline__ void wide_take_outliers(const PackedDev& p, const int* chan, unsigned char* slot, int row, int glane,
                                                   float (&ov)[NQ]) {
  const int k = p.n_channels;
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    ov[q] = 0.f;
    const int i = glane + 32 * WPR * q;
    if (i < k) {
      __nv_bfloat16* at = reinterpret_cast<__nv_bfloat16*>(slot + swz_channel(static_cast<uint32_t>(chan[i])));
      const __nv_bfloat16 o = *at;
      p.out_value[static_cast<long long>(row) * k + i] = o;
      ov[q] = __bfloat162float(o);
      *at = __float2bfloat16_rn(0.f);
    }
  }
}

template <int NSEG, int CH>
__device__ __forceinline__ void wide_load(const unsigned char* slot, int segw, int glane, bool active, uint4 (&raw)[NSEG][CH / 8]) {
#pragma unroll
  for (int s = 0; s < NSEG; ++s)
#pragma unroll
    for (int j = 0; j < CH / 8; ++j)
      raw[s][j] = active ? *reinterpret_cast<const uint4*>(slot + swz_piece(static_cast<uint32_t>(s * segw + glane * CH + 8 * j)))
                         : make_uint4(0u, 0u, 0u, 0u);
}

// Scale and pack the lane's rotated share (see chunk_scale_pack); the row's absmax comes from the whole group.
template <int BITS, int CH, bool GROUP, int WPR>
__device__ __forceinline__ void wide_scale_pack(const PackedDev& p, const f32x2 (&v)[8 / BITS][CH / 2], int row, int glane,
                                                bool active, float* red, int group, int wig, int lane) {
  using C = CodeTraits<BITS>;
  constexpr int NSEG = C::kSeg;
  constexpr int NPC = CH / 8;
  const int D = p.cols;
  const int segw = D / NSEG;
  const float qmax = static_cast<float>(C::kHi);
  const float rs = p.rotate ? rotate_norm(p.rotate) : 1.f;        // a power of two: scaling by it is exact
  float inv[NSEG];
  float amax = 0.f;
#pragma unroll
  for (int s = 0; s < NSEG; ++s) {
    float a8 = 0.f;
#pragma unroll
    for (int i = 0; i < CH / 2; ++i) {
      float lo, hi;
      f2_split(v[s][i], lo, hi);
      a8 = fmaxf(a8, fmaxf(fabsf(lo), fabsf(hi)));
    }
    if (GROUP) {
#pragma unroll
      for (int o = (128 / CH) >> 1; o > 0; o >>= 1) a8 = fmaxf(a8, __shfl_xor_sync(0xffffffffu, a8, o));
      a8 = __fmul_rn(a8, rs);
      const bool live = a8 > 0.f;
      inv[s] = live ? __fmul_rn(__fdiv_rn(qmax, a8), rs) : rs;
      if (active && (lane & (128 / CH - 1)) == 0)
        p.scales[static_cast<long long>(row) * (D >> 7) + ((s * segw + glane * CH) >> 7)] = live ? __fdiv_rn(a8, qmax) : 1.f;
    } else {
      amax = fmaxf(amax, a8);
    }
  }
  if (!GROUP) {
    amax = __fmul_rn(group_max<WPR>(amax, red, group, wig, lane), rs);
    const bool live = amax > 0.f;
    const float inv_row = live ? __fmul_rn(__fdiv_rn(qmax, amax), rs) : rs;
    if (glane == 0) p.scales[row] = live ? __fdiv_rn(amax, qmax) : 1.f;
#pragma unroll
    for (int s = 0; s < NSEG; ++s) inv[s] = inv_row;
  }
  if (!active) return;
  const float magic = kRoundMagic + static_cast<float>(BITS == 8 ? 128 : C::kOff);
  const f32x2 magic2 = f2_make(magic, magic);
  unsigned char* codes = p.codes + static_cast<long long>(row) * (D * BITS / 8) + glane * CH;
#pragma unroll
  for (int u = 0; u < NPC; u += 2) {
    uint32_t w[4] = {pack_cancel<BITS>(), pack_cancel<BITS>(), pack_cancel<BITS>(), pack_cancel<BITS>()};
#pragma unroll
    for (int s = 0; s < NSEG; ++s) {
      const f32x2 inv2 = f2_make(inv[s], inv[s]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float lo, hi;
        f2_split(f2_fma(v[s][4 * u + e], inv2, magic2), lo, hi);
        w[e >> 1] += __float_as_uint(lo) << pack_shift<BITS>(s, 2 * e);
        w[e >> 1] += __float_as_uint(hi) << pack_shift<BITS>(s, 2 * e + 1);
      }
    }
    if (BITS == 8) {
#pragma unroll
      for (int i = 0; i < 4; ++i) w[i] ^= 0x80808080u;
    }
    *reinterpret_cast<uint4*>(codes + 8 * u) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// raw bf16 -> (rotated) fp32 pairs; rotation off: just the unpacking
template <int NSEG, int CH>
__device__ __forceinline__ void wide_unpack_rotate(const uint4 (&raw)[NSEG][CH / 8], f32x2 (&v)[NSEG][CH / 2], int rotate, int lane) {
#pragma unroll
  for (int s = 0; s < NSEG; ++s) {
#pragma unroll
    for (int j = 0; j < CH / 8; ++j) {
      f32x2 f[4];
      unpack_bf16x8_pairs(raw[s][j], f);
#pragma unroll
      for (int e = 0; e < 4; ++e) v[s][4 * j + e] = f[e];
    }
    if (rotate) rotate_chunk<CH>(v[s], rotate, lane);
  }
}

// x * sigmoid(x) with the hardware exponential and reciprocal (a few units in the last place of fp32; the result
// is rounded to bf16, 8 bits): the exact routines cost about 35 instructions per element, which is more than all
// the rest of the pass together
__device__ __forceinline__ float act_silu(float x) { return __fdividef(x, 1.0f + __expf(-x)); }
__device__ __forceinline__ float act_gelu(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); }

// RN: the rotation block when the kernel is compiled for one (64, what rows of 11 008 and 14 336 channels use:
// the butterfly stages then carry no test of the block size and the segments of a row overlap), or -1: the
// record's own, read at run time.  Two kernels rather than two loops in one: a launch inside a training step
// starts with cold instruction caches, and code that is not run still costs there.
template <int BITS, int OP, int CH, bool GROUP, int WPR, int RN>
__global__ void __launch_bounds__(kWideWarps * 32, 1)
fwd_n_wide_kernel(const __grid_constant__ WideArgs a, const __grid_constant__ CUtensorMap in_map,
                  const __grid_constant__ CUtensorMap in2_map, const __grid_constant__ CUtensorMap y_map) {
  using C = CodeTraits<BITS>;
  constexpr int NSEG = C::kSeg;
  constexpr int NPC = CH / 8;
  constexpr int G = kWideWarps / WPR;               // row groups per CTA
  constexpr int NQ = kWarpOutPerLane;               // outlier channels a lane looks after: k <= 128 * WPR
  constexpr bool ACT = OP == kWideSilu || OP == kWideGelu;
  constexpr bool PROD = OP == kWideProduct;
  static_assert(NSEG * CH == 128, "a lane holds 128 channels");
  static_assert(kWideWarps % WPR == 0, "whole row groups");
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  const int D = p.cols;
  const int segw = D / NSEG;
  const int k = p.n_channels;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int group = warp / WPR, wig = warp % WPR, glane = wig * 32 + lane;
  const bool active = glane < a.lanes;
  const bool leader = glane == 0;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);          // two per group
  int* flags = reinterpret_cast<int*>(smem + 64 * 8);          // per group: a wait ran out
  int* chan = reinterpret_cast<int*>(smem + a.off_chan);
  int* chan2 = reinterpret_cast<int*>(smem + a.off_chan2);
  float* red = reinterpret_cast<float*>(smem + a.off_red) + group * 2 * WPR;
  // two slots per group.  compress / activation: the row and the row after it.  product: x1 and x2 of one row.
  unsigned char* slots = smem + a.off_slots + ((1024u - (smem_u32(smem) & 1023u)) & 1023u) +
                         static_cast<size_t>(group) * 2u * a.slot_stride;
  uint64_t* bar2 = &bars[2 * group];
  const uint32_t row_bytes = static_cast<uint32_t>(D) * 2u;
  const int rows = static_cast<int>(p.rows), stride = static_cast<int>(gridDim.x) * G;
  int row = static_cast<int>(blockIdx.x) * G + group;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2 * G; ++i) mbar_init(&bars[i], 1);
    fence_barrier_init();
  }
  if (threadIdx.x < G) flags[threadIdx.x] = 0;
  __syncthreads();
  if (leader) {
    if (PROD) {
      if (row < rows) {
        mbar_expect_tx(&bar2[0], row_bytes + a.tx_pad);
        tensor_load_row(slots, &in_map, row, &bar2[0]);
        mbar_expect_tx(&bar2[1], row_bytes + a.tx_pad);
        tensor_load_row(slots + a.slot_stride, &in2_map, row, &bar2[1]);
      }
    } else {
      for (int s = 0; s < 2; ++s) {
        const int r = row + s * stride;
        if (r < rows) {
          mbar_expect_tx(&bar2[s], row_bytes + a.tx_pad);
          tensor_load_row(slots + s * a.slot_stride, &in_map, r, &bar2[s]);
        }
      }
    }
  }
  for (int j = threadIdx.x; j < k; j += blockDim.x) chan[j] = p.channels[j];
  if (a.has_p2)
    for (int j = threadIdx.x; j < a.p2.n_channels; j += blockDim.x) chan2[j] = a.p2.channels[j];
  __syncthreads();

  uint32_t ph = 0;        // product: parity of both barriers; else: parity of slot 0's (slot 1 flips one row later)
  int st = 0;
  int rp = 0;             // which half of `red` the next absmax exchange uses
  const int nrot = RN >= 0 ? RN : p.rotate;
  for (; row < rows; row += stride) {
    // ---- wait for the row (both operands); the group decides together whether a wait ran out
    bool ok;
    if (PROD) {
      ok = mbar_wait_bounded(&bar2[0], ph, a.wait_cycles);
      ok = mbar_wait_bounded(&bar2[1], ph, a.wait_cycles) && ok;
    } else {
      ok = mbar_wait_bounded(&bar2[st], ph, a.wait_cycles);
    }
    if (WPR == 1) {
      ok = __all_sync(0xffffffffu, ok);
    } else {
      if (!ok) flags[group] = 1;
      group_sync<WPR>(group);
      ok = flags[group] == 0;
    }
    if (!ok) {
      if (leader && p.status) atomicOr(p.status, kStatusWaitExpired);
      // a copy into the other slot may still be in flight: give it a bounded chance to land
      if (!PROD && row + stride < rows) (void)mbar_wait_bounded(&bar2[st ^ 1], st ? ph ^ 1u : ph, a.wait_cycles);
      break;
    }
    unsigned char* slot = PROD ? slots + a.slot_stride : slots + st * a.slot_stride;      // the row C(x) is made of
    unsigned char* yslot = PROD ? slots : slot;                                           // where the output is built
    uint64_t* bar = PROD ? &bar2[1] : &bar2[st];
    const int next = PROD ? row + stride : row + 2 * stride;
    float ov[NQ];
    wide_take_outliers<WPR, NQ>(p, chan, slot, row, glane, ov);
    group_sync<WPR>(group);
    uint4 raw[NSEG][NPC];
    wide_load<NSEG, CH>(slot, segw, glane, active, raw);
    f32x2 v[NSEG][CH / 2];
    if (OP == kWideCompress || PROD) {
      // every lane has what it needs of this slot: hand it back to the copy engine
      group_sync<WPR>(group);
      if (leader && next < rows) {
        fence_proxy_async();
        mbar_expect_tx(bar, row_bytes + a.tx_pad);
        tensor_load_row(slot, PROD ? &in2_map : &in_map, next, bar);
      }
    }
    if (ACT || PROD) {
      // ---- the output, built over a staged row
      float patch[NQ];
      if (PROD) {
        // x2's outlier channels are zero in `raw`: their products come from the kept values and x1's staged row
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          patch[q] = 0.f;
          const int i = glane + 32 * WPR * q;
          if (i < k)
            patch[q] = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(yslot + swz_channel(static_cast<uint32_t>(chan[i])))) * ov[q];
        }
        group_sync<WPR>(group);
      }
      if (active) {
#pragma unroll
        for (int s = 0; s < NSEG; ++s) {
#pragma unroll
          for (int j = 0; j < NPC; ++j) {
            const uint32_t at = swz_piece(static_cast<uint32_t>(s * segw + glane * CH + 8 * j));
            float f[8], y[8];
            unpack_bf16x8(raw[s][j], f);
            if (PROD) {
              float g[8];
              unpack_bf16x8(*reinterpret_cast<const uint4*>(yslot + at), g);
#pragma unroll
              for (int e = 0; e < 8; ++e) y[e] = g[e] * f[e];
            } else {
#pragma unroll
              for (int e = 0; e < 8; ++e) y[e] = OP == kWideSilu ? act_silu(f[e]) : act_gelu(f[e]);
            }
            *reinterpret_cast<uint4*>(yslot + at) = pack_bf16x8(y);
          }
        }
      }
      // order the vector stores before the scalar stores of the outlier channels' outputs (other lanes)
      group_sync<WPR>(group);
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        const int i = glane + 32 * WPR * q;
        if (i < k) {
          const float y = PROD ? patch[q] : (OP == kWideSilu ? act_silu(ov[q]) : act_gelu(ov[q]));
          *reinterpret_cast<__nv_bfloat16*>(yslot + swz_channel(static_cast<uint32_t>(chan[i]))) = __float2bfloat16_rn(y);
        }
      }
      fence_proxy_async();
      group_sync<WPR>(group);
      if (leader) {
        tensor_store_row(&y_map, row, yslot);
        bulk_commit();
      }
    }
    // ---- the record of x (x2), from the registers
    wide_unpack_rotate<NSEG, CH>(raw, v, nrot, lane);
    wide_scale_pack<BITS, CH, GROUP, WPR>(p, v, row, glane, active, red + rp * WPR, group, wig, lane);
    rp ^= 1;
    if (ACT || PROD) {
      if (a.has_p2) {
        // ---- the record of the output, from its staged copy (once the store has read it)
        if (leader) bulk_wait_read();
        group_sync<WPR>(group);
        float ov2[NQ];
        wide_take_outliers<WPR, NQ>(a.p2, chan2, yslot, row, glane, ov2);
        group_sync<WPR>(group);
        wide_load<NSEG, CH>(yslot, segw, glane, active, raw);
        wide_unpack_rotate<NSEG, CH>(raw, v, a.p2.rotate, lane);
        wide_scale_pack<BITS, CH, GROUP, WPR>(a.p2, v, row, glane, active, red + rp * WPR, group, wig, lane);
        rp ^= 1;
      }
      group_sync<WPR>(group);
      if (leader) {
        bulk_wait_read();
        if (next < rows) {
          fence_proxy_async();
          uint64_t* ybar = PROD ? &bar2[0] : bar;
          mbar_expect_tx(ybar, row_bytes + a.tx_pad);
          tensor_load_row(yslot, &in_map, next, ybar);
        }
      }
    }
    if (PROD) {
      ph ^= 1u;
    } else {
      if (st) ph ^= 1u;
      st ^= 1;
    }
  }
  // no tensor store of this thread may still be reading shared memory when the CTA leaves
  if ((ACT || PROD) && leader) bulk_wait_all();
}

// ------------------------------------------------------------------ host: eligibility and launch

struct WidePlan {
  bool ok;
  int wpr, lanes, grid;
  uint32_t off_chan, off_chan2, off_red, off_slots, slot_stride, total;
};

// bf16 rows in the plain layout, a multiple of 128 channels wide, at most four warps per row; a rotation block
// either fits a lane's chunk or tiles the lanes at work; `q2`: record of the output, or nullptr.
inline WidePlan plan_wide(const hyc_packed* q, const hyc_dense* x, const hyc_packed* q2) {
  WidePlan w;
  memset(&w, 0, sizeof(w));
  if (q->mode != HYC_MODE_N || x->dtype != HYC_BF16 || x->chunks != 1) return w;
  if (q->bits != 2 && q->bits != 4 && q->bits != 8) return w;
  if (g_tune_threads || g_tune_stages || g_tune_ctas) return w;
  if (q->rows > 0x3fffffffLL || (x->row_stride * 2) % 16 != 0) return w;
  const int D = q->cols, nseg = 8 / q->bits, ch = 128 / nseg;
  if (D % 128) return w;
  const int lanes = D / 128;
  const int wpr = (lanes + 31) / 32;
  if (wpr > 4) return w;
  if (q->rotate > ch && (q->rotate / ch > 32 || lanes % (q->rotate / ch))) return w;
  if (q->group && ch < 128 && lanes % (128 / ch)) return w;
  if (q->n_channels > 32 * kWarpOutPerLane * wpr) return w;
  if (q2 && (q2->mode != HYC_MODE_N || q2->bits != q->bits || q2->group != q->group || q2->rotate != q->rotate ||
             q2->cols != q->cols || q2->rows != q->rows || q2->n_channels > 32 * kWarpOutPerLane * wpr))
    return w;
  if (!tensor_map_encoder()) return w;
  const int groups = kWideWarps / wpr;
  uint32_t off = 1024;                                     // mbarriers (two per group) and the groups' wait flags
  auto take = [&](uint32_t bytes, uint32_t align) { off = align_up(off, align); uint32_t o = off; off += bytes; return o; };
  w.off_chan = take((q->n_channels > 0 ? q->n_channels : 1) * 4, 16);
  w.off_chan2 = take((q2 && q2->n_channels > 0 ? q2->n_channels : 1) * 4, 16);
  w.off_red = take(groups * 2 * wpr * 4, 16);
  w.slot_stride = align_up(static_cast<uint32_t>(D) * 2u, 1024);     // the swizzle pattern's period
  w.off_slots = take(w.slot_stride * groups * 2, 1024);
  w.total = off + 1024;                                    // room to start the slots on a 1024-byte address
  if (w.total > kSmemPerCtaMax) return w;
  w.wpr = wpr;
  w.lanes = lanes;
  long long grid = sm_count();
  const long long need = (q->rows + groups - 1) / groups;
  if (grid > need) grid = need;
  w.grid = static_cast<int>(grid);
  w.ok = true;
  return w;
}

template <int BITS, int OP>
int launch_wide_op(const WideArgs& a, const WidePlan& w, const CUtensorMap& in_map, const CUtensorMap& in2_map,
                   const CUtensorMap& y_map, cudaStream_t stream) {
#define HYC_WIDE_LAUNCH(GROUP, WPR)                                                             \
  {                                                                                             \
    if (a.p.rotate == 64) {                                                                     \
      auto kern = fwd_n_wide_kernel<BITS, OP, 128 * BITS / 8, GROUP, WPR, 64>;                  \
      int rc = set_smem(kern, w.total);                                                         \
      if (rc) return rc;                                                                        \
      kern<<<w.grid, kWideWarps * 32, w.total, stream>>>(a, in_map, in2_map, y_map); HYC_LAUNCHED(); \
    } else {                                                                                    \
      auto kern = fwd_n_wide_kernel<BITS, OP, 128 * BITS / 8, GROUP, WPR, -1>;                  \
      int rc = set_smem(kern, w.total);                                                         \
      if (rc) return rc;                                                                        \
      kern<<<w.grid, kWideWarps * 32, w.total, stream>>>(a, in_map, in2_map, y_map); HYC_LAUNCHED(); \
    }                                                                                           \
  }
#define HYC_WIDE_WPR(GROUP)                                                                     \
  switch (w.wpr) {                                                                              \
    case 1: HYC_WIDE_LAUNCH(GROUP, 1) break;                                                    \
    case 2: HYC_WIDE_LAUNCH(GROUP, 2) break;                                                    \
    case 3: HYC_WIDE_LAUNCH(GROUP, 3) break;                                                    \
    default: HYC_WIDE_LAUNCH(GROUP, 4) break;                                                   \
  }
  if (a.p.group) { HYC_WIDE_WPR(true) } else { HYC_WIDE_WPR(false) }
#undef HYC_WIDE_WPR
#undef HYC_WIDE_LAUNCH
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? HYC_OK : cuda_fail(e, "fwd_n_wide_kernel launch");
}

// one translation unit per bit width and pair of operations
int launch_wide_b2_cp(const WideArgs& a, const WidePlan& w, int op, const CUtensorMap& m0, const CUtensorMap& m1, const CUtensorMap& m2, cudaStream_t s);
int launch_wide_b4_cp(const WideArgs& a, const WidePlan& w, int op, const CUtensorMap& m0, const CUtensorMap& m1, const CUtensorMap& m2, cudaStream_t s);
int launch_wide_b8_cp(const WideArgs& a, const WidePlan& w, int op, const CUtensorMap& m0, const CUtensorMap& m1, const CUtensorMap& m2, cudaStream_t s);
int launch_wide_b2_act(const WideArgs& a, const WidePlan& w, int op, const CUtensorMap& m0, const CUtensorMap& m1, const CUtensorMap& m2, cudaStream_t s);
int launch_wide_b4_act(const WideArgs& a, const WidePlan& w, int op, const CUtensorMap& m0, const CUtensorMap& m1, const CUtensorMap& m2, cudaStream_t s);
int launch_wide_b8_act(const WideArgs& a, const WidePlan& w, int op, const CUtensorMap& m0, const CUtensorMap& m1, const CUtensorMap& m2, cudaStream_t s);

inline int launch_wide(const WideArgs& a, const WidePlan& w, int op, const CUtensorMap& m0, const CUtensorMap& m1,
                       const CUtensorMap& m2, cudaStream_t s) {
  const bool act = op == kWideSilu || op == kWideGelu;
  if (a.p.bits == 2) return act ? launch_wide_b2_act(a, w, op, m0, m1, m2, s) : launch_wide_b2_cp(a, w, op, m0, m1, m2, s);
  if (a.p.bits == 4) return act ? launch_wide_b4_act(a, w, op, m0, m1, m2, s) : launch_wide_b4_cp(a, w, op, m0, m1, m2, s);
  return act ? launch_wide_b8_act(a, w, op, m0, m1, m2, s) : launch_wide_b8_cp(a, w, op, m0, m1, m2, s);
}

}  // namespace hyc
