// Warp-per-row forward kernel for the reference mode (bf16 rows of up to 4096 channels, 2/4/8-bit
// codes): compress-only and fused norm + compress with the reference's arithmetic
// (operators/compress_function.py:144-197) -- optional low-rank subtraction rounded to bf16, scalar
// threshold on |v| selecting element outliers, static scale, correctly rounded quotient rounded to bf16,
// round half to even, clamp, offset-binary segment packing.
//
// A warp owns its rows.  A row (and its low-rank row) lands in the warp's own shared-memory slot by bulk
// asynchronous copies on the warp's own mbarrier, and the warp makes two passes over the slot with short
// rolled loops: pass 1 takes the norm statistics and counts the row's outliers, the warp's lane 0 books the
// row's share of the pool with one global atomic, and pass 2 writes the norm output, the packed codes and --
// now that the place of every entry is known -- the outlier entries straight into the pool.  A row that does
// not fit the pool is known to be one before pass 2 starts, so it is simply quantised whole (the overflow
// bit is raised), with no second quantisation.  No CTA barrier in the row loop, no shared outlier list, no
// helper warp; twenty warps per SM cover the atomic's round trip and the copies.
//
// Arithmetic per element is that of fwd_r_fast_kernel (hyc_fwd_r_fast.cuh), whose helpers are used here:
// codes and the outlier set are identical.
#pragma once
#include <type_traits>

#include "hyc_fwd_r_fast.cuh"
#include "hyc_fwd_warp.cuh"

namespace hyc {

constexpr int kRWarpThreadsMax = 640;

struct RWarpArgs {
  PackedDev p;
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
  uint32_t off_csc, off_crcp, off_wsm, off_bsm, off_slots, slot_bytes, off_lr;
  long long wait_cycles;
};

// NK: 0 compress only, 1 RMSNorm (plain or Gemma), 2 LayerNorm
template <int BITS, int NK>
__global__ void __launch_bounds__(kRWarpThreadsMax, 1) fwd_r_warp_kernel(const __grid_constant__ RWarpArgs a) {
  using XT = __nv_bfloat16;
  constexpr int NSEG = 8 / BITS;
  constexpr bool NORM = NK != 0;
  constexpr bool ln = NK == 2;
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  const int D = p.cols;
  const int segw = D / NSEG;
  const int U = segw >> 3;
  const int upl = (U + 31) >> 5;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
  const float inv_d = 1.0f / static_cast<float>(D);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  uint64_t* bar = &bars[warp];
  unsigned char* slot = smem + a.off_slots + static_cast<size_t>(warp) * a.slot_bytes;
  const XT* xs = reinterpret_cast<const XT*>(slot);
  const __nv_bfloat16* lrs = p.lowrank ? reinterpret_cast<const __nv_bfloat16*>(slot + a.off_lr) : nullptr;
  const bool per_channel = p.scale_kind == kScaleChannel;
  // per-channel scales, negated (the form the quotient's remainder step takes), and their reciprocals as fp32
  // tables (the two halves of each group of 8 apart)
  float* csc = per_channel ? reinterpret_cast<float*>(smem + a.off_csc) : nullptr;
  float* crcp = per_channel ? reinterpret_cast<float*>(smem + a.off_crcp) : nullptr;
  float* wsm = reinterpret_cast<float*>(smem + a.off_wsm);
  float* bsm = reinterpret_cast<float*>(smem + a.off_bsm);
  const uint32_t row_bytes = static_cast<uint32_t>(D) * 2u;
  const long long rows = p.rows, stride = static_cast<long long>(gridDim.x) * W;
  long long row = static_cast<long long>(blockIdx.x) * W + warp;
  auto issue = [&](long long r) {
    mbar_expect_tx(bar, row_bytes + (p.lowrank ? row_bytes : 0u));
    bulk_g2s(slot, a.x + r * a.row_stride, row_bytes, bar);
    if (p.lowrank) bulk_g2s(slot + a.off_lr, p.lowrank + (r % p.seq) * static_cast<long long>(D), row_bytes, bar);
  };
  if (threadIdx.x == 0) {
    for (int i = 0; i < W; ++i) mbar_init(&bars[i], 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (lane == 0 && row < rows) issue(row);
  if (per_channel) {
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      csc[split_index(c, D)] = -__bfloat162float(p.scale[c]);
      crcp[split_index(c, D)] = r_safe_rcp(__bfloat162float(p.scale[c]));
    }
  }
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
  const float thr = bf16_round(*p.thr);   // the fp32 threshold is compared in the activation's dtype
  float sc_row = 1.f, rc_row = 1.f;
  if (p.scale_kind == kScaleTensor) {
    sc_row = __bfloat162float(p.scale[0]);
    rc_row = r_safe_rcp(sc_row);
  }
  const long long cb = static_cast<long long>(D) * BITS / 8;
  __syncthreads();
  uint32_t ph = 0;
  for (; row < rows; row += stride, ph ^= 1u) {
    if (p.scale_kind == kScaleToken) {
      sc_row = __bfloat162float(p.scale[row % p.seq]);
      rc_row = r_safe_rcp(sc_row);
    }
    if (!mbar_wait_bounded(bar, ph, a.wait_cycles)) {
      if (lane == 0 && p.status) atomicOr(p.status, kStatusWaitExpired);
      return;
    }
    // ---- pass 1: norm statistics (of x, before the low-rank part is removed) and the outlier count
    float mean = 0.f;
    if (ln) {
      float s1 = 0.f;
#pragma unroll 2
      for (int iu = 0; iu < upl; ++iu) {
        const int u = lane + 32 * iu;
        if (u < U) {
#pragma unroll
          for (int s = 0; s < NSEG; ++s) {
            float f[8];
            load8<XT>(xs, s * segw + (u << 3), f);
#pragma unroll
            for (int e = 0; e < 8; ++e) s1 += f[e];
          }
        }
      }
      mean = warp_sum(s1) * inv_d;
    }
    float ss = 0.f;
    uint32_t mine = 0;
    if (!lrs) {
      // no low-rank part: the values compared with the threshold are the staged bf16 values themselves, so the
      // count runs on packed pairs (|x| > thr gives 1.0 or 0.0 per half; a lane counts at most 128: exact in bf16)
      const __nv_bfloat162 thr2 = __float2bfloat162_rn(thr);
      __nv_bfloat162 cnt2 = __float2bfloat162_rn(0.f);
      const f32x2 mean2 = f2_make(mean, mean);
      f32x2 ss2 = 0ull;
#pragma unroll 2
      for (int iu = 0; iu < upl; ++iu) {
        const int u = lane + 32 * iu;
        if (u < U) {
#pragma unroll
          for (int s = 0; s < NSEG; ++s) {
            const uint4 w = *reinterpret_cast<const uint4*>(xs + s * segw + (u << 3));
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
            for (int e = 0; e < 4; ++e) cnt2 = __hadd2(cnt2, __hgt2(__habs2(h[e]), thr2));
            if (NORM) {
              // the sum of squares as two partial sums, two channels per instruction
              f32x2 f2[4];
              unpack_bf16x8_pairs(w, f2);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const f32x2 c = ln ? f2_sub(f2[i], mean2) : f2[i];
                ss2 = f2_fma(c, c, ss2);
              }
            }
          }
        }
      }
      {
        float lo, hi;
        f2_split(ss2, lo, hi);
        ss = lo + hi;
      }
      mine = static_cast<uint32_t>(__bfloat162float(__low2bfloat16(cnt2)) + __bfloat162float(__high2bfloat16(cnt2)));
    } else {
#pragma unroll 2
      for (int iu = 0; iu < upl; ++iu) {
        const int u = lane + 32 * iu;
        if (u < U) {
#pragma unroll
          for (int s = 0; s < NSEG; ++s) {
            const int col = s * segw + (u << 3);
            float f[8];
            load8<XT>(xs, col, f);
            if (NORM) {
#pragma unroll
              for (int e = 0; e < 8; ++e) { const float c = ln ? f[e] - mean : f[e]; ss = fmaf(c, c, ss); }
            }
            r_residual8<XT>(f, lrs, col);
#pragma unroll
            for (int e = 0; e < 8; ++e) mine += fabsf(f[e]) > thr ? 1u : 0u;
          }
        }
      }
    }
    // exclusive prefix of the lanes' counts and the row's total
    uint32_t incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const uint32_t n = __shfl_sync(0xffffffffu, incl, 31);
    // the row's share of the pool: the request leaves now, its answer is needed after the statistics
    uint32_t base = 0;
    if (lane == 0 && n > 0) base = atomicAdd(p.pool_used, n);
    float rstd = 0.f;
    if (NORM) {
      ss = warp_sum(ss);
      rstd = 1.0f / sqrtf(ss * inv_d + a.eps);
      if (lane == 0) {
        a.rstd[row] = rstd;
        if (ln) a.mean[row] = mean;
      }
    }
    base = __shfl_sync(0xffffffffu, base, 0);
    const bool over = n > 0 && (base > p.pool_cap || n > p.pool_cap - base);
    if (lane == 0) {
      p.row_meta[row] = make_uint2(base, over ? 0u : n);
      if (over && p.status) atomicOr(p.status, kStatusPoolOverflow);
    }
    const bool extract = !over;              // a row that does not fit the pool is quantised whole
    const float thr_row = extract ? thr : __int_as_float(0x7f800000);   // nothing exceeds +inf
    uint32_t at = base + incl - mine;        // where this lane's entries go
    // ---- pass 2: norm output, codes, outlier entries
    unsigned char* codes_row = p.codes + row * cb;
    XT* yrow = NORM ? a.y + row * a.row_stride : nullptr;
    // The loop is compiled once per combination of three launch-wide facts -- a low-rank row is staged, the
    // scale is per channel, every lane owns a unit in every round -- so that no test of them (a branch and a
    // reconvergence point each, per segment) is left between the loads and the arithmetic of a unit: the
    // compiler then overlaps the segments of a unit.  Each fact is passed as 0 (known false), 1 (known true) or
    // 2 (left to a test at run time).
    auto pass2 = [&](auto has_lr, auto has_csc, auto full_rounds) {
      constexpr int kLr = decltype(has_lr)::value, kCsc = decltype(has_csc)::value;
      const __nv_bfloat16* const lrs_c = kLr == 0 ? nullptr : lrs;
      const float* const csc_c = kCsc == 0 ? nullptr : csc;
      if (kLr == 1) __builtin_assume(lrs_c != nullptr);
      if (kCsc == 1) __builtin_assume(csc_c != nullptr);
#pragma unroll 2
    for (int iu = 0; iu < upl; ++iu) {
      const int u = lane + 32 * iu;
      if (decltype(full_rounds)::value == 1 || u < U) {
        // 2- and 4-bit codes: clamp, rounding and offset on packed bf16 pairs; 8-bit codes do not fit bf16's
        // eight significant bits and keep the fp32 form
        constexpr bool kPairs = BITS < 8;
        RPack<BITS> acc;
        RPackPairs<BITS> accp;
        bool ok = true;
        uint32_t flags = 0;
#pragma unroll
        for (int s = 0; s < NSEG; ++s) {
          const int col = s * segw + (u << 3);
          float v[8];
          load8<XT>(xs, col, v);
          if (NORM) {
            float y[8], wv[8];
            load8_split(wsm, D, col, wv);
            if (ln) {
              float bv[8];
              load8_split(bsm, D, col, bv);
#pragma unroll
              for (int e = 0; e < 8; ++e) y[e] = (v[e] - mean) * rstd * wv[e] + bv[e];
            } else {
              const f32x2 rstd2 = f2_make(rstd, rstd);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const f32x2 t = f2_mul(f2_make(v[2 * i], v[2 * i + 1]), rstd2);
                f2_split(f2_mul(t, f2_make(wv[2 * i], wv[2 * i + 1])), y[2 * i], y[2 * i + 1]);
              }
            }
            store8<XT>(yrow, col, y);
          }
          r_residual8<XT>(v, lrs_c, col);
          RScale8 sc;   // sc.sc: minus the scale
          if (csc_c) {
            load8_split(csc_c, D, col, sc.sc);
            load8_split(crcp, D, col, sc.rc);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) { sc.sc[e] = -sc_row; sc.rc[e] = rc_row; }
          }
          float q[8], vq[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const bool out = fabsf(v[e]) > thr_row;
            // what is quantised at an outlier's slot is x - x * mask as in the reference: 0, or NaN for an
            // infinite input (the unit is then redone with the division sequence, which keeps the NaN)
            vq[e] = v[e];
            if (out) {
              flags |= 1u << (s * 8 + e);
              vq[e] = vq[e] - vq[e];
            }
          }
          // the correctly rounded quotient (r_quotient_plain) of two channels per instruction
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const f32x2 v2 = f2_make(vq[2 * i], vq[2 * i + 1]);
            const f32x2 rc2 = f2_make(sc.rc[2 * i], sc.rc[2 * i + 1]);
            const f32x2 q0 = f2_mul(v2, rc2);
            const f32x2 rem = f2_fma(q0, f2_make(sc.sc[2 * i], sc.sc[2 * i + 1]), v2);
            const f32x2 q2 = f2_fma(rem, rc2, q0);
            accp.check(q2);
            f2_split(q2, q[2 * i], q[2 * i + 1]);
          }
          if (!kPairs) {
#pragma unroll
            for (int e = 0; e < 8; ++e) acc.add(bf16_round(q[e]), s, e);
          }
          if (kPairs) {
            accp.add(q[0], q[2], s, 0);
            accp.add(q[1], q[3], s, 1);
            accp.add(q[4], q[6], s, 4);
            accp.add(q[5], q[7], s, 5);
          }
        }
        ok = accp.ok();
        uint2 packed = kPairs ? accp.done() : acc.done();
        if (!ok) packed = r_unit_exact<XT, BITS>(xs, lrs_c, csc_c ? p.scale : nullptr, sc_row, segw, u, thr_row);
        *reinterpret_cast<uint2*>(codes_row + (u << 3)) = packed;
        // the unit's outliers, values read again from the staged row
        while (flags) {
          const int b = __ffs(flags) - 1;
          flags &= flags - 1;
          const int col = (b >> 3) * segw + (u << 3) + (b & 7);
          uint32_t vbits = reinterpret_cast<const uint16_t*>(xs)[col];   // the staged bf16 value as it is
          if (lrs_c) vbits = float_to_bf16_bits(bf16_round(__bfloat162float(xs[col]) - __bfloat162float(lrs_c[col])));
          p.pool[at++] = (vbits << 16) | static_cast<uint32_t>(col);
        }
      }
    }
    };
    using K0 = std::integral_constant<int, 0>;
    using K1 = std::integral_constant<int, 1>;
    using K2 = std::integral_constant<int, 2>;
    const bool full = (U & 31) == 0;
    if (lrs) {
      if (per_channel) { if (full) pass2(K1(), K1(), K1()); else pass2(K1(), K1(), K2()); }
      else { if (full) pass2(K1(), K0(), K1()); else pass2(K1(), K0(), K2()); }
    } else {
      if (per_channel) { if (full) pass2(K0(), K1(), K1()); else pass2(K0(), K1(), K2()); }
      else { if (full) pass2(K0(), K0(), K1()); else pass2(K0(), K0(), K2()); }
    }
    __syncwarp();   // every lane is done with the slot
    const long long next = row + stride;
    if (lane == 0 && next < rows) {
      fence_proxy_async();
      issue(next);
    }
  }
}

// ------------------------------------------------------------------ host: eligibility and launch

struct RWarpPlan {
  bool ok;
  int threads, grid;
  uint32_t off_csc, off_crcp, off_wsm, off_bsm, off_slots, slot_bytes, off_lr, total;
};

// bf16 rows in the plain layout, up to 4096 channels, 2/4/8-bit codes, at most 65535 columns per entry
inline RWarpPlan plan_r_warp(const hyc_packed* q, const hyc_dense* x, bool norm, bool ln) {
  RWarpPlan w;
  memset(&w, 0, sizeof(w));
  static const bool off_env = getenv("HYC_FWD_R_WARP") && getenv("HYC_FWD_R_WARP")[0] == '0';
  if (off_env || q->mode != HYC_MODE_R || x->dtype != HYC_BF16 || x->chunks != 1) return w;
  if (q->bits != 2 && q->bits != 4 && q->bits != 8) return w;
  if (g_tune_threads || g_tune_stages || g_tune_ctas) return w;
  const int D = q->cols;
  if (D > 4096) return w;
  uint32_t off = 64 * 8;
  auto take = [&](uint32_t bytes) { uint32_t o = off; off = align_up(off + bytes, 16); return o; };
  if (q->scale_kind == HYC_SCALE_CHANNEL) { w.off_csc = take(D * 4); w.off_crcp = take(D * 4); }
  if (norm) w.off_wsm = take(D * 4);
  if (ln) w.off_bsm = take(D * 4);
  off = align_up(off, 128);
  w.off_slots = off;
  w.off_lr = align_up(static_cast<uint32_t>(D) * 2u, 128);
  w.slot_bytes = w.off_lr * (q->lowrank ? 2u : 1u);
  int warps = static_cast<int>((kSmemPerCtaMax - 2048 - off) / w.slot_bytes);
  if (warps > kRWarpThreadsMax / 32) warps = kRWarpThreadsMax / 32;
  if (warps < 4) return w;
  w.threads = warps * 32;
  w.total = off + w.slot_bytes * warps;
  long long grid = sm_count();
  const long long need = (q->rows + warps - 1) / warps;
  if (grid > need) grid = need;
  w.grid = static_cast<int>(grid);
  w.ok = true;
  return w;
}

int launch_fwd_r_warp(const RWarpArgs& a, const RWarpPlan& w, bool norm, cudaStream_t stream);

}  // namespace hyc
