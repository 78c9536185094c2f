// Fast forward kernel for the channel-outlier mode: compress-only and fused
// norm + compress with the row slice of every thread held in registers.
//
// Each thread owns UPT "units" of the row (see hyc_rows.cuh for the unit
// mapping).  Pass 1 reads them once from the staged row into registers and
// accumulates the row statistics (sum of squares, absmax).  One CTA barrier
// publishes the statistics and at the same time releases the staging slot,
// which thread 0 refills immediately, so the next rows stream in while pass 2
// computes the norm output and the packed codes from registers.  Reduction
// scratch and group maxima are double-buffered by row parity, which is what
// makes a single barrier per row sufficient.
//
// Quantisation is one fused multiply-add per element against a rounding
// constant that already contains the code offset; the integer lands in the low
// mantissa bits and is merged into the packed word with one shift-add, the
// constant's exponent bits being cancelled once per word.
//
// Rotation (block size <= 256).  In the unit mapping a warp already holds 256
// consecutive channels of every segment, so when the segment width is a multiple of
// the rotation block (ROT == 2) the butterflies run in place on the registers of
// pass 1 and pass 2 packs from them; the norm output then re-reads the staged row,
// which therefore stays one row longer in its slot.  Otherwise (ROT == 1) pass 1 runs
// in the chunk mapping of fwht_row (lane l holds channels 8l..8l+7 of an aligned
// 256-channel chunk), writes the rotated fp32 row to shared memory and pass 2 packs
// from there.
#pragma once
#include "hyc_fwd.cuh"

namespace hyc {

template <typename XT>
struct Reg8;
template <>
struct Reg8<__nv_bfloat16> {
  uint4 v;
  __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = *reinterpret_cast<const uint4*>(p); }
  __device__ __forceinline__ void get(float (&f)[8]) const { unpack_bf16x8(v, f); }
};
template <>
struct Reg8<float> {
  float4 a, b;
  __device__ __forceinline__ void load(const float* p) {
    a = *reinterpret_cast<const float4*>(p);
    b = *reinterpret_cast<const float4*>(p + 4);
  }
  __device__ __forceinline__ void get(float (&f)[8]) const {
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w;
    f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
};

// bit position of element e (0..7) of segment s inside its 32-bit output word
template <int BITS>
__host__ __device__ constexpr uint32_t pack_shift(int s, int e) { return 8u * (e & 3) + static_cast<uint32_t>(s) * BITS; }

// minus the sum of the rounding constant's exponent bits over the fields of one word (mod 2^32)
template <int BITS>
__host__ __device__ constexpr uint32_t pack_cancel() {
  uint32_t c = 0;
  for (int s = 0; s < 8 / BITS; ++s)
    for (int e = 0; e < 4; ++e) c -= kRoundMagicBits << pack_shift<BITS>(s, e);
  return c;
}

template <int BITS>
struct PackAcc {
  uint32_t w0, w1;
  __device__ __forceinline__ PackAcc() : w0(pack_cancel<BITS>()), w1(pack_cancel<BITS>()) {}
  // 8 elements of segment s; `inv` is the reciprocal scale
  __device__ __forceinline__ void add(const float (&f)[8], float inv, int s) {
    // 8-bit codes are two's complement: bias by 128 here, flip the bias bit at the end
    const float magic = kRoundMagic + static_cast<float>(BITS == 8 ? 128 : CodeTraits<BITS>::kOff);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const uint32_t bits = __float_as_uint(__fmaf_rn(f[e], inv, magic));
      if (e < 4) w0 += bits << pack_shift<BITS>(s, e);
      else w1 += bits << pack_shift<BITS>(s, e);
    }
  }
  __device__ __forceinline__ uint2 done() const {
    return BITS == 8 ? make_uint2(w0 ^ 0x80808080u, w1 ^ 0x80808080u) : make_uint2(w0, w1);
  }
};

__device__ __forceinline__ float absmax8(const float (&f)[8]) {
  float a = fmaxf(fabsf(f[0]), fabsf(f[1]));
#pragma unroll
  for (int e = 2; e < 8; ++e) a = fmaxf(a, fabsf(f[e]));
  return a;
}

__device__ __forceinline__ void zero_masked(float (&f)[8], uint32_t m) {
#pragma unroll
  for (int e = 0; e < 8; ++e) f[e] = ((m >> e) & 1u) ? 0.f : f[e];
}

// warp + CTA reduction of (sum, max); `buf` holds [2][32] floats of this row parity.
// Contains exactly one __syncthreads().
__device__ __forceinline__ void reduce_sum_max(float& s, float& m, float* buf) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    s += __shfl_xor_sync(0xffffffffu, s, o);
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  }
  const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  if ((threadIdx.x & 31) == 0) { buf[warp] = s; buf[32 + warp] = m; }
  __syncthreads();
  s = buf[0]; m = buf[32];
  for (int w = 1; w < nwarps; ++w) { s += buf[w]; m = fmaxf(m, buf[32 + w]); }
}

// Shared-memory helpers for the outlier channels of a staged row: save the original values
// (fp32, ring of three rows), write them out as bf16 and zero them in the staged row, so that
// the streaming passes need no per-element masks.
template <typename XT>
__device__ __forceinline__ void gather_and_zero(const PackedDev& p, const Work& w, XT* xs, float* osm_row,
                                                long long row) {
  const int k = p.n_channels;
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    const int c = w.chan[j];
    const float o = static_cast<float>(xs[c]);
    osm_row[j] = o;
    p.out_value[row * k + j] = __float2bfloat16_rn(o);
    xs[c] = static_cast<XT>(0.f);
  }
}

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// UPT: units per thread (ROT == 1: 256-channel chunks per warp)
//
// Per row i:   pass 1 (registers <- staged row i, statistics)
//              wait for row i+1, save + zero its outlier channels
//              one CTA barrier  (publishes statistics and the zeroing, frees slot i)
//              refill slot i; write the norm output of row i-1 at its outlier channels
//              pass 2 (norm output and packed codes of row i from registers)
// The norm output of an outlier channel is computed from the saved original by the thread
// that saved it and stored one barrier after the vector stores of the row, which orders the
// two stores to the same address.
template <typename XT, int BITS, bool NORM, int UPT, int ROT>
__global__ void __launch_bounds__(384, 2) fwd_n_fast_kernel(const __grid_constant__ FwdArgs a) {
  using C = CodeTraits<BITS>;
  constexpr int NSEG = C::kSeg;
  constexpr int NR = ROT == 1 ? UPT : UPT * NSEG;
  constexpr bool kLateRefill = ROT == 2 && NORM;   // pass 2 re-reads the staged row
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  const int D = p.cols;
  const int segw = D / NSEG;
  const int U = segw >> 3;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int G = p.group ? (D >> 7) : 1;
  const int k = p.n_channels;
  const int group = p.group;
  const float qmax = static_cast<float>(C::kHi);
  const float inv_d = 1.0f / static_cast<float>(D);
  const float eps = a.eps;
  RowRing ring{reinterpret_cast<uint64_t*>(smem), smem + a.L.off_slots, a.L.slot_bytes, a.L.stages};
  ring.init();
  // the first rows start travelling before the per-CTA tables are set up
  const long long rows = p.rows, stride = gridDim.x;
  long long row = blockIdx.x;
  if (threadIdx.x == 0) {
    for (int s = 0; s < ring.stages; ++s) {
      const long long r = row + s * stride;
      if (r < rows) issue_x_row<XT>(a, ring, s, r);
    }
  }
  const Work w = make_work(smem, a.L);
  setup_packed(p, w);
  float* wsm = reinterpret_cast<float*>(smem + a.L.off_wsm);
  float* bsm = reinterpret_cast<float*>(smem + a.L.off_bsm);
  float* osm = reinterpret_cast<float*>(smem + a.L.off_osm);
  const bool ln = NORM && a.kind == HYC_NORM_LAYER;
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
  // row 0 of this CTA
  if (!mbar_wait_bounded(&ring.bars[0], 0)) w.misc[2] = 1;
  gather_and_zero<XT>(p, w, reinterpret_cast<XT*>(ring.slot(0)), osm, row);
  __syncthreads();
  float rstd_prev = 0.f, mean_prev = 0.f;
  long long row_prev = -1;
  int i = 0;
  // ring position and barrier phase of the current row, and the position in the ring of three saved-outlier
  // rows: counters instead of divisions by the (run-time) stage count
  int st = 0, st_prev = 0, o3 = 0;
  uint32_t ph = 0;
  for (; row < rows; ++i, row += stride) {
    const int par = i & 1;
    const XT* xs = reinterpret_cast<const XT*>(ring.slot(st));
    float* gamax = w.gamax + par * G;
    const float* o_cur = osm + o3 * k;
    const int o3_next = o3 == 2 ? 0 : o3 + 1, o3_prev = o3 == 0 ? 2 : o3 - 1;
    const int sn = st + 1 == ring.stages ? 0 : st + 1;
    const uint32_t phn = sn == 0 ? ph ^ 1u : ph;
    float f[NR][8];
    float mean = 0.f;
    // ---- pass 1
    if (ln) {
      float s1 = 0.f, dummy = 0.f;
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const int col = ROT == 1 ? (((warp + r * nwarps) << 8) + (lane << 3))
                            : ((r % NSEG) * segw + ((threadIdx.x + (r / NSEG) * blockDim.x) << 3));
        const bool ok = ROT == 1 ? (col < D) : ((threadIdx.x + (r / NSEG) * blockDim.x) < U);
        if (ok) {
          load8<XT>(xs, col, f[r]);
#pragma unroll
          for (int e = 0; e < 8; ++e) s1 += f[r][e];
        }
      }
      for (int j = threadIdx.x; j < k; j += blockDim.x) s1 += o_cur[j];
      reduce_sum_max(s1, dummy, w.red + 256 + par * 64);
      mean = s1 * inv_d;
    }
    float ss = 0.f, amax = 0.f;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const int col = ROT == 1 ? (((warp + r * nwarps) << 8) + (lane << 3))
                          : ((r % NSEG) * segw + ((threadIdx.x + (r / NSEG) * blockDim.x) << 3));
      const bool ok = ROT == 1 ? (col < D) : ((threadIdx.x + (r / NSEG) * blockDim.x) < U);
      float a8 = 0.f;
      if (ok) {
        if (!ln) load8<XT>(xs, col, f[r]);
        if (NORM) {
          if (ln) {
#pragma unroll
            for (int e = 0; e < 8; ++e) { const float c = f[r][e] - mean; ss = fmaf(c, c, ss); }
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) ss = fmaf(f[r][e], f[r][e], ss);
          }
        }
        if (ROT == 0) a8 = absmax8(f[r]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[r][e] = 0.f;
      }
      if (ROT == 2) {
        // in place: the norm output re-reads the staged row
        rotate_group(f[r], p.rotate, lane);
        a8 = absmax8(f[r]);
      }
      if (ROT == 1) {
        // rotate a copy; the original stays in f[r] for the norm output
        float t[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) t[e] = f[r][e];
        const int n = p.rotate;
        butterfly8(t);
#pragma unroll
        for (int m2 = 1; m2 <= 16; m2 <<= 1) {
          if ((m2 << 3) < n) {
            const float sgn = (lane & m2) ? -1.f : 1.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) t[e] = __fmaf_rn(sgn, t[e], __shfl_xor_sync(0xffffffffu, t[e], m2));
          }
        }
        const float rs = rotate_norm(n);
#pragma unroll
        for (int e = 0; e < 8; ++e) t[e] *= rs;
        a8 = absmax8(t);
        if (ok) store8<float>(w.rot, col, t);
      }
      if (group) {
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) a8 = fmaxf(a8, __shfl_xor_sync(0xffffffffu, a8, o));
        if (ok && (lane & 15) == 0) gamax[col >> 7] = a8;
      } else {
        amax = fmaxf(amax, a8);
      }
    }
    if (NORM) {
      // the zeroed outlier channels still belong to the row statistics
      for (int j = threadIdx.x; j < k; j += blockDim.x) {
        const float o = o_cur[j];
        ss += ln ? ((o - mean) * (o - mean) - mean * mean) : o * o;
      }
    }
    // ---- next row: save and zero its outlier channels before the barrier
    const long long row_next = row + stride;
    if (row_next < rows) {
      if (!mbar_wait_bounded(&ring.bars[sn], phn)) w.misc[2] = 1;
      gather_and_zero<XT>(p, w, reinterpret_cast<XT*>(ring.slot(sn)), osm + o3_next * k, row_next);
    }
    reduce_sum_max(ss, amax, w.red + par * 64);
    if (w.misc[2]) {
      if (threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusWaitExpired);
      drain_ring(ring, i + 1, row_next + stride, rows, stride, kLateRefill ? ring.stages - 2 : ring.stages - 1);
      return;
    }
    if (threadIdx.x == 0) {
      // the slot every thread has finished with: this row's, or the previous row's when pass 2 reads it again
      const long long freed = kLateRefill ? row_prev : row;
      const int slot_free = kLateRefill ? st_prev : st;
      const long long next = freed + ring.stages * stride;
      if (freed >= 0 && next < rows) {
        fence_proxy_async();
        issue_x_row<XT>(a, ring, slot_free, next);
      }
    }
    // ---- norm output of the previous row at its outlier channels
    if (NORM && row_prev >= 0) {
      const float* o_prv = osm + o3_prev * k;
      XT* yprev = reinterpret_cast<XT*>(a.y) + row_prev * a.row_stride;
      for (int j = threadIdx.x; j < k; j += blockDim.x) {
        const int c = w.chan[j];
        const int cs = split_index(c, D);
        const float y = ln ? ((o_prv[j] - mean_prev) * rstd_prev * wsm[cs] + bsm[cs]) : (o_prv[j] * rstd_prev * wsm[cs]);
        yprev[c] = from_float<XT>(y);
      }
    }
    float rstd = 0.f;
    if (NORM) {
      rstd = 1.0f / sqrtf(ss * inv_d + eps);
      if (threadIdx.x == 0) {
        a.rstd[row] = rstd;
        if (ln) a.mean[row] = mean;
      }
    }
    float inv_row = 1.f;
    if (!group) {
      const bool live = amax > 0.f;
      inv_row = live ? __fdiv_rn(qmax, amax) : 1.f;
      if (threadIdx.x == 0) p.scales[row] = live ? __fdiv_rn(amax, qmax) : 1.f;
    }
    // ---- pass 2
    unsigned char* codes_row = p.codes + row * (static_cast<long long>(D) * BITS / 8);
    XT* yrow = NORM ? reinterpret_cast<XT*>(a.y) + row * a.row_stride : nullptr;
    if (NORM) {
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        const int col = ROT == 1 ? (((warp + r * nwarps) << 8) + (lane << 3))
                            : ((r % NSEG) * segw + ((threadIdx.x + (r / NSEG) * blockDim.x) << 3));
        const bool ok = ROT == 1 ? (col < D) : ((threadIdx.x + (r / NSEG) * blockDim.x) < U);
        if (ok) {
          float y[8], wv[8];
          load8_split(wsm, D, col, wv);
          float xv[8];
          if (ROT == 2) {
            load8<XT>(xs, col, xv);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) xv[e] = f[r][e];
          }
          if (ln) {
            float bv[8];
            load8_split(bsm, D, col, bv);
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = (xv[e] - mean) * rstd * wv[e] + bv[e];
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) y[e] = xv[e] * rstd * wv[e];
          }
          store8<XT>(yrow, col, y);
        }
      }
    }
    if (ROT != 1) {
#pragma unroll
      for (int iu = 0; iu < UPT; ++iu) {
        const int u = threadIdx.x + iu * blockDim.x;
        if (u < U) {
          PackAcc<BITS> acc;
#pragma unroll
          for (int s = 0; s < NSEG; ++s) {
            const int col = s * segw + (u << 3);
            float inv = inv_row;
            if (group) {
              const float ga = gamax[col >> 7];
              const bool live = ga > 0.f;
              inv = live ? __fdiv_rn(qmax, ga) : 1.f;
              if ((lane & 15) == 0) p.scales[row * G + (col >> 7)] = live ? __fdiv_rn(ga, qmax) : 1.f;
            }
            acc.add(f[iu * NSEG + s], inv, s);
          }
          *reinterpret_cast<uint2*>(codes_row + (u << 3)) = acc.done();
        }
      }
    } else {
      for (int u = threadIdx.x; u < U; u += blockDim.x) {
        PackAcc<BITS> acc;
#pragma unroll
        for (int s = 0; s < NSEG; ++s) {
          const int col = s * segw + (u << 3);
          float t[8];
          load8<float>(w.rot, col, t);
          float inv = inv_row;
          if (group) {
            const float ga = gamax[col >> 7];
            const bool live = ga > 0.f;
            inv = live ? __fdiv_rn(qmax, ga) : 1.f;
            if ((col & 127) == 0) p.scales[row * G + (col >> 7)] = live ? __fdiv_rn(ga, qmax) : 1.f;
          }
          acc.add(t, inv, s);
        }
        *reinterpret_cast<uint2*>(codes_row + (u << 3)) = acc.done();
      }
      __syncthreads();  // the rotated row is rewritten by the next iteration
    }
    row_prev = row;
    rstd_prev = rstd;
    mean_prev = mean;
    st_prev = st;
    st = sn;
    ph = phn;
    o3 = o3_next;
  }
  if (NORM && row_prev >= 0) {
    __syncthreads();
    const float* o_prv = osm + (o3 == 0 ? 2 : o3 - 1) * k;
    XT* yprev = reinterpret_cast<XT*>(a.y) + row_prev * a.row_stride;
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
      const int c = w.chan[j];
      const int cs = split_index(c, D);
        const float y = ln ? ((o_prv[j] - mean_prev) * rstd_prev * wsm[cs] + bsm[cs]) : (o_prv[j] * rstd_prev * wsm[cs]);
      yprev[c] = from_float<XT>(y);
    }
  }
}

// ------------------------------------------------------------------ host: eligibility and launch

struct FastPlan {
  bool ok;
  int threads, upt;
  int rot;   // 0 none, 1 through shared memory (chunk mapping), 2 in registers (unit mapping)
};

// The fast kernel takes the channel-outlier mode with no rotation or a rotation block <= 256;
// group scales need 128-channel groups that do not straddle segments.
inline FastPlan plan_fast(const hyc_packed* q, int elem_size) {
  FastPlan f{false, 0, 0, 0};
  if (q->mode != HYC_MODE_N) return f;
  const int D = q->cols, nseg = 8 / q->bits;
  if (q->rotate > 256) return f;
  // rotation in registers needs every segment to start on a rotation-block boundary
  f.rot = q->rotate == 0 ? 0 : 1;
  if (q->rotate && (D / nseg) % q->rotate == 0 && !(q->group && (D / nseg) % 128 != 0)) f.rot = 2;
  const int reg_cap = elem_size == 2 ? 8 : 4;  // 8-element register groups per thread
  int threads = g_tune_threads ? g_tune_threads : (D <= 1024 ? 64 : D <= 4096 ? 128 : 256);
  if (f.rot == 1) {
    const int chunks = (D + 255) / 256;
    for (; threads <= 256; threads *= 2) {
      const int cpt = (chunks + threads / 32 - 1) / (threads / 32);
      if (cpt <= reg_cap) { f.ok = true; f.threads = threads; f.upt = cpt; break; }
    }
  } else {
    if (q->group && (D / nseg) % 128 != 0) return f;
    const int U = D / nseg / 8;
    while (threads > 32 && threads / 2 >= U) threads /= 2;   // a thread owns whole units
    for (; threads <= 384; threads *= 2) {
      const int upt = (U + threads - 1) / threads;
      if (upt * nseg <= reg_cap) { f.ok = true; f.threads = threads; f.upt = upt; break; }
    }
  }
  if (f.ok) {
    // instantiated unit counts: 1, 2, 4, 8
    int u = 1;
    while (u < f.upt) u *= 2;
    f.upt = u;
    // units per thread round up to an instantiated count: give the spare slots back as threads (whole warps),
    // e.g. 688 units at 4 per thread run on 192 threads instead of 256
    if (f.rot != 1 && !g_tune_threads) {
      const int U = q->cols / (8 / q->bits) / 8;
      const int fit = ((U + f.upt - 1) / f.upt + 31) / 32 * 32;
      if (fit < f.threads) f.threads = fit;
    }
  }
  return f;
}

template <typename XT, bool NORM>
static int launch_fwd_fast(const FwdArgs& a, const LaunchPlan& plan, const FastPlan& f, cudaStream_t stream) {
  // register groups per thread are capped by plan_fast; larger combinations are never instantiated
#define HYC_FAST_LAUNCH(BITS, UPT, ROT)                                     \
  {                                                                         \
    if constexpr ((ROT == 1 ? UPT : UPT * (8 / BITS)) <= (sizeof(XT) == 2 ? 8 : 4)) { \
      auto kern = fwd_n_fast_kernel<XT, BITS, NORM, UPT, ROT>;              \
      int rc = set_smem(kern, plan.L.total);                                \
      if (rc) return rc;                                                    \
      kern<<<resident_grid(kern, plan.threads, plan.L.total, plan.grid), plan.threads, plan.L.total, stream>>>(a); HYC_LAUNCHED(); \
    } else {                                                                \
      return HYC_ERR_SMEM;                                                  \
    }                                                                       \
  }
#define HYC_FAST_UPT(BITS, ROT)                                             \
  switch (f.upt) {                                                          \
    case 1: HYC_FAST_LAUNCH(BITS, 1, ROT) break;                            \
    case 2: HYC_FAST_LAUNCH(BITS, 2, ROT) break;                            \
    case 4: HYC_FAST_LAUNCH(BITS, 4, ROT) break;                            \
    default: HYC_FAST_LAUNCH(BITS, 8, ROT) break;                           \
  }
#define HYC_FAST_BITS(ROT)                                                  \
  switch (a.p.bits) {                                                       \
    case 2: HYC_FAST_UPT(2, ROT) break;                                     \
    case 4: HYC_FAST_UPT(4, ROT) break;                                     \
    default: HYC_FAST_UPT(8, ROT) break;                                    \
  }
  if (f.rot == 1) { HYC_FAST_BITS(1) } else if (f.rot == 2) { HYC_FAST_BITS(2) } else { HYC_FAST_BITS(0) }
#undef HYC_FAST_BITS
#undef HYC_FAST_UPT
#undef HYC_FAST_LAUNCH
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? HYC_OK : cuda_fail(e, "fwd_n_fast_kernel launch");
}

int launch_fwd_fast_bf16(const FwdArgs& a, const LaunchPlan& plan, const FastPlan& f, bool norm, cudaStream_t stream);
int launch_fwd_fast_f32(const FwdArgs& a, const LaunchPlan& plan, const FastPlan& f, bool norm, cudaStream_t stream);

}  // namespace hyc
