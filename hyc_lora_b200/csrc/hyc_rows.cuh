// Per-row passes over a row staged in shared memory: quantise + pack,
// unpack + dequantise, block Walsh-Hadamard rotation, outlier handling.
//
// Thread mapping.  A row of D channels is cut into 8/BITS contiguous segments
// of segw = D*BITS/8 channels.  A "unit" u covers channels 8u..8u+7 of every
// segment, i.e. exactly the 8 packed bytes 8u..8u+7 of the row.  Thread t
// takes units t, t+blockDim, ... so shared-memory reads are 16-byte,
// conflict-free, and the code store is one coalesced 8-byte store per unit.
// Passes that do not pack use "vectors" of 8 consecutive channels the same way.
#pragma once

#include "hyc_common.cuh"

namespace hyc {

enum : int { kModeR = 0, kModeN = 1 };
enum : int { kScaleTensor = 0, kScaleChannel = 1, kScaleToken = 2 };

// Device view of hyc_packed (same meaning, typed pointers).
struct PackedDev {
  int mode, bits;
  long long rows;
  int cols, seq;
  unsigned char* codes;
  uint32_t* status;
  // reference mode
  int scale_kind;
  const __nv_bfloat16* scale;
  const float* thr;
  const __nv_bfloat16* lowrank;
  uint32_t* pool;
  uint32_t pool_cap;
  uint32_t* pool_used;
  uint2* row_meta;
  // north-star mode
  const int* channels;
  int n_channels, group, rotate;
  __nv_bfloat16* out_value;
  float* scales;
};

// Per-CTA shared-memory work areas (any pointer may be null when unused).
struct Work {
  float* red;        // reduction slots: [site][64]
  uint32_t* misc;    // [0] outlier count of the row, [1] pool base, [2] error flag, [3] overflow flag
  uint32_t* omask;   // N: bit per channel, 1 = outlier channel      [D/32]
  int* chan;         // N: outlier channel list                      [k]
  float* gamax;      // N: group absmax                              [D/128]
  float* ginv;       // N: group reciprocal scale                    [D/128]
  float* rot;        // N rotate: fp32 row                           [D]
  uint32_t* list;    // R: outlier entries of the row                [D]
  float* cscale;     // R per-channel: scale as fp32                 [D]
  __nv_bfloat16* xr; // decompressed row                             [D]
};

template <int BITS>
struct CodeTraits {
  static constexpr int kSeg = 8 / BITS;
  static constexpr int kOff = (BITS == 8) ? 0 : (1 << (BITS - 1));
  static constexpr int kLo = -(1 << (BITS - 1));
  static constexpr int kHi = (1 << (BITS - 1)) - 1;
  static constexpr uint32_t kMask = (1u << BITS) - 1u;
};

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return max(lo, min(hi, v)); }

// rint(x * inv) with a single rounding of the exact product: the fused multiply-add
// against 1.5 * 2^23 leaves the integer in the low mantissa bits (|x * inv| < 2^22).
constexpr float kRoundMagic = 12582912.f;
constexpr uint32_t kRoundMagicBits = 0x4B400000u;
__device__ __forceinline__ int round_product(float x, float inv) {
  return __float_as_int(__fmaf_rn(x, inv, kRoundMagic)) - static_cast<int>(kRoundMagicBits);
}

__device__ __forceinline__ uint32_t mask8(const uint32_t* omask, int col) {
  return (omask[col >> 5] >> (col & 31)) & 0xffu;
}

__device__ __forceinline__ float rotate_norm(int n) {
  // 1/sqrt(n) for n in {16,64,256,1024,4096}: an exact power of two
  return n == 16 ? 0.25f : n == 64 ? 0.125f : n == 256 ? 0.0625f : n == 1024 ? 0.03125f : 0.015625f;
}

// ------------------------------------------------------------------ rotation

__device__ __forceinline__ void butterfly8(float (&f)[8]) {
  float t;
#pragma unroll
  for (int i = 0; i < 8; i += 2) { t = f[i]; f[i] = t + f[i + 1]; f[i + 1] = t - f[i + 1]; }
#pragma unroll
  for (int i = 0; i < 8; i += 4) {
    t = f[i]; f[i] = t + f[i + 2]; f[i + 2] = t - f[i + 2];
    t = f[i + 1]; f[i + 1] = t + f[i + 3]; f[i + 3] = t - f[i + 3];
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) { t = f[i]; f[i] = t + f[i + 4]; f[i + 4] = t - f[i + 4]; }
}

// Rotation of the 8 values a lane holds of a 256-channel window (lane l: channels 8l..8l+7),
// block size n <= 256: three butterfly stages inside the thread, then one shuffle stage per
// doubling, then the normalisation.  Every lane of the warp must call it.
__device__ __forceinline__ void rotate_group(float (&f)[8], int n, int lane) {
  butterfly8(f);
#pragma unroll
  for (int m2 = 1; m2 <= 16; m2 <<= 1) {
    if ((m2 << 3) < n) {
      const float sgn = (lane & m2) ? -1.f : 1.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = __fmaf_rn(sgn, f[e], __shfl_xor_sync(0xffffffffu, f[e], m2));
    }
  }
  const float rs = rotate_norm(n);
#pragma unroll
  for (int e = 0; e < 8; ++e) f[e] = __fmul_rn(f[e], rs);   // exact (power of two) and never fused into what follows
}

// Normalised Walsh-Hadamard transform of every aligned block of n channels of
// the row `src` (masked outlier channels read as 0), result in `rot` (fp32).
// src may alias rot.  Lane l of a warp holds channels 8l..8l+7 of a 256-channel
// chunk: strides 1,2,4 run in registers, strides 8..128 through shuffles,
// strides >= 256 through shared memory.  Butterfly order and operand order
// (lower + upper, lower - upper) are fixed, so the result is bit-identical to a
// sequential evaluation.  Ends with a __syncthreads().
template <typename ST, bool MASKED>
__device__ void fwht_row(const ST* src, const uint32_t* omask, float* rot, int D, int n) {
  const int nvec = D >> 3;
  const int lane = threadIdx.x & 31;
  const float rs = rotate_norm(n);
  for (int v0 = (threadIdx.x >> 5) << 5; v0 < nvec; v0 += blockDim.x) {
    const int v = v0 + lane;
    const bool active = v < nvec;
    float f[8];
    if (active) {
      load8<ST>(src, v << 3, f);
      if (MASKED) {
        const uint32_t m = mask8(omask, v << 3);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = ((m >> e) & 1u) ? 0.f : f[e];
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
    }
    butterfly8(f);
#pragma unroll
    for (int m = 1; m <= 16; m <<= 1) {
      if ((m << 3) < n) {
        const bool upper = (lane & m) != 0;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float other = __shfl_xor_sync(0xffffffffu, f[e], m);
          f[e] = upper ? (other - f[e]) : (f[e] + other);
        }
      }
    }
    if (n <= 256) {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] *= rs;
    }
    if (active) store8<float>(rot, v << 3, f);
  }
  if (n > 256) {
    const int half = D >> 1;
    for (int h = 256; h < n; h <<= 1) {
      __syncthreads();
      const bool last = (h << 1) == n;
      for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const int j = i & (h - 1);
        const int lo = ((i - j) << 1) + j;
        const float a = rot[lo], b = rot[lo + h];
        rot[lo] = last ? (a + b) * rs : (a + b);
        rot[lo + h] = last ? (a - b) * rs : (a - b);
      }
    }
  }
  __syncthreads();
}

// ------------------------------------------------------------------ north-star mode: compress

// absmax of the row (or of each 128-channel group) -> reciprocal scale(s).
// Writes the scales of this row to global memory.  Returns the per-row
// reciprocal (GROUPED: reciprocals are left in w.ginv).  Contains block syncs.
template <typename ST, int BITS, bool MASKED, bool GROUPED>
__device__ float n_scales_row(const PackedDev& p, const Work& w, const ST* src, long long row) {
  const int D = p.cols;
  const int nvec = D >> 3;
  const int lane = threadIdx.x & 31;
  const float qmax = static_cast<float>(CodeTraits<BITS>::kHi);
  float amax = 0.f;
  for (int v0 = (threadIdx.x >> 5) << 5; v0 < nvec; v0 += blockDim.x) {
    const int v = v0 + lane;
    float a = 0.f;
    if (v < nvec) {
      float f[8];
      load8<ST>(src, v << 3, f);
      const uint32_t m = MASKED ? mask8(w.omask, v << 3) : 0u;
#pragma unroll
      for (int e = 0; e < 8; ++e) a = fmaxf(a, ((m >> e) & 1u) ? 0.f : fabsf(f[e]));
    }
    if (GROUPED) {
      // 16 consecutive lanes hold one 128-channel group
#pragma unroll
      for (int s = 8; s > 0; s >>= 1) a = fmaxf(a, __shfl_xor_sync(0xffffffffu, a, s));
      if ((lane & 15) == 0 && v < nvec) w.gamax[v >> 4] = a;
    } else {
      amax = fmaxf(amax, a);
    }
  }
  if (GROUPED) {
    __syncthreads();
    const int G = D >> 7;
    for (int g = threadIdx.x; g < G; g += blockDim.x) {
      const float a = w.gamax[g];
      const bool live = a > 0.f;
      p.scales[row * G + g] = live ? __fdiv_rn(a, qmax) : 1.f;
      w.ginv[g] = live ? __fdiv_rn(qmax, a) : 1.f;
    }
    __syncthreads();
    return 0.f;
  } else {
    float r[1] = {amax};
    block_reduce<1>(r, w.red + 64, OpMax());
    const bool live = r[0] > 0.f;
    if (threadIdx.x == 0) p.scales[row] = live ? __fdiv_rn(r[0], qmax) : 1.f;
    return live ? __fdiv_rn(qmax, r[0]) : 1.f;
  }
}

// quantise + pack one row; one 8-byte store per unit
template <typename ST, int BITS, bool MASKED, bool GROUPED>
__device__ void n_quant_row(const Work& w, const ST* src, float inv_row, unsigned char* codes_row, int D) {
  using C = CodeTraits<BITS>;
  const int segw = D / C::kSeg;
  const int units = segw >> 3;
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    uint32_t b0 = 0, b1 = 0;
#pragma unroll
    for (int s = 0; s < C::kSeg; ++s) {
      const int col = s * segw + (u << 3);
      float f[8];
      load8<ST>(src, col, f);
      const uint32_t m = MASKED ? mask8(w.omask, col) : 0u;
      const float inv = GROUPED ? w.ginv[col >> 7] : inv_row;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float x = ((m >> e) & 1u) ? 0.f : f[e];
        const int q = clampi(round_product(x, inv), C::kLo, C::kHi) + C::kOff;
        const uint32_t c = (static_cast<uint32_t>(q) & 0xffu) << (s * BITS);
        if (e < 4) b0 |= c << (8 * e); else b1 |= c << (8 * (e - 4));
      }
    }
    *reinterpret_cast<uint2*>(codes_row + (u << 3)) = make_uint2(b0, b1);
  }
}

// Full north-star compression of the staged row xs.
template <typename XT, int BITS>
__device__ void n_compress_row(const PackedDev& p, const Work& w, const XT* xs, long long row) {
  const int D = p.cols;
  const int k = p.n_channels;
  for (int j = threadIdx.x; j < k; j += blockDim.x)
    p.out_value[row * k + j] = __float2bfloat16_rn(static_cast<float>(xs[w.chan[j]]));
  unsigned char* codes_row = p.codes + row * (static_cast<long long>(D) * BITS / 8);
  if (p.rotate) {
    fwht_row<XT, true>(xs, w.omask, w.rot, D, p.rotate);
    if (p.group) {
      n_scales_row<float, BITS, false, true>(p, w, w.rot, row);
      n_quant_row<float, BITS, false, true>(w, w.rot, 0.f, codes_row, D);
    } else {
      const float inv = n_scales_row<float, BITS, false, false>(p, w, w.rot, row);
      n_quant_row<float, BITS, false, false>(w, w.rot, inv, codes_row, D);
    }
  } else {
    if (p.group) {
      n_scales_row<XT, BITS, true, true>(p, w, xs, row);
      n_quant_row<XT, BITS, true, true>(w, xs, 0.f, codes_row, D);
    } else {
      const float inv = n_scales_row<XT, BITS, true, false>(p, w, xs, row);
      n_quant_row<XT, BITS, true, false>(w, xs, inv, codes_row, D);
    }
  }
}

// ------------------------------------------------------------------ north-star mode: decompress

// Rebuild the bf16 row into w.xr from packed codes (`codes_row`: shared or
// global, 8-byte aligned).  Ends with a __syncthreads(); w.xr is then readable
// by every thread.
template <int BITS>
__device__ void n_dequant_row(const PackedDev& p, const Work& w, const unsigned char* codes_row, long long row) {
  using C = CodeTraits<BITS>;
  const int D = p.cols;
  const int segw = D / C::kSeg;
  const int units = segw >> 3;
  const int G = p.group ? (D >> 7) : 1;
  const float* sc_row = p.scales + row * G;
  const float sc_tok = p.group ? 0.f : __ldg(sc_row);
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    const uint2 cb = *reinterpret_cast<const uint2*>(codes_row + (u << 3));
#pragma unroll
    for (int s = 0; s < C::kSeg; ++s) {
      const int col = s * segw + (u << 3);
      const float sc = p.group ? __ldg(sc_row + (col >> 7)) : sc_tok;
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t byte = ((e < 4 ? cb.x >> (8 * e) : cb.y >> (8 * (e - 4))) & 0xffu);
        const int iv = (BITS == 8) ? static_cast<int>(static_cast<signed char>(byte))
                                   : static_cast<int>((byte >> (s * BITS)) & C::kMask) - C::kOff;
        f[e] = static_cast<float>(iv) * sc;
      }
      if (p.rotate) store8<float>(w.rot, col, f);
      else store8<__nv_bfloat16>(w.xr, col, f);
    }
  }
  __syncthreads();
  if (p.rotate) {
    fwht_row<float, false>(w.rot, nullptr, w.rot, D, p.rotate);
    for (int v = threadIdx.x; v < (D >> 3); v += blockDim.x) {
      float f[8];
      load8<float>(w.rot, v << 3, f);
      store8<__nv_bfloat16>(w.xr, v << 3, f);
    }
    __syncthreads();
  }
  const int k = p.n_channels;
  if (k > 0) {
    for (int j = threadIdx.x; j < k; j += blockDim.x) w.xr[w.chan[j]] = p.out_value[row * k + j];
    __syncthreads();
  }
}

// ------------------------------------------------------------------ reference mode: compress

// One quantise+pack pass.  With `extract`, elements with |x| > thr go to the
// row's shared outlier list and are quantised as 0.
template <typename XT, int BITS>
__device__ void r_quant_row(const PackedDev& p, const Work& w, const XT* xs, long long row, float thr,
                            bool extract, unsigned char* codes_row) {
  using C = CodeTraits<BITS>;
  constexpr bool kBf16 = sizeof(XT) == 2;
  const int D = p.cols;
  const int segw = D / C::kSeg;
  const int units = segw >> 3;
  const int pos = static_cast<int>(row % p.seq);
  const __nv_bfloat16* lr = p.lowrank ? p.lowrank + static_cast<long long>(pos) * D : nullptr;
  float sc_row = 1.f;
  if (p.scale_kind == kScaleTensor) sc_row = __bfloat162float(p.scale[0]);
  else if (p.scale_kind == kScaleToken) sc_row = __bfloat162float(p.scale[pos]);
  const bool per_channel = p.scale_kind == kScaleChannel;
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    uint32_t b0 = 0, b1 = 0;
#pragma unroll
    for (int s = 0; s < C::kSeg; ++s) {
      const int col = s * segw + (u << 3);
      float f[8];
      load8<XT>(xs, col, f);
      if (lr) {
        float l[8];
        load8<__nv_bfloat16>(lr, col, l);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = kBf16 ? bf16_round(f[e] - l[e]) : (f[e] - l[e]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float x = f[e];
        if (extract && fabsf(x) > thr) {
          const uint32_t at = atomicAdd(&w.misc[0], 1u);
          w.list[at] = (float_to_bf16_bits(x) << 16) | static_cast<uint32_t>(col + e);
          x = x - x;   // the reference's x - x * mask: 0, or NaN for an infinite input
        }
        const float sc = per_channel ? w.cscale[col + e] : sc_row;
        float q = __fdiv_rn(x, sc);
        if (kBf16) q = bf16_round(q);
        // a NaN quotient (0/0 on a channel whose calibrated range is empty) is stored as
        // byte value 0, which is what the eager float -> uint8 / int8 cast produces
        const int qi = (q != q) ? 0 : clampi(__float2int_rn(q), C::kLo, C::kHi) + C::kOff;
        const uint32_t c = (static_cast<uint32_t>(qi) & 0xffu) << (s * BITS);
        if (e < 4) b0 |= c << (8 * e); else b1 |= c << (8 * (e - 4));
      }
    }
    *reinterpret_cast<uint2*>(codes_row + (u << 3)) = make_uint2(b0, b1);
  }
}

// Full reference-mode compression of the staged row.  The caller guarantees
// w.misc[0] == 0 on entry and a __syncthreads() since it was zeroed.
template <typename XT, int BITS>
__device__ void r_compress_row(const PackedDev& p, const Work& w, const XT* xs, long long row, float thr) {
  const int D = p.cols;
  unsigned char* codes_row = p.codes + row * (static_cast<long long>(D) * BITS / 8);
  r_quant_row<XT, BITS>(p, w, xs, row, thr, true, codes_row);
  __syncthreads();
  const uint32_t cnt = w.misc[0];
  if (threadIdx.x == 0) {
    uint32_t base = 0, over = 0;
    if (cnt > 0) {
      base = atomicAdd(p.pool_used, cnt);
      if (base > p.pool_cap || cnt > p.pool_cap - base) over = 1;
    }
    w.misc[1] = base;
    w.misc[3] = over;
    p.row_meta[row] = make_uint2(base, over ? 0u : cnt);
    if (over && p.status) atomicOr(p.status, kStatusPoolOverflow);
  }
  __syncthreads();
  const uint32_t base = w.misc[1];
  if (w.misc[3]) {
    // the pool is full: keep every element of this row in the quantised part
    r_quant_row<XT, BITS>(p, w, xs, row, thr, false, codes_row);
  } else {
    for (uint32_t j = threadIdx.x; j < cnt; j += blockDim.x) p.pool[base + j] = w.list[j];
  }
  __syncthreads();
  if (threadIdx.x == 0) w.misc[0] = 0;
}

// ------------------------------------------------------------------ reference mode: decompress

// bf16 row into w.xr: bf16(bf16(lowrank + outlier) + bf16((code - off) * scale)),
// each operation rounded to bf16 as the reference's eager chain does.
template <int BITS>
__device__ void r_dequant_row(const PackedDev& p, const Work& w, const unsigned char* codes_row, long long row) {
  using C = CodeTraits<BITS>;
  const int D = p.cols;
  const int segw = D / C::kSeg;
  const int units = segw >> 3;
  const int pos = static_cast<int>(row % p.seq);
  const __nv_bfloat16* lr = p.lowrank ? p.lowrank + static_cast<long long>(pos) * D : nullptr;
  float sc_row = 1.f;
  if (p.scale_kind == kScaleTensor) sc_row = __bfloat162float(p.scale[0]);
  else if (p.scale_kind == kScaleToken) sc_row = __bfloat162float(p.scale[pos]);
  const bool per_channel = p.scale_kind == kScaleChannel;
  for (int u = threadIdx.x; u < units; u += blockDim.x) {
    const uint2 cb = *reinterpret_cast<const uint2*>(codes_row + (u << 3));
#pragma unroll
    for (int s = 0; s < C::kSeg; ++s) {
      const int col = s * segw + (u << 3);
      float l[8];
      if (lr) load8<__nv_bfloat16>(lr, col, l);
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const uint32_t byte = ((e < 4 ? cb.x >> (8 * e) : cb.y >> (8 * (e - 4))) & 0xffu);
        const int iv = (BITS == 8) ? static_cast<int>(static_cast<signed char>(byte))
                                   : static_cast<int>((byte >> (s * BITS)) & C::kMask) - C::kOff;
        const float sc = per_channel ? w.cscale[col + e] : sc_row;
        const float xq = bf16_round(static_cast<float>(iv) * sc);
        f[e] = lr ? bf16_round(l[e] + xq) : xq;
      }
      store8<__nv_bfloat16>(w.xr, col, f);
    }
  }
  __syncthreads();
  const uint2 meta = p.row_meta[row];
  for (uint32_t j = threadIdx.x; j < meta.y; j += blockDim.x) {
    const uint32_t e = p.pool[meta.x + j];
    const int col = static_cast<int>(e & 0xffffu);
    float val = bf16_bits_to_float(e >> 16);
    if (lr) val = bf16_round(__bfloat162float(lr[col]) + val);
    w.xr[col] = __float2bfloat16_rn(val);
  }
  __syncthreads();
}

}  // namespace hyc
