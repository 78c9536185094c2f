// Chunk-per-lane forward kernel for ROTATED channel-mode codes (bf16 rows whose packed segment is 32 chunks
// wide, i.e. 1024..4096 channels): compress-only, fused norm + compress, and the two-record variant that
// also compresses the norm output.
//
// The rotating warp-per-row kernel of hyc_fwd_warp.cuh gives a lane 8 consecutive channels at a time, so of
// the eight butterfly stages of a 256-wide Walsh-Hadamard block three run inside the lane and five cross
// lanes: five shuffles per element, and shuffles share the shared-memory data pipe -- that pipe, not HBM,
// bounds the kernel.  Here a lane owns one CHUNK of CH = segment/32 consecutive channels of every packed
// segment (64 channels x 2 segments at 4 bits and 4096 channels): the stages of strides 1..CH/2 run inside the
// lane on registers and only log2(256/CH) stages (two) cross lanes.
//
// A lane that reads 128 consecutive bytes of a row would hit the same shared-memory banks as its neighbours,
// so a row is staged by ONE tensor copy (cp.async.bulk.tensor, 3-D map [rows][D/64][64 channels]) with the
// 128-byte swizzle: the eight 16-byte pieces of every 128-byte line are stored XOR-ed with the line number,
// and eight neighbouring lanes reading "their" piece j touch eight different bank groups.  The norm output is
// written back over the staged row (same swizzle) and leaves through one tensor store; the two-record variant
// then compresses it from there.  No multicast, no cluster.
//
// Arithmetic (butterfly order, operand order, scale, rounding) is that of the other forward kernels: codes,
// scales and outlier values are bit-identical.
#pragma once
#include <cuda.h>

#include "hyc_fwd_warp.cuh"

namespace hyc {

// One CTA per SM.  The register file is four banks of 16 384 registers, one per warp scheduler, so the warp
// count goes in steps of four: 12 warps leave 168 registers per thread, 8 warps 255.  The rotated row of a lane
// is 128 fp32 values.
// Many rows per warp: 12 warps hide more latency.  Few rows (at most two rounds of 8 warps per SM): a row's own
// latency is what counts, and 8 warps without register spills finish it sooner.
constexpr int kChunkWarpsMany = 12, kChunkWarpsFew = 8;

struct ChunkFwdArgs {
  PackedDev p;
  PackedDev p2;          // two-record variant: the record of the norm output
  int kind;
  float eps;
  const void* weight;
  const void* bias;
  int param_bf16;
  float* rstd;
  float* mean;
  uint32_t off_chan, off_chan2, off_wsm, off_bsm, off_slots, slot_bytes;
  long long wait_cycles;
  uint32_t tx_pad;       // test hook: bytes announced beyond what a copy brings (0 in normal use)
};

// Byte offset, inside a staged row, of the 16-byte piece that holds channels e..e+7 (e a multiple of 8).
__device__ __forceinline__ uint32_t swz_piece(uint32_t e) {
  const uint32_t line = e >> 6, piece = (e >> 3) & 7u;
  return (line << 7) | ((piece ^ (line & 7u)) << 4);
}
__device__ __forceinline__ uint32_t swz_channel(uint32_t c) { return swz_piece(c & ~7u) + ((c & 7u) << 1); }

__device__ __forceinline__ void tensor_load_row(void* dst, const CUtensorMap* map, int row, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(0), "r"(0), "r"(row), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tensor_store_row(const CUtensorMap* map, int row, const void* src) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(0), "r"(0), "r"(row), "r"(smem_u32(src))
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the stores this thread committed have read their shared-memory source
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// ... and have completed
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// UNNORMALISED Walsh-Hadamard transform of blocks of n channels; the lane holds CH consecutive channels as
// CH / 2 pairs and lane l ^ m the chunk m * CH channels away.  Stage order 1, 2, 4, ..., operands
// (lower + upper, lower - upper).  The normalisation 1 / sqrt(n) is a power of two: the caller folds it
// into the scale, exactly.
template <int CH>
__device__ __forceinline__ void rotate_chunk(f32x2 (&v)[CH / 2], int n, int lane) {
  // stride 1: inside a pair
#pragma unroll
  for (int i = 0; i < CH / 2; ++i) {
    float lo, hi;
    f2_split(v[i], lo, hi);
    v[i] = f2_make(lo + hi, lo - hi);
  }
  // strides 2 .. CH / 2: pairs h / 2 apart
#pragma unroll
  for (int h = 1; h < CH / 2; h <<= 1) {
    if (h < 8 || 2 * h < n) {          // blocks are at least 16 wide
#pragma unroll
      for (int i = 0; i < CH / 2; ++i) {
        if ((i & h) == 0) {
          const f32x2 lo = v[i], hi = v[i + h];
          v[i] = f2_add(lo, hi);
          v[i + h] = f2_sub(lo, hi);
        }
      }
    }
  }
  // strides CH ..: the partner chunk lives in another lane
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
    if (m * CH < n) {
      const float sgn = (lane & m) ? -1.f : 1.f;
      const f32x2 sgn2 = f2_make(sgn, sgn);
#pragma unroll
      for (int i = 0; i < CH / 2; ++i) {
        float lo, hi;
        f2_split(v[i], lo, hi);
        const f32x2 o = f2_make(__shfl_xor_sync(0xffffffffu, lo, m), __shfl_xor_sync(0xffffffffu, hi, m));
        v[i] = f2_fma(sgn2, v[i], o);
      }
    }
  }
}

// Outlier channels of one record (`chan`: the list in shared memory; lane l looks after entries l, l + 32, ...):
// keep the staged value, write it out, zero it in the staged row.
__device__ __forceinline__ void chunk_take_outliers(const PackedDev& p, const int* chan, unsigned char* slot, int row, int lane,
                                                    float (&ov)[kWarpOutPerLane]) {
  const int k = p.n_channels;
#pragma unroll
  for (int q = 0; q < kWarpOutPerLane; ++q) {
    ov[q] = 0.f;
    if (lane + 32 * q < k) {
      __nv_bfloat16* at = reinterpret_cast<__nv_bfloat16*>(slot + swz_channel(static_cast<uint32_t>(chan[lane + 32 * q])));
      const __nv_bfloat16 o = *at;
      p.out_value[static_cast<long long>(row) * k + lane + 32 * q] = o;
      ov[q] = __bfloat162float(o);
      *at = __float2bfloat16_rn(0.f);
    }
  }
}

// The lane's share of a staged row: NSEG chunks of CH channels, as raw bf16.
template <int NSEG, int CH>
__device__ __forceinline__ void chunk_load(const unsigned char* slot, int segw, int lane, uint4 (&raw)[NSEG][CH / 8]) {
#pragma unroll
  for (int s = 0; s < NSEG; ++s)
#pragma unroll
    for (int j = 0; j < CH / 8; ++j)
      raw[s][j] = *reinterpret_cast<const uint4*>(slot + swz_piece(static_cast<uint32_t>(s * segw + lane * CH + 8 * j)));
}

// The lane's share from raw bf16 to rotated fp32 pairs (unnormalised, see rotate_chunk).
template <int NSEG, int CH>
__device__ __forceinline__ void chunk_unpack_rotate(const uint4 (&raw)[NSEG][CH / 8], f32x2 (&v)[NSEG][CH / 2], int rotate, int lane) {
#pragma unroll
  for (int s = 0; s < NSEG; ++s) {
#pragma unroll
    for (int j = 0; j < CH / 8; ++j) {
      f32x2 f[4];
      unpack_bf16x8_pairs(raw[s][j], f);
#pragma unroll
      for (int e = 0; e < 4; ++e) v[s][4 * j + e] = f[e];
    }
    rotate_chunk<CH>(v[s], rotate, lane);
  }
}

// Scale and pack the lane's rotated share; writes the record's scales and codes of this row.
template <int BITS, int CH, bool GROUP>
__device__ __forceinline__ void chunk_scale_pack(const PackedDev& p, const f32x2 (&v)[8 / BITS][CH / 2], int row, int lane) {
  using C = CodeTraits<BITS>;
  constexpr int NSEG = C::kSeg;
  constexpr int NPC = CH / 8;
  static_assert(CH <= 128, "one 128-channel scale group per chunk at most");
  const int D = p.cols;
  const int segw = D / NSEG;
  const float qmax = static_cast<float>(C::kHi);
  const float rs = rotate_norm(p.rotate);        // a power of two: scaling by it is exact
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
      // a 128-channel group is one chunk (CH = 128) or 128 / CH neighbouring lanes
#pragma unroll
      for (int o = (128 / CH) >> 1; o > 0; o >>= 1) a8 = fmaxf(a8, __shfl_xor_sync(0xffffffffu, a8, o));
      a8 = __fmul_rn(a8, rs);
      const bool live = a8 > 0.f;
      inv[s] = live ? __fmul_rn(__fdiv_rn(qmax, a8), rs) : rs;
      if ((lane & (128 / CH - 1)) == 0)
        p.scales[static_cast<long long>(row) * (D >> 7) + ((s * segw + lane * CH) >> 7)] = live ? __fdiv_rn(a8, qmax) : 1.f;
    } else {
      amax = fmaxf(amax, a8);
    }
  }
  if (!GROUP) {
    amax = __fmul_rn(warp_max(amax), rs);
    const bool live = amax > 0.f;
    const float inv_row = live ? __fmul_rn(__fdiv_rn(qmax, amax), rs) : rs;
    if (lane == 0) p.scales[row] = live ? __fdiv_rn(amax, qmax) : 1.f;
#pragma unroll
    for (int s = 0; s < NSEG; ++s) inv[s] = inv_row;
  }
  // code = rint((v * rs) * (qmax / absmax)): v * rs is exact, so one fused multiply-add with rs folded into the
  // reciprocal scale rounds the same exact product once
  const float magic = kRoundMagic + static_cast<float>(BITS == 8 ? 128 : C::kOff);
  const f32x2 magic2 = f2_make(magic, magic);
  unsigned char* codes = p.codes + static_cast<long long>(row) * (D * BITS / 8) + lane * CH;
#pragma unroll
  for (int u = 0; u < NPC; u += 2) {
    uint32_t w[4] = {pack_cancel<BITS>(), pack_cancel<BITS>(), pack_cancel<BITS>(), pack_cancel<BITS>()};
#pragma unroll
    for (int s = 0; s < NSEG; ++s) {
      const f32x2 inv2 = f2_make(inv[s], inv[s]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {            // pair e of the two units: channels 2e, 2e + 1 of the 16
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

// NK: 0 compress only, 1 RMSNorm (plain or Gemma), 2 LayerNorm;  CH: channels of a segment per lane;
// DUAL: a second record (a.p2, with its own outlier channels) takes the compressed norm output.
// RN: the rotation block when the kernel is compiled for one (256: the butterfly stages then carry no test of the
// block size and are one stretch of code), or 0: the record's own, read at run time.  Only the many-warps build
// for long inputs exists with RN = 256: inside a training step a launch starts with cold instruction caches, and
// there the smaller code of the few-warps build counts for more.
template <int BITS, int NK, int CH, bool GROUP, bool DUAL, int WARPS, int RN = 0>
__global__ void __launch_bounds__(WARPS * 32, 1)
fwd_n_chunk_kernel(const __grid_constant__ ChunkFwdArgs a, const __grid_constant__ CUtensorMap in_map,
                   const __grid_constant__ CUtensorMap y_map) {
  using C = CodeTraits<BITS>;
  constexpr int NSEG = C::kSeg;
  constexpr int NPC = CH / 8;
  constexpr bool NORM = NK != 0;
  constexpr bool ln = NK == 2;
  static_assert(CH >= 32 && CH <= 128 && NSEG * CH <= 128, "a lane holds at most 128 channels");
  static_assert(!DUAL || NORM, "the second record is the norm output's");
  constexpr bool FUSE = WARPS <= 8;
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  const int D = p.cols;
  const int segw = D / NSEG;                  // == 32 * CH
  const int k = p.n_channels;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
  const float inv_d = 1.0f / static_cast<float>(D);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  int* chan = reinterpret_cast<int*>(smem + a.off_chan);
  int* chan2 = reinterpret_cast<int*>(smem + a.off_chan2);
  // norm weight (and bias) as fp32 in two planes: floats 0..3 and 4..7 of every group of eight channels, each
  // plane laid out like a staged row (16 bytes per group, same swizzle), so a lane's reads are conflict-free
  unsigned char* wsm = smem + a.off_wsm;
  unsigned char* bsm = smem + a.off_bsm;
  const uint32_t plane = static_cast<uint32_t>(D) * 2u;
  // two slots per warp: the row after this one is already travelling while this one is worked on
  // (the swizzle pattern repeats every 1024 bytes of ADDRESS: slots start on such a boundary whatever the
  // base of the dynamic shared memory is)
  unsigned char* slots = smem + a.off_slots + ((1024u - (smem_u32(smem) & 1023u)) & 1023u) +
                         static_cast<size_t>(warp) * 2u * a.slot_bytes;
  uint64_t* bar2 = &bars[2 * warp];
  const uint32_t row_bytes = static_cast<uint32_t>(D) * 2u;
  // row numbers fit 30 bits (checked by the host): 32-bit arithmetic in the loop
  const int rows = static_cast<int>(p.rows), stride = static_cast<int>(gridDim.x) * W;
  int row = static_cast<int>(blockIdx.x) * W + warp;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2 * W; ++i) mbar_init(&bars[i], 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (lane == 0) {
    for (int s = 0; s < 2; ++s) {
      const int r = row + s * stride;
      if (r < rows) {
        mbar_expect_tx(&bar2[s], row_bytes + a.tx_pad);
        tensor_load_row(slots + s * a.slot_bytes, &in_map, r, &bar2[s]);
      }
    }
  }
  for (int j = threadIdx.x; j < k; j += blockDim.x) chan[j] = p.channels[j];
  if (DUAL)
    for (int j = threadIdx.x; j < a.p2.n_channels; j += blockDim.x) chan2[j] = a.p2.channels[j];
  if (NORM) {
    const float plus = a.kind == HYC_NORM_RMS_GEMMA ? 1.f : 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      const uint32_t at = swz_piece(static_cast<uint32_t>(c & ~7)) + ((c >> 2) & 1) * plane + ((c & 3) << 2);
      *reinterpret_cast<float*>(wsm + at) = (a.param_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.weight)[c])
                                                         : static_cast<const float*>(a.weight)[c]) + plus;
      if (ln)
        *reinterpret_cast<float*>(bsm + at) = a.param_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.bias)[c])
                                                          : static_cast<const float*>(a.bias)[c];
    }
  }
  __syncthreads();
  uint32_t ph = 0;
  int st = 0;
  for (; row < rows; row += stride) {
    unsigned char* slot = slots + st * a.slot_bytes;
    uint64_t* bar = &bar2[st];
    if (!mbar_wait_bounded(bar, ph, a.wait_cycles)) {
      if (lane == 0 && p.status) atomicOr(p.status, kStatusWaitExpired);
      // the copy into the other slot may still be in flight: give it a bounded chance to land
      if (row + stride < rows) (void)mbar_wait_bounded(&bar2[st ^ 1], st ? ph ^ 1u : ph, a.wait_cycles);
      break;
    }
    const int next = row + 2 * stride;
    float ov[kWarpOutPerLane];
    chunk_take_outliers(p, chan, slot, row, lane, ov);
    __syncwarp();
    uint4 raw[NSEG][NPC];
    chunk_load<NSEG, CH>(slot, segw, lane, raw);
    f32x2 v[NSEG][CH / 2];
    if (!NORM) {
      // every lane has what it needs: hand the slot back to the copy engine
      __syncwarp();
      if (lane == 0 && next < rows) {
        fence_proxy_async();
        mbar_expect_tx(bar, row_bytes + a.tx_pad);
        tensor_load_row(slot, &in_map, next, bar);
      }
      chunk_unpack_rotate<NSEG, CH>(raw, v, RN ? RN : p.rotate, lane);
    } else {
      // ---- statistics of the norm (the zeroed outlier channels still belong to them)
      float mean = 0.f;
      if (ln) {
        f32x2 s2 = f2_make(0.f, 0.f);
#pragma unroll
        for (int s = 0; s < NSEG; ++s)
#pragma unroll
          for (int j = 0; j < NPC; ++j) {
            f32x2 f[4];
            unpack_bf16x8_pairs(raw[s][j], f);
#pragma unroll
            for (int e = 0; e < 4; ++e) s2 = f2_add(s2, f[e]);
          }
        float lo, hi;
        f2_split(s2, lo, hi);
        float s1 = lo + hi;
#pragma unroll
        for (int q = 0; q < kWarpOutPerLane; ++q) s1 += ov[q];
        mean = warp_sum(s1) * inv_d;
#pragma unroll
        for (int s = 0; s < NSEG; ++s)
#pragma unroll
          for (int j = 0; j < NPC; ++j) forget_unpacked(raw[s][j]);
      }
      const f32x2 mean2 = f2_make(mean, mean);
      f32x2 ss2 = f2_make(0.f, 0.f);
#pragma unroll
      for (int s = 0; s < NSEG; ++s)
#pragma unroll
        for (int j = 0; j < NPC; ++j) {
          f32x2 f[4];
          unpack_bf16x8_pairs(raw[s][j], f);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const f32x2 c = ln ? f2_sub(f[e], mean2) : f[e];
            ss2 = f2_fma(c, c, ss2);
          }
        }
      float ss;
      {
        float lo, hi;
        f2_split(ss2, lo, hi);
        ss = lo + hi;
      }
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q)
        if (lane + 32 * q < k) ss += ln ? ((ov[q] - mean) * (ov[q] - mean) - mean * mean) : ov[q] * ov[q];
      ss = warp_sum(ss);
      const float rstd = 1.0f / sqrtf(ss * inv_d + a.eps);
      if (lane == 0) {
        a.rstd[row] = rstd;
        if (ln) a.mean[row] = mean;
      }
#pragma unroll
      for (int s = 0; s < NSEG; ++s)
#pragma unroll
        for (int j = 0; j < NPC; ++j) forget_unpacked(raw[s][j]);
      // ---- the norm output takes the row's place in the slot; with registers to spare (the 8-warp build) the
      //      same unpacked values go straight into the rotation, else the rotation unpacks them again
      const f32x2 rstd2 = f2_make(rstd, rstd);
#pragma unroll
      for (int s = 0; s < NSEG; ++s) {
#pragma unroll
        for (int j = 0; j < NPC; ++j) {
          const uint32_t at = swz_piece(static_cast<uint32_t>(s * segw + lane * CH + 8 * j));
          f32x2 f[4];
          unpack_bf16x8_pairs(raw[s][j], f);
          const ulonglong2 w0 = *reinterpret_cast<const ulonglong2*>(wsm + at);
          const ulonglong2 w1 = *reinterpret_cast<const ulonglong2*>(wsm + plane + at);
          const f32x2 wv[4] = {w0.x, w0.y, w1.x, w1.y};
          uint32_t y[4];
          if (ln) {
            const ulonglong2 b0 = *reinterpret_cast<const ulonglong2*>(bsm + at);
            const ulonglong2 b1 = *reinterpret_cast<const ulonglong2*>(bsm + plane + at);
            const f32x2 bv[4] = {b0.x, b0.y, b1.x, b1.y};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float lo, hi;
              f2_split(f2_fma(f2_mul(f2_sub(f[e], mean2), rstd2), wv[e], bv[e]), lo, hi);
              y[e] = pack_bf16x2(lo, hi);
            }
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float lo, hi;
              f2_split(f2_mul(f2_mul(f[e], rstd2), wv[e]), lo, hi);
              y[e] = pack_bf16x2(lo, hi);
            }
          }
          *reinterpret_cast<uint4*>(slot + at) = make_uint4(y[0], y[1], y[2], y[3]);
          if (FUSE) {
#pragma unroll
            for (int e = 0; e < 4; ++e) v[s][4 * j + e] = f[e];
          }
        }
        if (FUSE) rotate_chunk<CH>(v[s], RN ? RN : p.rotate, lane);
        else if (s + 1 < NSEG) asm volatile("" ::: "memory");
      }
      // the vector stores wrote the norm of the zeroed value at the outlier channels: order them before the
      // scalar stores of the real values (same warp, other lanes)
      __syncwarp();
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q) {
        if (lane + 32 * q < k) {
          const uint32_t c = static_cast<uint32_t>(chan[lane + 32 * q]);
          const uint32_t at = swz_piece(c & ~7u) + ((c >> 2) & 1u) * plane + ((c & 3u) << 2);
          const float wv = *reinterpret_cast<const float*>(wsm + at);
          const float y = ln ? ((ov[q] - mean) * rstd * wv + *reinterpret_cast<const float*>(bsm + at)) : (ov[q] * rstd * wv);
          *reinterpret_cast<__nv_bfloat16*>(slot + swz_channel(c)) = __float2bfloat16_rn(y);
        }
      }
      // shared-memory writes of every lane -> visible to the tensor store
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        tensor_store_row(&y_map, row, slot);
        bulk_commit();
      }
      if (!FUSE) {
#pragma unroll
        for (int s = 0; s < NSEG; ++s)
#pragma unroll
          for (int j = 0; j < NPC; ++j) forget_unpacked(raw[s][j]);
        chunk_unpack_rotate<NSEG, CH>(raw, v, RN ? RN : p.rotate, lane);
      }
    }
    // ---- the record of the row itself, from the registers
    chunk_scale_pack<BITS, CH, GROUP>(p, v, row, lane);
    if (DUAL) {
      // ---- the record of the norm output, from the slot (once the store has read it)
      if (lane == 0) bulk_wait_read();
      __syncwarp();
      float ov2[kWarpOutPerLane];
      chunk_take_outliers(a.p2, chan2, slot, row, lane, ov2);
      __syncwarp();
      chunk_load<NSEG, CH>(slot, segw, lane, raw);
      chunk_unpack_rotate<NSEG, CH>(raw, v, RN ? RN : p.rotate, lane);
      chunk_scale_pack<BITS, CH, GROUP>(a.p2, v, row, lane);
    }
    if (NORM) {
      __syncwarp();
      if (lane == 0) {
        bulk_wait_read();
        if (next < rows) {
          fence_proxy_async();
          mbar_expect_tx(bar, row_bytes + a.tx_pad);
          tensor_load_row(slot, &in_map, next, bar);
        }
      }
    }
    if (st) ph ^= 1u;
    st ^= 1;
  }
  // no tensor store of this thread may still be reading shared memory when the CTA leaves
  if (NORM && lane == 0) bulk_wait_all();
}

// ------------------------------------------------------------------ host: eligibility and launch

struct ChunkPlan {
  bool ok, dual;
  int ch;          // channels of a segment per lane (instantiated: 32, 64, 128)
  int warps, grid;
  uint32_t off_chan, off_chan2, off_wsm, off_bsm, off_slots, slot_bytes, total;
};

typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
TensorMapEncodeFn tensor_map_encoder();       // cuTensorMapEncodeTiled through the runtime's driver entry point

// A [rows][cols] bf16 matrix (row stride in elements) as a 3-D tensor of 64-channel lines, one row per box.
inline bool row_tensor_map(CUtensorMap* map, const void* base, long long rows, int cols, long long row_stride) {
  TensorMapEncodeFn fn = tensor_map_encoder();
  if (!fn) return false;
  const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(cols / 64), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[2] = {128, static_cast<cuuint64_t>(row_stride) * 2u};
  const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(cols / 64), 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Rotated bf16 rows in the plain layout whose packed segment is 32 chunks of 32, 64 or 128 channels, at most
// 128 channels per lane and 128 outlier channels; the rotation block divides the segment.
// `q2`: second record for the norm output (two-record variant), or nullptr.
inline ChunkPlan plan_chunk_fwd(const hyc_packed* q, const hyc_dense* x, bool norm, bool ln, const hyc_packed* q2 = nullptr) {
  ChunkPlan w;
  memset(&w, 0, sizeof(w));
  if (q2) {
    if (!norm || q2->mode != HYC_MODE_N || q2->bits != q->bits || q2->group != q->group || q2->rotate != q->rotate ||
        q2->cols != q->cols || q2->rows != q->rows || q2->n_channels > 32 * kWarpOutPerLane)
      return w;
    // measured (4096 channels, rotation 256; one launch against norm + compress and compress of the output):
    // 25 against 29 us at 2048 rows, 44 against 50 at 4096, 139 against 138 at 16384, 519 against 463 at 65536
    if (q2->rotate && q->rows > 8192) return w;
    w.dual = true;
  }
  if (q->mode != HYC_MODE_N || x->dtype != HYC_BF16 || x->chunks != 1 || !q->rotate) return w;
  if (q->bits != 2 && q->bits != 4 && q->bits != 8) return w;
  if (q->n_channels > 32 * kWarpOutPerLane) return w;
  if (g_tune_threads || g_tune_stages || g_tune_ctas) return w;     // explicit tuning addresses the CTA-per-row kernels
  if (q->rows > 0x3fffffffLL || (x->row_stride * 2) % 16 != 0) return w;
  const int D = q->cols, nseg = 8 / q->bits;
  const int segw = D / nseg;
  if (D % nseg || segw % 32) return w;
  const int ch = segw / 32;
  if ((ch != 32 && ch != 64 && ch != 128) || ch * nseg > 128) return w;
  if (q->rotate > segw || segw % q->rotate) return w;
  if (!tensor_map_encoder()) return w;
  w.ch = ch;
  // (the two-record variant holds more state: its 12-warp build spills and is slower than two launches)
  const int choices[2] = {(q2 || q->rows <= 2LL * kChunkWarpsFew * sm_count()) ? kChunkWarpsFew : kChunkWarpsMany, kChunkWarpsFew};
  for (int c = 0; c < 2; ++c) {
    const int warps = choices[c];
    uint32_t off = 64 * 8;                                   // two mbarriers per warp
    auto take = [&](uint32_t bytes, uint32_t align) { off = align_up(off, align); uint32_t o = off; off += bytes; return o; };
    w.off_chan = take((q->n_channels > 0 ? q->n_channels : 1) * 4, 16);
    w.off_chan2 = take((q2 && q2->n_channels > 0 ? q2->n_channels : 1) * 4, 16);
    w.off_wsm = norm ? take(D * 4, 128) : 0;
    w.off_bsm = ln ? take(D * 4, 128) : 0;
    w.slot_bytes = static_cast<uint32_t>(D) * 2u;            // a multiple of 1024: the swizzle pattern's period
    w.off_slots = take(w.slot_bytes * warps * 2, 1024);
    w.total = off + 1024;                                    // room to start the slots on a 1024-byte address
    w.warps = warps;
    if (w.total <= kSmemPerCtaMax) break;
    w.warps = 0;
  }
  if (!w.warps) return w;
  long long grid = sm_count();
  const long long need = (q->rows + w.warps - 1) / w.warps;
  if (grid > need) grid = need;
  w.grid = static_cast<int>(grid);
  w.ok = true;
  return w;
}

template <int BITS, int CH>
int launch_fwd_chunk_one(const ChunkFwdArgs& a, const ChunkPlan& w, bool norm, const CUtensorMap& in_map,
                         const CUtensorMap& y_map, cudaStream_t stream) {
#define HYC_CHUNK_LAUNCH_W(NK, GROUP, DUAL, WARPS)                                              \
  {                                                                                             \
    auto kern = fwd_n_chunk_kernel<BITS, NK, CH, GROUP, DUAL, WARPS>;                           \
    int rc = set_smem(kern, w.total);                                                           \
    if (rc) return rc;                                                                          \
    kern<<<w.grid, WARPS * 32, w.total, stream>>>(a, in_map, y_map); HYC_LAUNCHED();            \
  }
#define HYC_CHUNK_LAUNCH(NK, GROUP, DUAL)                                                       \
  {                                                                                             \
    if (w.warps == kChunkWarpsFew) HYC_CHUNK_LAUNCH_W(NK, GROUP, DUAL, kChunkWarpsFew)          \
    else if (!DUAL && a.p.rotate == 256) {                                                      \
      auto kern = fwd_n_chunk_kernel<BITS, NK, CH, GROUP, false, kChunkWarpsMany, 256>;         \
      int rc = set_smem(kern, w.total);                                                         \
      if (rc) return rc;                                                                        \
      kern<<<w.grid, kChunkWarpsMany * 32, w.total, stream>>>(a, in_map, y_map); HYC_LAUNCHED(); \
    } else HYC_CHUNK_LAUNCH_W(NK, GROUP, DUAL, kChunkWarpsMany)                                 \
  }
#define HYC_CHUNK_NK(NK)                                                                        \
  if (a.p.group) {                                                                              \
    if (w.dual) { if constexpr (NK != 0) HYC_CHUNK_LAUNCH(NK, true, true) }                     \
    else HYC_CHUNK_LAUNCH(NK, true, false)                                                      \
  } else {                                                                                      \
    if (w.dual) { if constexpr (NK != 0) HYC_CHUNK_LAUNCH(NK, false, true) }                    \
    else HYC_CHUNK_LAUNCH(NK, false, false)                                                     \
  }
  const int nk = !norm ? 0 : a.kind == HYC_NORM_LAYER ? 2 : 1;
  if (w.dual && nk == 0) return HYC_ERR_SHAPE;
  if (nk == 2) { HYC_CHUNK_NK(2) } else if (nk == 1) { HYC_CHUNK_NK(1) } else { HYC_CHUNK_NK(0) }
#undef HYC_CHUNK_NK
#undef HYC_CHUNK_LAUNCH
#undef HYC_CHUNK_LAUNCH_W
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? HYC_OK : cuda_fail(e, "fwd_n_chunk_kernel launch");
}

int launch_fwd_chunk_b2(const ChunkFwdArgs& a, const ChunkPlan& w, bool norm, const CUtensorMap& in_map,
                        const CUtensorMap& y_map, cudaStream_t stream);
int launch_fwd_chunk_b4(const ChunkFwdArgs& a, const ChunkPlan& w, bool norm, const CUtensorMap& in_map,
                        const CUtensorMap& y_map, cudaStream_t stream);
int launch_fwd_chunk_b8(const ChunkFwdArgs& a, const ChunkPlan& w, bool norm, const CUtensorMap& in_map,
                        const CUtensorMap& y_map, cudaStream_t stream);

}  // namespace hyc
