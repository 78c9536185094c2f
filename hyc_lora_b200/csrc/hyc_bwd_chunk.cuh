// Chunk-per-lane CONSUMER kernels for rotated channel-mode records (bf16 rows whose packed segment is 32 chunks of
// 32, 64 or 128 channels wide, i.e. 1024..4096 channels): decompress, and decompress + norm backward with a
// frozen norm weight and a bf16 gradient (the adapter case).
//
// The rotated consumers of hyc_bwd_warp.cuh / hyc_bwd_fast.cuh give a lane 8 consecutive channels at a time:
// five of the eight butterfly stages of a 256-block cross lanes (five shuffles per element, the shared-memory
// data pipe bounds them).  Here, as in hyc_fwd_chunk.cuh, a lane owns one chunk of segment/32 consecutive
// channels of every packed segment, so six stages are register butterflies on packed fp32 pairs and two cross
// lanes.  A lane's codes are CH consecutive bytes of the row: they come straight from global memory, one row
// ahead (16 registers), together with the row's scale, statistics and stored outlier values.  The gradient row
// is staged by a tensor copy with the 128-byte swizzle (two slots per warp); the result row is built in a third
// slot in the same swizzle and leaves through one tensor store.
//
// Outlier channels hold the stored original, not what the inverse rotation leaves in their place: the rebuilt
// row passes through the result slot as bf16, where the lanes that look after an outlier channel read what
// the rotation left there (to take it out of the row sum) and later overwrite the channel's result.
//
// Arithmetic is that of the other consumers: (code - offset) * scale as one rounded product per element BEFORE the
// butterflies (the 1 / sqrt(n) of the transform, a power of two, is folded into the scale: exact), fixed stage
// and operand order, one rounding to bf16 of the rebuilt value.
#pragma once
#include "hyc_fwd_chunk.cuh"

namespace hyc {

constexpr int kChunkBwdWarps = 8;
enum { kChunkDecompress = 0, kChunkNormBwdRms = 1, kChunkNormBwdLn = 2 };

struct ChunkBwdArgs {
  PackedDev p;
  int kind;               // norm kind (Gemma adds 1 to the weight)
  const void* weight;
  int param_bf16;
  const float* rstd;
  const float* mean;
  int ref_compat_c2;
  uint32_t off_chan, off_wsm, off_slots, slot_bytes;
  long long wait_cycles;
  uint32_t tx_pad;       // test hook: bytes announced beyond what a copy brings (0 in normal use)
};

// codes of one 8-channel unit pair -> (code - offset) * scale as fp32 pairs, for segment s
template <int BITS>
__device__ __forceinline__ void chunk_dequant16(const uint4& cw, int s, f32x2 sc2, f32x2 (&f)[8]) {
  using C = CodeTraits<BITS>;
  uint32_t w[4] = {cw.x, cw.y, cw.z, cw.w};
  float bias;
  if (BITS == 8) {
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] ^= 0x80808080u;       // two's complement -> offset 128
    bias = 8388608.f + 128.f;
  } else {
    const uint32_t m = 0x01010101u * C::kMask;
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = (w[i] >> (s * BITS)) & m;
    bias = 8388608.f + static_cast<float>(C::kOff);
  }
  const f32x2 bias2 = f2_make(bias, bias);
  // integer -> float through the mantissa of 2^23 (one byte permute per element); the product is rounded on its
  // own: fused into the first butterfly's addition the sums would round differently from the oracle's
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const f32x2 lo = f2_make(__uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7650)),
                             __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7651)));
    const f32x2 hi = f2_make(__uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7652)),
                             __uint_as_float(__byte_perm(w[i], 0x4B000000u, 0x7653)));
    f[2 * i] = f2_mul(f2_sub(lo, bias2), sc2);
    f[2 * i + 1] = f2_mul(f2_sub(hi, bias2), sc2);
  }
}

// round both halves to bf16 (round to nearest even): the packed pair, and the rounded values as fp32
__device__ __forceinline__ uint32_t f2_to_bf16x2(f32x2 v, f32x2& rounded) {
  float lo, hi;
  f2_split(v, lo, hi);
  const uint32_t b = pack_bf16x2(lo, hi);
  rounded = f2_make(__uint_as_float(b << 16), __uint_as_float(b & 0xffff0000u));
  return b;
}

// (decompress needs nothing row-wide: it rebuilds and stores one segment's chunk at a time -- with two or four
// segments that is 64 or 32 fp32 values in flight instead of 128, and two CTAs share an SM)
// RN: the rotation block when the kernel is compiled for one (256: no test of the block size in front of the
// butterfly stages), or 0: the record's own, read at run time.  The launcher takes RN = 256 for long inputs only:
// inside a training step a launch starts with cold instruction caches, where the smaller code counts for more.
template <int BITS, int OP, int CH, bool GROUP, int RN = 0>
__global__ void __launch_bounds__(kChunkBwdWarps * 32, (OP == kChunkDecompress && BITS < 8) ? 2 : 1)
bwd_n_chunk_kernel(const __grid_constant__ ChunkBwdArgs a, const __grid_constant__ CUtensorMap dy_map,
                   const __grid_constant__ CUtensorMap out_map) {
  using C = CodeTraits<BITS>;
  constexpr int NSEG = C::kSeg;
  constexpr int NPC = CH / 8;
  constexpr int NCW = CH / 16;                 // 16-byte pieces of codes per lane
  constexpr bool NORMB = OP != kChunkDecompress;
  constexpr bool ln = OP == kChunkNormBwdLn;
  static_assert(CH >= 32 && CH <= 128 && NSEG * CH <= 128, "a lane holds at most 128 channels");
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  const int D = p.cols;
  const int segw = D / NSEG;                  // == 32 * CH
  const int k = p.n_channels;
  const int G = GROUP ? (D >> 7) : 1;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, W = blockDim.x >> 5;
  const float inv_d = 1.0f / static_cast<float>(D);
  const float rs = rotate_norm(p.rotate);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  int* chan = reinterpret_cast<int*>(smem + a.off_chan);
  unsigned char* wsm = smem + a.off_wsm;                      // two planes, swizzled like a staged row
  const uint32_t plane = static_cast<uint32_t>(D) * 2u;
  // per warp: the result slot, then (norm backward) two gradient slots
  constexpr int SLOTS = NORMB ? 3 : 1;
  unsigned char* oslot = smem + a.off_slots + ((1024u - (smem_u32(smem) & 1023u)) & 1023u) +
                         static_cast<size_t>(warp) * SLOTS * a.slot_bytes;
  unsigned char* gslots = oslot + a.slot_bytes;
  uint64_t* bar2 = &bars[2 * warp];
  const uint32_t row_bytes = static_cast<uint32_t>(D) * 2u;
  const int rows = static_cast<int>(p.rows), stride = static_cast<int>(gridDim.x) * W;
  int row = static_cast<int>(blockIdx.x) * W + warp;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2 * W; ++i) mbar_init(&bars[i], 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (NORMB && lane == 0) {
    for (int s = 0; s < 2; ++s) {
      const int r = row + s * stride;
      if (r < rows) {
        mbar_expect_tx(&bar2[s], row_bytes + a.tx_pad);
        tensor_load_row(gslots + s * a.slot_bytes, &dy_map, r, &bar2[s]);
      }
    }
  }
  for (int j = threadIdx.x; j < k; j += blockDim.x) chan[j] = max(0, min(D - 1, p.channels[j]));
  if (NORMB) {
    const float plus = a.kind == HYC_NORM_RMS_GEMMA ? 1.f : 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      const uint32_t at = swz_piece(static_cast<uint32_t>(c & ~7)) + ((c >> 2) & 1) * plane + ((c & 3) << 2);
      *reinterpret_cast<float*>(wsm + at) = (a.param_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.weight)[c])
                                                         : static_cast<const float*>(a.weight)[c]) + plus;
    }
  }
  __syncthreads();
  const uint32_t cb = static_cast<uint32_t>(D) * BITS / 8;    // bytes of codes per row
  // what the next row needs from global memory, fetched one row ahead
  uint4 cw_nxt[NCW];
  float sc_nxt[NSEG], rstd_nxt = 0.f, mean_nxt = 0.f;
  float ov_nxt[kWarpOutPerLane];
  auto fetch = [&](int r) {
    const unsigned char* codes = p.codes + static_cast<long long>(r) * cb + lane * CH;
#pragma unroll
    for (int i = 0; i < NCW; ++i) cw_nxt[i] = __ldg(reinterpret_cast<const uint4*>(codes) + i);
#pragma unroll
    for (int s = 0; s < NSEG; ++s)
      sc_nxt[s] = __ldg(p.scales + static_cast<long long>(r) * G + (GROUP ? ((s * segw + lane * CH) >> 7) : 0));
    if (NORMB) {
      rstd_nxt = __ldg(a.rstd + r);
      if (ln) mean_nxt = __ldg(a.mean + r);
    }
#pragma unroll
    for (int q = 0; q < kWarpOutPerLane; ++q)
      ov_nxt[q] = (lane + 32 * q) < k ? __bfloat162float(p.out_value[static_cast<long long>(r) * k + lane + 32 * q]) : 0.f;
  };
  if (row < rows) fetch(row);

  uint32_t ph = 0;
  int st = 0;
  bool stored = false;        // lane 0: a tensor store of this warp may still be reading the result slot
  for (; row < rows; row += stride) {
    uint4 cw[NCW];
    float sc[NSEG], ov[kWarpOutPerLane];
#pragma unroll
    for (int i = 0; i < NCW; ++i) cw[i] = cw_nxt[i];
#pragma unroll
    for (int s = 0; s < NSEG; ++s) sc[s] = sc_nxt[s];
#pragma unroll
    for (int q = 0; q < kWarpOutPerLane; ++q) ov[q] = ov_nxt[q];
    const float rstd = rstd_nxt, mean = mean_nxt;
    if (row + stride < rows) fetch(row + stride);
    // ---- rebuild the lane's share: dequantise, rotate back, round to bf16
    f32x2 v[NORMB ? NSEG : 1][CH / 2];
    auto rebuild = [&](int s, f32x2 (&vs)[CH / 2]) {
      const float scs = __fmul_rn(sc[s], rs);                 // exact: rs is a power of two
      const f32x2 sc2 = f2_make(scs, scs);
#pragma unroll
      for (int i = 0; i < NCW; ++i) {
        f32x2 f[8];
        chunk_dequant16<BITS>(cw[i], s, sc2, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) vs[8 * i + e] = f[e];
      }
      rotate_chunk<CH>(vs, RN ? RN : p.rotate, lane);
    };
    auto to_slot = [&](int s, f32x2 (&vs)[CH / 2]) {
#pragma unroll
      for (int j = 0; j < NPC; ++j) {
        uint32_t b[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) b[e] = f2_to_bf16x2(vs[4 * j + e], vs[4 * j + e]);
        *reinterpret_cast<uint4*>(oslot + swz_piece(static_cast<uint32_t>(s * segw + lane * CH + 8 * j))) = make_uint4(b[0], b[1], b[2], b[3]);
      }
    };
    if (NORMB) {
#pragma unroll
      for (int s = 0; s < NSEG; ++s) rebuild(s, v[s]);
    } else {
      rebuild(0, v[0]);
    }
    // the result slot is free once the previous row's store has read it
    if (lane == 0 && stored) bulk_wait_read();
    __syncwarp();
    if (NORMB) {
#pragma unroll
      for (int s = 0; s < NSEG; ++s) to_slot(s, v[s]);
    } else {
      to_slot(0, v[0]);
#pragma unroll
      for (int s = 1; s < NSEG; ++s) {
        rebuild(s, v[0]);
        to_slot(s, v[0]);
      }
    }
    __syncwarp();
    if (!NORMB) {
      // ---- decompress: the stored originals take the outlier channels' places, the row leaves
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q)
        if (lane + 32 * q < k)
          *reinterpret_cast<__nv_bfloat16*>(oslot + swz_channel(static_cast<uint32_t>(chan[lane + 32 * q]))) = __float2bfloat16_rn(ov[q]);
    } else {
      unsigned char* gslot = gslots + st * a.slot_bytes;
      uint64_t* bar = &bar2[st];
      if (!mbar_wait_bounded(bar, ph, a.wait_cycles)) {
        if (lane == 0 && p.status) atomicOr(p.status, kStatusWaitExpired);
        if (row + stride < rows) (void)mbar_wait_bounded(&bar2[st ^ 1], st ? ph ^ 1u : ph, a.wait_cycles);
        break;
      }
      // ---- outlier channels: what the rotation left in their place leaves the row sum, the original enters it
      float wq[kWarpOutPerLane], corr = 0.f;
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q) {
        wq[q] = 0.f;
        if (lane + 32 * q < k) {
          const uint32_t c = static_cast<uint32_t>(chan[lane + 32 * q]);
          const uint32_t at = swz_piece(c & ~7u) + ((c >> 2) & 1u) * plane + ((c & 3u) << 2);
          const float left = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(oslot + swz_channel(c)));
          wq[q] = *reinterpret_cast<const float*>(wsm + at) * __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(gslot + swz_channel(c)));
          corr = fmaf(ov[q] - left, wq[q], corr);
        }
      }
      // ---- pass 1: S1 = sum x * w dy, S2 = sum w dy
      f32x2 s1 = f2_make(0.f, 0.f), s2 = f2_make(0.f, 0.f);
#pragma unroll
      for (int s = 0; s < NSEG; ++s)
#pragma unroll
        for (int j = 0; j < NPC; ++j) {
          const uint32_t at = swz_piece(static_cast<uint32_t>(s * segw + lane * CH + 8 * j));
          f32x2 g[4];
          unpack_bf16x8_pairs(*reinterpret_cast<const uint4*>(gslot + at), g);
          const ulonglong2 w0 = *reinterpret_cast<const ulonglong2*>(wsm + at);
          const ulonglong2 w1 = *reinterpret_cast<const ulonglong2*>(wsm + plane + at);
          const f32x2 wv[4] = {w0.x, w0.y, w1.x, w1.y};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const f32x2 wd = f2_mul(wv[e], g[e]);
            s1 = f2_fma(v[s][4 * j + e], wd, s1);
            s2 = f2_add(s2, wd);
          }
        }
      float s1s, s2s;
      {
        float lo, hi;
        f2_split(s1, lo, hi);
        s1s = warp_sum(lo + hi + corr);
        f2_split(s2, lo, hi);
        s2s = warp_sum(lo + hi);
      }
      const float c1 = rstd * (s1s - mean * s2s) * inv_d;
      const float c2 = (ln || a.ref_compat_c2) ? s2s * inv_d : 0.f;
      // ---- pass 2: dx = (w dy - (x-hat * c1 + c2)) * rstd = ka * w dy + kb * x + kc with three row constants
      const float ka = rstd, kb = -rstd * rstd * c1, kc = (mean * rstd * c1 - c2) * rstd;
      const f32x2 ka2 = f2_make(ka, ka), kb2 = f2_make(kb, kb), kc2 = f2_make(kc, kc);
#pragma unroll
      for (int s = 0; s < NSEG; ++s)
#pragma unroll
        for (int j = 0; j < NPC; ++j) {
          const uint32_t at = swz_piece(static_cast<uint32_t>(s * segw + lane * CH + 8 * j));
          f32x2 g[4];
          unpack_bf16x8_pairs(*reinterpret_cast<const uint4*>(gslot + at), g);
          const ulonglong2 w0 = *reinterpret_cast<const ulonglong2*>(wsm + at);
          const ulonglong2 w1 = *reinterpret_cast<const ulonglong2*>(wsm + plane + at);
          const f32x2 wv[4] = {w0.x, w0.y, w1.x, w1.y};
          uint32_t b[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float lo, hi;
            f2_split(f2_fma(ka2, f2_mul(wv[e], g[e]), f2_fma(kb2, v[s][4 * j + e], kc2)), lo, hi);
            b[e] = pack_bf16x2(lo, hi);
          }
          *reinterpret_cast<uint4*>(oslot + at) = make_uint4(b[0], b[1], b[2], b[3]);
        }
      // every lane is done with the gradient slot: the row after next may start travelling
      __syncwarp();
      const int next = row + 2 * stride;
      if (lane == 0 && next < rows) {
        fence_proxy_async();
        mbar_expect_tx(bar, row_bytes + a.tx_pad);
        tensor_load_row(gslot, &dy_map, next, bar);
      }
      // the vector stores above come before the outlier channels' results (other lanes)
#pragma unroll
      for (int q = 0; q < kWarpOutPerLane; ++q)
        if (lane + 32 * q < k)
          *reinterpret_cast<__nv_bfloat16*>(oslot + swz_channel(static_cast<uint32_t>(chan[lane + 32 * q]))) =
              __float2bfloat16_rn(fmaf(ka, wq[q], fmaf(kb, ov[q], kc)));
      if (st) ph ^= 1u;
      st ^= 1;
    }
    // shared-memory writes of every lane -> visible to the tensor store
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) {
      tensor_store_row(&out_map, row, oslot);
      bulk_commit();
      stored = true;
    }
  }
  // no tensor store of this thread may still be reading shared memory when the CTA leaves
  if (lane == 0) bulk_wait_all();
}

// ------------------------------------------------------------------ host: eligibility and launch

struct ChunkBwdPlan {
  bool ok;
  int ch, grid;
  uint32_t off_chan, off_wsm, off_slots, slot_bytes, total;
};

// Rotated channel-mode records of the shapes hyc_fwd_chunk.cuh takes; `norm`: norm backward (three slots per warp
// and the weight planes) instead of decompress.
inline ChunkBwdPlan plan_chunk_bwd(const hyc_packed* q, bool norm) {
  ChunkBwdPlan w;
  memset(&w, 0, sizeof(w));
  static const bool off_env = getenv("HYC_BWD_CHUNK") && getenv("HYC_BWD_CHUNK")[0] == '0';
  if (off_env) return w;
  if (q->mode != HYC_MODE_N || !q->rotate) return w;
  if (q->bits != 2 && q->bits != 4 && q->bits != 8) return w;
  if (q->n_channels > 32 * kWarpOutPerLane) return w;
  if (g_tune_threads || g_tune_stages || g_tune_ctas) return w;
  if (q->rows > 0x3fffffffLL) return w;
  const int D = q->cols, nseg = 8 / q->bits;
  const int segw = D / nseg;
  if (D % nseg || segw % 32) return w;
  const int ch = segw / 32;
  if ((ch != 32 && ch != 64 && ch != 128) || ch * nseg > 128) return w;
  if (q->rotate > segw || segw % q->rotate) return w;
  if (!tensor_map_encoder()) return w;
  w.ch = ch;
  uint32_t off = 64 * 8;                                   // two mbarriers per warp
  auto take = [&](uint32_t bytes, uint32_t align) { off = align_up(off, align); uint32_t o = off; off += bytes; return o; };
  w.off_chan = take((q->n_channels > 0 ? q->n_channels : 1) * 4, 16);
  w.off_wsm = norm ? take(D * 4, 128) : 0;
  w.slot_bytes = static_cast<uint32_t>(D) * 2u;
  w.off_slots = take(w.slot_bytes * kChunkBwdWarps * (norm ? 3 : 1), 1024);
  w.total = off + 1024;
  if (w.total > kSmemPerCtaMax) return w;
  long long grid = static_cast<long long>(sm_count()) * ((norm || q->bits == 8) ? 1 : 2);
  const long long need = (q->rows + kChunkBwdWarps - 1) / kChunkBwdWarps;
  if (grid > need) grid = need;
  w.grid = static_cast<int>(grid);
  w.ok = true;
  return w;
}

constexpr long long kChunkBwdLongRows = 8192;   // from here on the kernel compiled for the block of 256 is taken

template <int BITS, int CH>
int launch_bwd_chunk_one(const ChunkBwdArgs& a, const ChunkBwdPlan& w, int op, const CUtensorMap& dy_map,
                         const CUtensorMap& out_map, cudaStream_t stream) {
#define HYC_CB_LAUNCH(OP, GROUP)                                                                \
  {                                                                                             \
    if (!GROUP && a.p.rotate == 256 && a.p.rows >= kChunkBwdLongRows) {                         \
      auto kern = bwd_n_chunk_kernel<BITS, OP, CH, false, 256>;                                 \
      int rc = set_smem(kern, w.total);                                                         \
      if (rc) return rc;                                                                        \
      kern<<<w.grid, kChunkBwdWarps * 32, w.total, stream>>>(a, dy_map, out_map); HYC_LAUNCHED(); \
    } else {                                                                                    \
      auto kern = bwd_n_chunk_kernel<BITS, OP, CH, GROUP>;                                      \
      int rc = set_smem(kern, w.total);                                                         \
      if (rc) return rc;                                                                        \
      kern<<<w.grid, kChunkBwdWarps * 32, w.total, stream>>>(a, dy_map, out_map); HYC_LAUNCHED(); \
    }                                                                                           \
  }
#define HYC_CB_OP(OP) if (a.p.group) HYC_CB_LAUNCH(OP, true) else HYC_CB_LAUNCH(OP, false)
  if (op == kChunkNormBwdLn) { HYC_CB_OP(kChunkNormBwdLn) }
  else if (op == kChunkNormBwdRms) { HYC_CB_OP(kChunkNormBwdRms) }
  else { HYC_CB_OP(kChunkDecompress) }
#undef HYC_CB_OP
#undef HYC_CB_LAUNCH
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? HYC_OK : cuda_fail(e, "bwd_n_chunk_kernel launch");
}

int launch_bwd_chunk_b2(const ChunkBwdArgs& a, const ChunkBwdPlan& w, int op, const CUtensorMap& dy_map,
                        const CUtensorMap& out_map, cudaStream_t stream);
int launch_bwd_chunk_b4(const ChunkBwdArgs& a, const ChunkBwdPlan& w, int op, const CUtensorMap& dy_map,
                        const CUtensorMap& out_map, cudaStream_t stream);
int launch_bwd_chunk_b8(const ChunkBwdArgs& a, const ChunkBwdPlan& w, int op, const CUtensorMap& dy_map,
                        const CUtensorMap& out_map, cudaStream_t stream);

// One call for both entry points: `dy` NULL = decompress into `out` (row stride in elements), else norm backward.
inline int run_chunk_bwd(const hyc_packed* q, const ChunkBwdPlan& w, const void* dy, void* out, long long out_stride,
                         int kind, const void* weight, int param_bf16, const float* rstd, const float* mean, int ref_compat_c2,
                         cudaStream_t stream) {
  CUtensorMap dy_map, out_map;
  if (!row_tensor_map(&out_map, out, q->rows, q->cols, out_stride)) return HYC_ERR_SHAPE;
  dy_map = out_map;
  if (dy && !row_tensor_map(&dy_map, dy, q->rows, q->cols, q->cols)) return HYC_ERR_SHAPE;
  ChunkBwdArgs a;
  memset(&a, 0, sizeof(a));
  a.p = to_dev(q);
  a.kind = kind; a.weight = weight; a.param_bf16 = param_bf16; a.rstd = rstd; a.mean = mean; a.ref_compat_c2 = ref_compat_c2;
  a.off_chan = w.off_chan; a.off_wsm = w.off_wsm; a.off_slots = w.off_slots; a.slot_bytes = w.slot_bytes;
  a.wait_cycles = g_debug_wait_cycles > 0 ? g_debug_wait_cycles : kWaitCycles;
  a.tx_pad = g_debug_tx_pad;
  const int op = !dy ? kChunkDecompress : kind == HYC_NORM_LAYER ? kChunkNormBwdLn : kChunkNormBwdRms;
  return q->bits == 2 ? launch_bwd_chunk_b2(a, w, op, dy_map, out_map, stream)
       : q->bits == 4 ? launch_bwd_chunk_b4(a, w, op, dy_map, out_map, stream)
                      : launch_bwd_chunk_b8(a, w, op, dy_map, out_map, stream);
}

}  // namespace hyc
