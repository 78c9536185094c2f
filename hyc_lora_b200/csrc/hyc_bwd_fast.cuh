// Register-resident kernels that consume a packed activation of the
// channel-outlier mode: decompress to bf16, decompress + activation backward,
// decompress + norm backward.
//
// A CTA walks rows (row = blockIdx.x + i*gridDim.x).  The packed bytes of a row
// and the row of the upstream gradient are staged in shared memory by bulk
// asynchronous copies, two or three rows ahead; every thread rebuilds its own
// units of the row in registers and uses them at once.  One CTA barrier per
// row releases the staging slot and, at the same time, orders the streamed
// vector stores before the few scalar stores that rewrite the outlier
// channels: the streaming pass treats those channels as the zeros their codes
// encode, and after the barrier the threads that own the outlier list fix the
// outputs there from the stored bf16 originals (prefetched at the top of the
// iteration).  Rotation: in the unit mapping a warp holds 256 consecutive
// channels of every segment, so when the segment width is a multiple of the
// rotation block the butterflies run in registers on the freshly dequantised
// values (ROT == 2); otherwise (ROT == 1) the row is handed over through shared
// memory to a mapping of aligned 256-channel chunks.
//
// Reference mode (ROT == 3) uses the same kernels: the row is rebuilt with the reference's bf16
// rounding points, bf16(bf16(lowrank) + bf16((code - offset) * scale)), element outliers are
// streamed as the zero their code encodes and fixed after the row's barrier from the row's
// pool entries (column, bf16 value); the low-rank row travels in the staging slot.
#pragma once
#include "hyc_fwd_fast.cuh"

namespace hyc {

// (code - offset) * scale for the 8 elements of segment s of one unit (8 packed bytes).
// Integer -> float goes through the mantissa of 2^23 (one byte permute per element).
template <int BITS>
__device__ __forceinline__ void dequant8(const uint2& cb, int s, float sc, float (&f)[8]) {
  using C = CodeTraits<BITS>;
  uint32_t lo = cb.x, hi = cb.y;
  float bias;
  if (BITS == 8) {
    lo ^= 0x80808080u; hi ^= 0x80808080u;  // two's complement -> offset 128
    bias = 8388608.f + 128.f;
  } else {
    const uint32_t m = 0x01010101u * C::kMask;
    lo = (lo >> (s * BITS)) & m;
    hi = (hi >> (s * BITS)) & m;
    bias = 8388608.f + static_cast<float>(C::kOff);
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    // an explicit rounded multiply: the product must not be fused into a later addition (the rotation's
    // butterflies), or the sums would round differently from a sequential evaluation
    f[e] = __fmul_rn(__uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7650 + e)) - bias, sc);
    f[e + 4] = __fmul_rn(__uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7650 + e)) - bias, sc);
  }
}

// round 8 values to bf16 and back: one pack per pair, one shift/mask per element
__device__ __forceinline__ void round_bf16x8(float (&f)[8]) {
  const uint4 v = pack_bf16x8(f);
  unpack_bf16x8(v, f);
}

__device__ __forceinline__ uint2 ld_stream_u2(const void* p) {
  uint2 v;
  asm volatile("ld.global.cs.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

template <typename T>
__device__ __forceinline__ void ld_stream8(const T* p, float (&f)[8]);
template <>
__device__ __forceinline__ void ld_stream8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  unpack_bf16x8(v, f);
}
template <>
__device__ __forceinline__ void ld_stream8<float>(const float* p, float (&f)[8]) {
  load8<float>(p, 0, f);
}

struct BwdSmem {
  uint32_t off_red, off_misc, off_chan, off_chan2, off_rot, off_wsm, off_acc, off_slots, slot_bytes, total;
  uint32_t off_csc, off_csc2;   // reference mode: per-channel scales (bf16 [D]) of the operands
  uint32_t off_lr, off_lr2;     // reference mode: low-rank rows inside a staging slot
  int stages;
  uint32_t debug_tx_pad;        // test hook: bytes a row announces beyond what is copied (0 in normal use)
  long long wait_cycles;        // limit of the waits on staged rows
};

// Per-thread register groups: NR groups of 8 channels; col[r] < 0 marks an idle group.
// ROT: 0 no rotation, 1 rotation through shared memory (chunk mapping), 2 rotation in registers (unit mapping),
// 3 reference mode (unit mapping, no rotation)
template <int BITS, int UPT, int ROT>
struct Groups {
  static constexpr int NSEG = 8 / BITS;
  static constexpr int NR = ROT == 1 ? UPT : UPT * NSEG;
  int col[NR];
  uint32_t mask[2];  // 8 bits per register group: outlier channels inside the group
  // chan: this CTA's shared copy of the ascending outlier channel list
  __device__ __forceinline__ void init_masks(const int* chan, int k) {
    mask[0] = mask[1] = 0;
    for (int j = 0; j < k; ++j) {
      const int c = chan[j];
#pragma unroll
      for (int r = 0; r < NR; ++r)
        if (col[r] >= 0 && (c >> 3) == (col[r] >> 3)) mask[r >> 2] |= 1u << (((r & 3) << 3) + (c & 7));
    }
  }
  __device__ __forceinline__ uint32_t group_mask(int r) const { return (mask[r >> 2] >> ((r & 3) << 3)) & 0xffu; }
  __device__ __forceinline__ void init(int D) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int segw = D / NSEG, U = segw >> 3;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const int c = ROT == 1 ? (((warp + r * nwarps) << 8) + (lane << 3))
                             : ((r % NSEG) * segw + ((threadIdx.x + (r / NSEG) * blockDim.x) << 3));
      const bool ok = ROT == 1 ? (c < D) : ((threadIdx.x + (r / NSEG) * blockDim.x) < U);
      col[r] = ok ? c : -1;
    }
  }
};

// Rebuild this thread's slice of a row from its packed bytes `codes_row` (staged in shared
// memory).  Outlier channels come out as the zero their code encodes (ROT: see ZERO).
// ROUND: values are rounded to bf16 (what a reconstruction holds); without it the caller
// rounds when it packs its output.  ROT == 1: goes through w_rot (shared, fp32 [D]) and contains
// two CTA barriers.  ROT == 2: every warp executes the shuffles, idle groups carry zeros.
// what the reference-mode rebuild needs besides the packed bytes
struct RefCtx {
  const __nv_bfloat16* csc;   // per-channel scales in shared memory, or nullptr
  const __nv_bfloat16* lrs;   // low-rank row in the staging slot, or nullptr
  float sc_row;               // per-tensor / per-token scale
};

__device__ __forceinline__ RefCtx ref_ctx(const PackedDev& p, const __nv_bfloat16* csc, const unsigned char* slot,
                                          uint32_t off_lr, long long row) {
  RefCtx c;
  c.csc = p.scale_kind == kScaleChannel ? csc : nullptr;
  c.lrs = p.lowrank ? reinterpret_cast<const __nv_bfloat16*>(slot + off_lr) : nullptr;
  c.sc_row = p.scale_kind == kScaleTensor ? __bfloat162float(p.scale[0])
             : p.scale_kind == kScaleToken ? __bfloat162float(p.scale[row % p.seq]) : 1.f;
  return c;
}

// reconstruction of one element outlier (pool entry e) the way the reference adds it:
// bf16(lowrank + value); `lr_row` is the low-rank row in global memory or nullptr
__device__ __forceinline__ float ref_outlier_value(uint32_t e, const __nv_bfloat16* lr_row) {
  float val = bf16_bits_to_float(e >> 16);
  if (lr_row) val = bf16_round(__bfloat162float(lr_row[e & 0xffffu]) + val);
  return val;
}

template <int BITS, int UPT, int ROT, bool ROUND, bool ZERO = false>
__device__ __forceinline__ void rebuild_row(const PackedDev& p, const Groups<BITS, UPT, ROT>& g, float* w_rot,
                                            const unsigned char* codes_row, long long row,
                                            float (&f)[Groups<BITS, UPT, ROT>::NR][8], const RefCtx* rc = nullptr) {
  constexpr int NSEG = 8 / BITS;
  constexpr int NR = Groups<BITS, UPT, ROT>::NR;
  const int D = p.cols;
  if (ROT == 3) {
#pragma unroll
    for (int iu = 0; iu < UPT; ++iu) {
      if (g.col[iu * NSEG] >= 0) {
        const uint2 cb = *reinterpret_cast<const uint2*>(codes_row + g.col[iu * NSEG]);
#pragma unroll
        for (int s = 0; s < NSEG; ++s) {
          const int r = iu * NSEG + s, col = g.col[r];
          dequant8<BITS>(cb, s, 1.f, f[r]);          // code - offset
          float sc[8];
          if (rc->csc) {
            load8<__nv_bfloat16>(rc->csc, col, sc);
          } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) sc[e] = rc->sc_row;
          }
#pragma unroll
          for (int e = 0; e < 8; ++e) f[r][e] *= sc[e];
          round_bf16x8(f[r]);
          if (rc->lrs) {
            float l[8];
            load8<__nv_bfloat16>(rc->lrs, col, l);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[r][e] += l[e];
            round_bf16x8(f[r]);
          }
        }
      }
    }
    return;
  }
  const int G = p.group ? (D >> 7) : 1;
  const float* sc_row = p.scales + row * G;
  const float sc_tok = p.group ? 0.f : __ldg(sc_row);
  if (ROT != 1) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int iu = 0; iu < UPT; ++iu) {
      if (g.col[iu * NSEG] >= 0) {
        // unit u starts at byte 8u, which is also its first column
        const uint2 cb = *reinterpret_cast<const uint2*>(codes_row + g.col[iu * NSEG]);
#pragma unroll
        for (int s = 0; s < NSEG; ++s) {
          const float sc = p.group ? __ldg(sc_row + (g.col[iu * NSEG + s] >> 7)) : sc_tok;
          dequant8<BITS>(cb, s, sc, f[iu * NSEG + s]);
          if (ROUND && ROT == 0) round_bf16x8(f[iu * NSEG + s]);
        }
      } else if (ROT == 2) {
#pragma unroll
        for (int s = 0; s < NSEG; ++s)
#pragma unroll
          for (int e = 0; e < 8; ++e) f[iu * NSEG + s][e] = 0.f;
      }
      if (ROT == 2) {
#pragma unroll
        for (int s = 0; s < NSEG; ++s) {
          const int r = iu * NSEG + s;
          rotate_group(f[r], p.rotate, lane);
          if (ROUND) round_bf16x8(f[r]);
          if (ZERO) {
            const uint32_t m = g.group_mask(r);
            if (m) zero_masked(f[r], m);
          }
        }
      }
    }
  } else {
    const int segw = D / NSEG, U = segw >> 3;
    for (int u = threadIdx.x; u < U; u += blockDim.x) {
      const uint2 cb = *reinterpret_cast<const uint2*>(codes_row + (u << 3));
#pragma unroll
      for (int s = 0; s < NSEG; ++s) {
        const int col = s * segw + (u << 3);
        const float sc = p.group ? __ldg(sc_row + (col >> 7)) : sc_tok;
        float t[8];
        dequant8<BITS>(cb, s, sc, t);
        store8<float>(w_rot, col, t);
      }
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int n = p.rotate;
    const float rs = rotate_norm(n);
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      if (g.col[r] >= 0) load8<float>(w_rot, g.col[r], f[r]);
      else {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[r][e] = 0.f;
      }
      butterfly8(f[r]);
#pragma unroll
      for (int m2 = 1; m2 <= 16; m2 <<= 1) {
        if ((m2 << 3) < n) {
          const float sgn = (lane & m2) ? -1.f : 1.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) f[r][e] = __fmaf_rn(sgn, f[r][e], __shfl_xor_sync(0xffffffffu, f[r][e], m2));
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) f[r][e] *= rs;
      if (ROUND) round_bf16x8(f[r]);
      // after the inverse rotation an outlier channel holds quantisation noise, not the zero
      // its code encodes: callers that correct for "zero" ask for it to be cleared
      if (ZERO) {
        const uint32_t m = g.group_mask(r);
        if (m) zero_masked(f[r], m);
      }
    }
    __syncthreads();  // w_rot is rewritten for the next row
  }
}

// The staging ring of the consumers: `streams` byte ranges per row land in one slot.
struct RowFeed {
  RowRing ring;
  uint32_t bytes[5];
  uint32_t offset[5];
  const unsigned char* base[5];
  int period[5];   // 0: one source row per row; n: source row = row % n (low-rank rows repeat every sequence)
  int streams;
  uint32_t tx_pad;
  __device__ __forceinline__ void add(const void* src, uint32_t nbytes, uint32_t off, int per = 0) {
    base[streams] = static_cast<const unsigned char*>(src);
    bytes[streams] = nbytes; offset[streams] = off; period[streams] = per;
    ++streams;
  }
  __device__ __forceinline__ void issue(int stage, long long row) {
    uint32_t total = 0;
    for (int q = 0; q < streams; ++q) total += bytes[q];
    mbar_expect_tx(&ring.bars[stage], total + tx_pad);
    for (int q = 0; q < streams; ++q) {
      const long long src_row = period[q] ? row % period[q] : row;
      bulk_g2s(ring.slot(stage) + offset[q], base[q] + src_row * bytes[q], bytes[q], &ring.bars[stage]);
    }
  }
  __device__ __forceinline__ void prologue(long long first, long long rows, long long stride) {
    if (threadIdx.x == 0)
      for (int s = 0; s < ring.stages; ++s)
        if (first + s * stride < rows) issue(s, first + s * stride);
  }
  // after the row's barrier: hand the slot back to the copy engine
  __device__ __forceinline__ void refill(int stage, long long row, long long rows, long long stride) {
    if (threadIdx.x == 0) {
      const long long next = row + ring.stages * stride;
      if (next < rows) { fence_proxy_async(); issue(stage, next); }
    }
  }
};

// ------------------------------------------------------------------ common CTA prologue

struct FeedSetup {
  RowFeed feed;
  int* chan;
  int* chan2;
  float* w_rot;
  uint32_t* misc;
};

__device__ __forceinline__ FeedSetup feed_setup(unsigned char* smem, const BwdSmem& L) {
  FeedSetup s;
  s.feed.ring = RowRing{reinterpret_cast<uint64_t*>(smem), smem + L.off_slots, L.slot_bytes, L.stages};
  s.feed.ring.wait_cycles = L.wait_cycles;
  s.feed.ring.init();
  s.feed.streams = 0;
  s.feed.tx_pad = L.debug_tx_pad;
  s.chan = reinterpret_cast<int*>(smem + L.off_chan);
  s.chan2 = reinterpret_cast<int*>(smem + L.off_chan2);
  s.w_rot = reinterpret_cast<float*>(smem + L.off_rot);
  s.misc = reinterpret_cast<uint32_t*>(smem + L.off_misc);
  if (threadIdx.x == 0) s.misc[0] = 0;
  return s;
}

// bounded wait on slot `st` in barrier phase `ph`; an expired wait raises the CTA's sticky flag
__device__ __forceinline__ void feed_wait(FeedSetup& s, int st, uint32_t ph) {
  if (!mbar_wait_bounded(&s.feed.ring.bars[st], ph, s.feed.ring.wait_cycles)) s.misc[0] = 1;
}

// next ring position / barrier phase (counters instead of divisions by the run-time stage count)
__device__ __forceinline__ void feed_advance(const FeedSetup& s, int& st, uint32_t& ph) {
  if (++st == s.feed.ring.stages) { st = 0; ph ^= 1u; }
}

// after the row's barrier: true if the CTA must stop (some wait expired)
__device__ __forceinline__ bool feed_failed(FeedSetup& s, uint32_t* status, int i, long long row, long long rows,
                                            long long stride) {
  if (!s.misc[0]) return false;
  if (threadIdx.x == 0 && status) atomicOr(status, kStatusWaitExpired);
  drain_ring(s.feed.ring, i, row + stride, rows, stride);
  return true;
}

// ------------------------------------------------------------------ decompress

struct DecFastArgs {
  PackedDev p;
  __nv_bfloat16* out;
  long long row_stride, batch_stride, chunk_stride;
  int chunks;
  BwdSmem L;
};

template <int BITS, int UPT, int ROT>
__global__ void __launch_bounds__(512, 2) decompress_n_fast_kernel(const __grid_constant__ DecFastArgs a) {
  constexpr int NR = Groups<BITS, UPT, ROT>::NR;
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  const int D = p.cols, k = p.n_channels;
  FeedSetup fs = feed_setup(smem, a.L);
  fs.feed.add(p.codes, static_cast<uint32_t>(D) * BITS / 8, 0);
  if (ROT == 3 && p.lowrank) fs.feed.add(p.lowrank, static_cast<uint32_t>(D) * 2, a.L.off_lr, p.seq);
  // the first rows start travelling before the per-CTA tables are set up
  const long long rows = p.rows, stride = gridDim.x;
  long long row = blockIdx.x;
  fs.feed.prologue(row, rows, stride);
  __nv_bfloat16* csc = reinterpret_cast<__nv_bfloat16*>(smem + a.L.off_csc);
  if (ROT == 3) {
    if (p.scale_kind == kScaleChannel)
      for (int c = threadIdx.x; c < D; c += blockDim.x) csc[c] = p.scale[c];
  } else {
    for (int j = threadIdx.x; j < k; j += blockDim.x) fs.chan[j] = max(0, min(D - 1, p.channels[j]));
  }
  Groups<BITS, UPT, ROT> g;
  g.init(D);
  // output offset of every register group (head layouts cut the row into chunks)
  const int clen = D / a.chunks;
  long long ooff[NR];
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    const int c = g.col[r] >= 0 ? g.col[r] / clen : 0;
    ooff[r] = c * a.chunk_stride + (g.col[r] - c * clen);
  }
  __syncthreads();
  uint2 meta_pref = (ROT == 3 && row < rows) ? p.row_meta[row] : make_uint2(0u, 0u);
  int st = 0;
  uint32_t ph = 0;
  for (int i = 0; row < rows; ++i, row += stride, feed_advance(fs, st, ph)) {
    // the outlier values of this row, fetched early by the threads that will store them
    __nv_bfloat16 ov = __float2bfloat16_rn(0.f);
    // reference mode: this row's pool range was fetched one row ahead, so that the entry load
    // below does not wait for it
    const uint2 meta = meta_pref;
    uint32_t ent = 0;
    if (ROT == 3) {
      const long long nr = row + stride;
      meta_pref = nr < rows ? p.row_meta[nr] : make_uint2(0u, 0u);
      if (threadIdx.x < meta.y) ent = p.pool[meta.x + threadIdx.x];
    } else if (threadIdx.x < k) {
      ov = p.out_value[row * k + threadIdx.x];
    }
    feed_wait(fs, st, ph);
    float f[NR][8];
    RefCtx rc;
    if (ROT == 3) rc = ref_ctx(p, csc, fs.feed.ring.slot(st), a.L.off_lr, row);
    rebuild_row<BITS, UPT, ROT, false>(p, g, fs.w_rot, fs.feed.ring.slot(st), row, f, &rc);
    __nv_bfloat16* orow = a.chunks == 1 ? a.out + row * a.row_stride
                                        : a.out + (row / p.seq) * a.batch_stride + (row % p.seq) * a.row_stride;
#pragma unroll
    for (int r = 0; r < NR; ++r)
      if (g.col[r] >= 0) store8<__nv_bfloat16>(orow + ooff[r], 0, f[r]);
    __syncthreads();
    if (feed_failed(fs, p.status, i, row, rows, stride)) return;
    fs.feed.refill(st, row, rows, stride);
    if (ROT == 3) {
      const __nv_bfloat16* lr_row = p.lowrank ? p.lowrank + (row % p.seq) * static_cast<long long>(D) : nullptr;
      for (uint32_t j = threadIdx.x; j < meta.y; j += blockDim.x) {
        const uint32_t e = j == threadIdx.x ? ent : p.pool[meta.x + j];
        const int cc = static_cast<int>(e & 0xffffu);
        const int c = cc / clen;
        orow[c * a.chunk_stride + (cc - c * clen)] = __float2bfloat16_rn(ref_outlier_value(e, lr_row));
      }
    } else {
      for (int j = threadIdx.x; j < k; j += blockDim.x) {
        const int cc = fs.chan[j];
        const int c = cc / clen;
        orow[c * a.chunk_stride + (cc - c * clen)] = j == threadIdx.x ? ov : p.out_value[row * k + j];
      }
    }
  }
}

// ------------------------------------------------------------------ activation backward

struct ActFastArgs {
  PackedDev p1, p2;
  const unsigned char* g;
  unsigned char* dx1;
  unsigned char* dx2;
  BwdSmem L;
};

__device__ __forceinline__ float silu_grad_f(float x) {
  const float s = __fdividef(1.f, 1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

__device__ __forceinline__ float gelu_tanh_grad_f(float x) {
  const float gamma = 0.7978845608028654f, kappa = 0.044715f;
  const float y = gamma * (x + kappa * x * x * x);
  const float t = 1.f - __fdividef(2.f, 1.f + __expf(2.f * y));  // tanh(y)
  return 0.5f * ((1.f + t) + x * ((1.f - t * t) * gamma * (1.f + 3.f * kappa * x * x)));
}

template <int BITS, int UPT, int ROT, typename GT, int OP>
__global__ void __launch_bounds__(512, 2) act_bwd_n_fast_kernel(const __grid_constant__ ActFastArgs a) {
  constexpr int NR = Groups<BITS, UPT, ROT>::NR;
  constexpr bool PROD = OP == HYC_ACT_PRODUCT;
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p1;
  const int D = p.cols, k = p.n_channels;
  const int k2 = PROD ? a.p2.n_channels : 0;
  const uint32_t cb = static_cast<uint32_t>(D) * BITS / 8;
  const uint32_t off_c2 = (cb + 127u) & ~127u;
  const uint32_t off_g = PROD ? 2 * off_c2 : off_c2;
  FeedSetup fs = feed_setup(smem, a.L);
  fs.feed.add(p.codes, cb, 0);
  fs.feed.add(a.g, static_cast<uint32_t>(D) * sizeof(GT), off_g);
  if (PROD) fs.feed.add(a.p2.codes, cb, off_c2);
  if (ROT == 3 && p.lowrank) fs.feed.add(p.lowrank, static_cast<uint32_t>(D) * 2, a.L.off_lr, p.seq);
  if (ROT == 3 && PROD && a.p2.lowrank) fs.feed.add(a.p2.lowrank, static_cast<uint32_t>(D) * 2, a.L.off_lr2, a.p2.seq);
  // the first rows start travelling before the per-CTA tables are set up
  const long long rows = p.rows, stride = gridDim.x;
  long long row = blockIdx.x;
  fs.feed.prologue(row, rows, stride);
  __nv_bfloat16* csc = reinterpret_cast<__nv_bfloat16*>(smem + a.L.off_csc);
  __nv_bfloat16* csc2 = reinterpret_cast<__nv_bfloat16*>(smem + a.L.off_csc2);
  if (ROT == 3) {
    if (p.scale_kind == kScaleChannel)
      for (int c = threadIdx.x; c < D; c += blockDim.x) csc[c] = p.scale[c];
    if (PROD && a.p2.scale_kind == kScaleChannel)
      for (int c = threadIdx.x; c < D; c += blockDim.x) csc2[c] = a.p2.scale[c];
  } else {
    for (int j = threadIdx.x; j < k; j += blockDim.x) fs.chan[j] = max(0, min(D - 1, p.channels[j]));
    for (int j = threadIdx.x; j < k2; j += blockDim.x) fs.chan2[j] = max(0, min(D - 1, a.p2.channels[j]));
  }
  Groups<BITS, UPT, ROT> g;
  g.init(D);
  __syncthreads();
  uint2 meta_pref = (ROT == 3 && row < rows) ? p.row_meta[row] : make_uint2(0u, 0u);
  uint2 meta_pref2 = (ROT == 3 && PROD && row < rows) ? a.p2.row_meta[row] : make_uint2(0u, 0u);
  int st = 0;
  uint32_t ph = 0;
  for (int i = 0; row < rows; ++i, row += stride, feed_advance(fs, st, ph)) {
    float ov = 0.f, ov2 = 0.f;
    const uint2 meta = meta_pref, meta2 = meta_pref2;
    if (ROT == 3) {
      const long long nr = row + stride;
      meta_pref = nr < rows ? p.row_meta[nr] : make_uint2(0u, 0u);
      if (PROD) meta_pref2 = nr < rows ? a.p2.row_meta[nr] : make_uint2(0u, 0u);
    } else {
      if (threadIdx.x < k) ov = __bfloat162float(p.out_value[row * k + threadIdx.x]);
      if (PROD && threadIdx.x < k2) ov2 = __bfloat162float(a.p2.out_value[row * k2 + threadIdx.x]);
    }
    feed_wait(fs, st, ph);
    const unsigned char* slot = fs.feed.ring.slot(st);
    const GT* gs = reinterpret_cast<const GT*>(slot + off_g);
    GT* d1 = reinterpret_cast<GT*>(a.dx1) + row * D;
    GT* d2 = reinterpret_cast<GT*>(a.dx2) + row * D;
    float f[NR][8];
    RefCtx rc;
    if (ROT == 3) rc = ref_ctx(p, csc, slot, a.L.off_lr, row);
    rebuild_row<BITS, UPT, ROT, true>(p, g, fs.w_rot, slot, row, f, &rc);
    if (PROD) {
      // dx2 = x1 * g is finished before the second operand is rebuilt
#pragma unroll
      for (int r = 0; r < NR; ++r) {
        if (g.col[r] >= 0) {
          float gv[8], o[8];
          load8<GT>(gs, g.col[r], gv);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = f[r][e] * gv[e];
          store8<GT>(d2, g.col[r], o);
        }
      }
      if (ROT == 3) rc = ref_ctx(a.p2, csc2, slot, a.L.off_lr2, row);
      rebuild_row<BITS, UPT, ROT, true>(a.p2, g, fs.w_rot, slot + off_c2, row, f, &rc);
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      if (g.col[r] >= 0) {
        float gv[8], o[8];
        load8<GT>(gs, g.col[r], gv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          if (PROD) o[e] = gv[e] * f[r][e];
          else o[e] = (OP == HYC_ACT_SILU ? silu_grad_f(f[r][e]) : gelu_tanh_grad_f(f[r][e])) * gv[e];
        }
        store8<GT>(d1, g.col[r], o);
      }
    }
    // upstream gradient at the outlier channels, read before the slot is handed back
    float gq = 0.f, gq2 = 0.f;
    if (ROT != 3) {
      if (threadIdx.x < k) gq = static_cast<float>(gs[fs.chan[threadIdx.x]]);
      if (PROD && threadIdx.x < k2) gq2 = static_cast<float>(gs[fs.chan2[threadIdx.x]]);
    }
    __syncthreads();
    if (feed_failed(fs, p.status, i, row, rows, stride)) return;
    fs.feed.refill(st, row, rows, stride);
    const GT* grow = reinterpret_cast<const GT*>(a.g) + row * D;
    if (ROT == 3) {
      // element outliers of the row: the outputs that depend on the reconstruction are redone there
      const __nv_bfloat16* lr_row = p.lowrank ? p.lowrank + (row % p.seq) * static_cast<long long>(D) : nullptr;
      for (uint32_t j = threadIdx.x; j < meta.y; j += blockDim.x) {
        const uint32_t e = p.pool[meta.x + j];
        const int c = static_cast<int>(e & 0xffffu);
        const float o = ref_outlier_value(e, lr_row);
        const float gv = static_cast<float>(grow[c]);
        if (PROD) d2[c] = from_float<GT>(o * gv);
        else d1[c] = from_float<GT>((OP == HYC_ACT_SILU ? silu_grad_f(o) : gelu_tanh_grad_f(o)) * gv);
      }
      if (PROD) {
        const __nv_bfloat16* lr_row2 = a.p2.lowrank ? a.p2.lowrank + (row % a.p2.seq) * static_cast<long long>(D) : nullptr;
        for (uint32_t j = threadIdx.x; j < meta2.y; j += blockDim.x) {
          const uint32_t e = a.p2.pool[meta2.x + j];
          const int c = static_cast<int>(e & 0xffffu);
          d1[c] = from_float<GT>(static_cast<float>(grow[c]) * ref_outlier_value(e, lr_row2));
        }
      }
      continue;
    }
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
      const int c = fs.chan[j];
      const float o = j == threadIdx.x ? ov : __bfloat162float(p.out_value[row * k + j]);
      const float gv = j == threadIdx.x ? gq : static_cast<float>(grow[c]);
      if (PROD) d2[c] = from_float<GT>(o * gv);
      else d1[c] = from_float<GT>((OP == HYC_ACT_SILU ? silu_grad_f(o) : gelu_tanh_grad_f(o)) * gv);
    }
    if (PROD) {
      for (int j = threadIdx.x; j < k2; j += blockDim.x) {
        const int c = fs.chan2[j];
        const float o = j == threadIdx.x ? ov2 : __bfloat162float(a.p2.out_value[row * k2 + j]);
        const float gv = j == threadIdx.x ? gq2 : static_cast<float>(grow[c]);
        d1[c] = from_float<GT>(gv * o);
      }
    }
  }
}

// ------------------------------------------------------------------ norm backward

struct NormBwdFastArgs {
  PackedDev p;
  int kind, ref_compat_c2, param_bf16;
  const void* weight;
  const unsigned char* dy;
  const float* rstd;
  const float* mean;
  __nv_bfloat16* dx;
  float* partials;
  int need_dw, need_db;
  BwdSmem L;
};

template <int BITS, int UPT, int ROT, typename GT>
__global__ void __launch_bounds__(256, 3) norm_bwd_n_fast_kernel(const __grid_constant__ NormBwdFastArgs a) {
  constexpr int NR = Groups<BITS, UPT, ROT>::NR;
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  const int D = p.cols, k = p.n_channels;
  const uint32_t cb = static_cast<uint32_t>(D) * BITS / 8;
  const uint32_t off_g = (cb + 127u) & ~127u;
  FeedSetup fs = feed_setup(smem, a.L);
  fs.feed.add(p.codes, cb, 0);
  fs.feed.add(a.dy, static_cast<uint32_t>(D) * sizeof(GT), off_g);
  if (ROT == 3 && p.lowrank) fs.feed.add(p.lowrank, static_cast<uint32_t>(D) * 2, a.L.off_lr, p.seq);
  // the first rows start travelling before the per-CTA tables are set up
  const long long rows = p.rows, stride = gridDim.x;
  long long row = blockIdx.x;
  fs.feed.prologue(row, rows, stride);
  __nv_bfloat16* csc = reinterpret_cast<__nv_bfloat16*>(smem + a.L.off_csc);
  if (ROT == 3 && p.scale_kind == kScaleChannel)
    for (int c = threadIdx.x; c < D; c += blockDim.x) csc[c] = p.scale[c];
  float* wsm = reinterpret_cast<float*>(smem + a.L.off_wsm);
  float* red = reinterpret_cast<float*>(smem + a.L.off_red);
  float* acc_w = reinterpret_cast<float*>(smem + a.L.off_acc);
  float* acc_b = acc_w + D;
  const bool ln = a.kind == HYC_NORM_LAYER;
  const float plus = a.kind == HYC_NORM_RMS_GEMMA ? 1.f : 0.f;
  if (ROT != 3)
    for (int j = threadIdx.x; j < k; j += blockDim.x) fs.chan[j] = max(0, min(D - 1, p.channels[j]));
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    wsm[split_index(c, D)] = (a.param_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.weight)[c])
                           : static_cast<const float*>(a.weight)[c]) + plus;
    if (a.need_dw) { acc_w[c] = 0.f; if (a.need_db) acc_b[c] = 0.f; }
  }
  Groups<BITS, UPT, ROT> g;
  g.init(D);
  __syncthreads();
  if (ROT == 1 || ROT == 2) g.init_masks(fs.chan, k);
  const float inv_d = 1.0f / static_cast<float>(D);
  uint2 meta_pref = (ROT == 3 && row < rows) ? p.row_meta[row] : make_uint2(0u, 0u);
  int st = 0;
  uint32_t ph = 0;
  for (int i = 0; row < rows; ++i, row += stride, feed_advance(fs, st, ph)) {
    __nv_bfloat16* dxrow = a.dx + row * D;
    const float rstd = __ldg(a.rstd + row);
    const float mean = ln ? __ldg(a.mean + row) : 0.f;
    float ov = 0.f;
    // reference mode: this row's pool range was fetched one row ahead, so that the entry load
    // below does not wait for it
    const uint2 meta = meta_pref;
    uint32_t ent = 0;
    if (ROT == 3) {
      const long long nr = row + stride;
      meta_pref = nr < rows ? p.row_meta[nr] : make_uint2(0u, 0u);
      if (threadIdx.x < meta.y) ent = p.pool[meta.x + threadIdx.x];
    } else if (threadIdx.x < k) {
      ov = __bfloat162float(p.out_value[row * k + threadIdx.x]);
    }
    feed_wait(fs, st, ph);
    const unsigned char* slot = fs.feed.ring.slot(st);
    const GT* gs = reinterpret_cast<const GT*>(slot + off_g);
    float f[NR][8];
    RefCtx rc;
    if (ROT == 3) rc = ref_ctx(p, csc, slot, a.L.off_lr, row);
    rebuild_row<BITS, UPT, ROT, true, true>(p, g, fs.w_rot, slot, row, f, &rc);
    // f becomes x-hat, wd = w * dy
    float c1 = 0.f, c2 = 0.f;
    float wd[NR][8];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      if (g.col[r] >= 0) {
        float gv[8], wv[8];
        load8<GT>(gs, g.col[r], gv);
        load8_split(wsm, D, g.col[r], wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float gy = sizeof(GT) == 4 ? bf16_round(gv[e]) : gv[e];
          f[r][e] = (f[r][e] - mean) * rstd;   // x-hat (outlier channels: from the zero their code encodes)
          wd[r][e] = wv[e] * gy;
          c1 = fmaf(f[r][e], wd[r][e], c1);
          c2 += wd[r][e];
        }
      }
    }
    // outlier channels: the true x-hat differs from the streamed one by o * rstd
    float gq = 0.f;
    if (ROT == 3) {
      // element outliers: the streamed x-hat used the low-rank value alone (their code is the zero code)
      for (uint32_t j = threadIdx.x; j < meta.y; j += blockDim.x) {
        const uint32_t e = j == threadIdx.x ? ent : p.pool[meta.x + j];
        const int c = static_cast<int>(e & 0xffffu);
        const float was = rc.lrs ? __bfloat162float(rc.lrs[c]) : 0.f;
        const float o = ref_outlier_value(e, rc.lrs) - was;
        float gy = static_cast<float>(gs[c]);
        if (sizeof(GT) == 4) gy = bf16_round(gy);
        c1 = fmaf(o * rstd, wsm[split_index(c, D)] * gy, c1);
      }
    } else {
      for (int j = threadIdx.x; j < k; j += blockDim.x) {
        const int c = fs.chan[j];
        const float o = j == threadIdx.x ? ov : __bfloat162float(p.out_value[row * k + j]);
        float gy = static_cast<float>(gs[c]);
        if (sizeof(GT) == 4) gy = bf16_round(gy);
        if (j == threadIdx.x) gq = gy;
        c1 = fmaf(o * rstd, wsm[split_index(c, D)] * gy, c1);
      }
    }
    {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        c1 += __shfl_xor_sync(0xffffffffu, c1, o);
        c2 += __shfl_xor_sync(0xffffffffu, c2, o);
      }
      float* buf = red + (i & 1) * 64;
      const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
      if ((threadIdx.x & 31) == 0) { buf[warp] = c1; buf[32 + warp] = c2; }
      __syncthreads();
      const int l = threadIdx.x & 7;
      c1 = l < nwarps ? buf[l] : 0.f;
      c2 = l < nwarps ? buf[32 + l] : 0.f;
#pragma unroll
      for (int o = 4; o > 0; o >>= 1) {
        c1 += __shfl_xor_sync(0xffffffffu, c1, o);
        c2 += __shfl_xor_sync(0xffffffffu, c2, o);
      }
    }
    if (feed_failed(fs, p.status, i, row, rows, stride)) break;
    c1 *= inv_d;
    c2 = (ln || a.ref_compat_c2) ? c2 * inv_d : 0.f;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      if (g.col[r] >= 0) {
        float d[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) d[e] = (wd[r][e] - (f[r][e] * c1 + c2)) * rstd;
        store8<__nv_bfloat16>(dxrow, g.col[r], d);
        if (a.need_dw) {
          // weight / bias gradient partials: this thread owns these columns; the update sits after
          // the row's reduction barrier so that it never overlaps the outlier correction below
          float gv[8];
          load8<GT>(gs, g.col[r], gv);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float gy = sizeof(GT) == 4 ? bf16_round(gv[e]) : gv[e];
            acc_w[g.col[r] + e] += gy * f[r][e];
            if (a.need_db) acc_b[g.col[r] + e] += gy;
          }
        }
      }
    }
    // second barrier: orders the vector stores before the outlier fix and frees the slot
    __syncthreads();
    fs.feed.refill(st, row, rows, stride);
    const GT* grow = reinterpret_cast<const GT*>(a.dy) + row * D;
    if (ROT == 3) {
      const __nv_bfloat16* lr_row = p.lowrank ? p.lowrank + (row % p.seq) * static_cast<long long>(D) : nullptr;
      for (uint32_t j = threadIdx.x; j < meta.y; j += blockDim.x) {
        const uint32_t e = j == threadIdx.x ? ent : p.pool[meta.x + j];
        const int c = static_cast<int>(e & 0xffffu);
        const float o = ref_outlier_value(e, lr_row);
        const float was = lr_row ? __bfloat162float(lr_row[c]) : 0.f;
        float gy = static_cast<float>(grow[c]);
        if (sizeof(GT) == 4) gy = bf16_round(gy);
        const float xh = (o - mean) * rstd;
        dxrow[c] = __float2bfloat16_rn((wsm[split_index(c, D)] * gy - (xh * c1 + c2)) * rstd);
        if (a.need_dw) acc_w[c] += gy * ((o - was) * rstd);
      }
      continue;
    }
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
      const int c = fs.chan[j];
      const float o = j == threadIdx.x ? ov : __bfloat162float(p.out_value[row * k + j]);
      float gy = j == threadIdx.x ? gq : static_cast<float>(grow[c]);
      if (sizeof(GT) == 4 && j != threadIdx.x) gy = bf16_round(gy);
      const float xh = (o - mean) * rstd;
      dxrow[c] = __float2bfloat16_rn((wsm[split_index(c, D)] * gy - (xh * c1 + c2)) * rstd);
      if (a.need_dw) acc_w[c] += gy * (o * rstd);  // the streamed pass added gy * (0 - mean) * rstd
    }
  }
  if (a.need_dw) {
    __syncthreads();
    float* pw = a.partials + static_cast<long long>(blockIdx.x) * D;
    float* pb = a.partials + (static_cast<long long>(gridDim.x) + blockIdx.x) * D;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
      pw[c] = acc_w[c];
      if (a.need_db) pb[c] = acc_b[c];
    }
  }
}

// ------------------------------------------------------------------ host planning

struct BwdPlan {
  bool ok;
  int threads, upt, grid;
  int rot;   // 0 none, 1 through shared memory, 2 in registers
  BwdSmem L;
};

// reg_groups: cap on 8-channel register groups per thread for the kernel at hand;
// slot_bytes: bytes one staged row needs (codes, gradient row, ...)
inline BwdPlan plan_bwd_fast(const hyc_packed* q, const hyc_packed* q2, int reg_groups, bool want_w, int acc_rows,
                             int max_threads, int grid_cap, uint32_t slot_bytes, int min_threads = 0,
                             int default_stages = 3) {
  BwdPlan b;
  memset(&b, 0, sizeof(b));
  const bool ref = q->mode == HYC_MODE_R;
  if (ref ? (q->bits != 2 && q->bits != 4 && q->bits != 8) : q->rotate > 256) return b;
  if (q2 && q2->mode != q->mode) return b;
  const int D = q->cols, nseg = 8 / q->bits;
  // rotation in registers needs every segment to start on a rotation-block boundary
  b.rot = ref ? 3 : q->rotate == 0 ? 0 : ((D / nseg) % q->rotate == 0 ? 2 : 1);
  int threads = g_tune_threads ? g_tune_threads : (D <= 1024 ? 64 : D <= 4096 ? 128 : 256);
  // kernels that hold two operands per element in registers run better with fewer elements per thread
  if (!g_tune_threads && min_threads && threads < min_threads && D >= 8 * min_threads) threads = min_threads;
  if (b.rot == 1) {
    const int chunks = (D + 255) / 256;
    for (; threads <= max_threads; threads *= 2) {
      const int cpt = (chunks + threads / 32 - 1) / (threads / 32);
      if (cpt <= reg_groups) { b.ok = true; b.threads = threads; b.upt = cpt; break; }
    }
  } else {
    const int U = D / nseg / 8;
    // a thread owns whole units: more threads than units would idle
    while (threads > 32 && threads / 2 >= U) threads /= 2;
    for (; threads <= max_threads; threads *= 2) {
      const int upt = (U + threads - 1) / threads;
      if (upt * nseg <= reg_groups) { b.ok = true; b.threads = threads; b.upt = upt; break; }
    }
  }
  if (!b.ok) return b;
  int u = 1;
  while (u < b.upt) u *= 2;
  b.upt = u;
  // units per thread round up to an instantiated count: give the spare slots back as threads (whole warps),
  // e.g. 688 units at 4 per thread run on 192 threads instead of 256
  if (b.rot != 1 && !g_tune_threads) {
    const int U = D / nseg / 8;
    const int fit = ((U + b.upt - 1) / b.upt + 31) / 32 * 32;
    if (fit < b.threads) b.threads = fit;
  }
  uint32_t off = 64;  // mbarriers
  auto take = [&](uint32_t bytes) { uint32_t o = off; off = align_up(off + bytes, 16); return o; };
  b.L.off_red = take(2 * 64 * 4);
  b.L.off_misc = take(16);
  b.L.off_chan = take((!ref && q->n_channels > 0 ? q->n_channels : 1) * 4);
  b.L.off_chan2 = take(((!ref && q2 && q2->n_channels > 0) ? q2->n_channels : 1) * 4);
  if (ref && q->scale_kind == HYC_SCALE_CHANNEL) b.L.off_csc = take(D * 2);
  if (ref && q2 && q2->scale_kind == HYC_SCALE_CHANNEL) b.L.off_csc2 = take(D * 2);
  if (ref) {
    // low-rank rows ride at the end of a staging slot
    slot_bytes = align_up(slot_bytes, 128);
    if (q->lowrank) { b.L.off_lr = slot_bytes; slot_bytes += align_up(static_cast<uint32_t>(D) * 2, 128); }
    if (q2 && q2->lowrank) { b.L.off_lr2 = slot_bytes; slot_bytes += align_up(static_cast<uint32_t>(D) * 2, 128); }
  }
  if (b.rot == 1) b.L.off_rot = take(D * 4);
  if (want_w) b.L.off_wsm = take(D * 4);
  if (acc_rows) b.L.off_acc = take(static_cast<uint32_t>(acc_rows) * D * 4);
  off = align_up(off, 128);
  b.L.off_slots = off;
  b.L.slot_bytes = align_up(slot_bytes, 128);
  b.L.stages = g_tune_stages ? g_tune_stages : default_stages;
  if (b.L.stages > kMaxStages) b.L.stages = kMaxStages;
  while (b.L.stages > 2 && off + b.L.slot_bytes * b.L.stages > 64 * 1024) --b.L.stages;
  b.L.total = off + b.L.slot_bytes * b.L.stages;
  b.L.debug_tx_pad = g_debug_tx_pad;
  b.L.wait_cycles = g_debug_wait_cycles > 0 ? g_debug_wait_cycles : kWaitCycles;
  if (b.L.total > kSmemPerCtaMax) { b.ok = false; return b; }
  int ctas = g_tune_ctas ? g_tune_ctas : 2048 / b.threads;
  while (ctas > 1 && (static_cast<uint32_t>(ctas) * (b.L.total + 1024) > kSmemBudget || ctas * b.threads > 2048)) --ctas;
  long long grid = static_cast<long long>(sm_count()) * ctas;
  if (grid_cap && grid > grid_cap) grid = grid_cap;
  if (grid > q->rows) grid = q->rows;
  b.grid = static_cast<int>(grid);
  return b;
}

// dispatch helpers: BITS in {2,4,8}, UPT in {1,2,4,8}, ROT; combinations beyond the register cap are not instantiated
#define HYC_BWD_DISPATCH(PLAN, BITS_V, CAP, LAUNCH)                                            \
  {                                                                                            \
    const int bits__ = (BITS_V);                                                               \
    bool done__ = false;                                                                       \
    HYC_BWD_ONE(PLAN, bits__, 2, CAP, LAUNCH) HYC_BWD_ONE(PLAN, bits__, 4, CAP, LAUNCH)        \
    HYC_BWD_ONE(PLAN, bits__, 8, CAP, LAUNCH)                                                  \
    if (!done__) return HYC_ERR_SMEM;                                                          \
  }
#define HYC_BWD_ONE(PLAN, bits__, B, CAP, LAUNCH)                                              \
  if (bits__ == B) {                                                                           \
    HYC_BWD_UPT(PLAN, B, 1, CAP, LAUNCH) HYC_BWD_UPT(PLAN, B, 2, CAP, LAUNCH)                  \
    HYC_BWD_UPT(PLAN, B, 4, CAP, LAUNCH) HYC_BWD_UPT(PLAN, B, 8, CAP, LAUNCH)                  \
  }
#define HYC_BWD_UPT(PLAN, B, UP, CAP, LAUNCH)                                                  \
  if ((PLAN).upt == UP) {                                                                      \
    if ((PLAN).rot == 1) {                                                                     \
      if constexpr (UP <= CAP) { LAUNCH(B, UP, 1) done__ = true; }                             \
    } else if ((PLAN).rot == 2) {                                                              \
      if constexpr (UP * (8 / B) <= CAP) { LAUNCH(B, UP, 2) done__ = true; }                   \
    } else if ((PLAN).rot == 3) {                                                              \
      if constexpr (UP * (8 / B) <= CAP) { LAUNCH(B, UP, 3) done__ = true; }                   \
    } else {                                                                                   \
      if constexpr (UP * (8 / B) <= CAP) { LAUNCH(B, UP, 0) done__ = true; }                   \
    }                                                                                          \
  }

}  // namespace hyc
