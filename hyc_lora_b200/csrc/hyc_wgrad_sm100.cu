// LoRA-A weight gradient straight from packed codes on the 5th-generation tensor cores:
//
//     dA[n, d] = sum_t G[t, n] * X_hat[t, d]        (n < rank, d < D, t < T)
//
// X_hat is never written to HBM.  A CTA owns 128 packed byte columns of the code rows (that is
// 8/bits tiles of 128 channels, one per row segment) and a slice of the tokens.  For every
// chunk of 64 tokens all threads turn the packed fields into exact bf16 integers (code minus
// offset: one byte permute drops a field pair into the mantissas of 128.0, one packed subtract
// removes 128 + offset) and store them, 16 bytes per token and 8 channels, into shared memory
// in the MN-major no-swizzle core-matrix layout tcgen05 reads; the scale of the token (or of
// the token and the 128-channel tile) is folded into the gradient rows, which are rounded to
// bf16 and stored in the same layout:  sum_t G[t,n] * (q[t,d] * s[t])  =  sum_t (G[t,n] s[t]) * q[t,d].
// (8-bit codes are dequantised on the A side instead.)  One thread then issues
// tcgen05.mma (M = 128 channels, N = rank, K = 16 tokens per instruction) with the
// accumulators in tensor memory, and commits to an mbarrier that tells everybody when the
// staging buffer may be overwritten (two buffers; the packed bytes of chunk c+1 are already in
// registers while chunk c is converted).  At the end four warps read the accumulators back
// with tcgen05.ld and store one partial [rank, D] slab per token slice; wgrad_finish_kernel adds
// the slabs, rotates the rows back and drops in the outlier channels' columns.  Those columns,
// grad^T * out_value, come from extra CTAs of the same launch whose A operand is the stored
// bf16 outlier values (128 outlier channels per CTA) instead of converted codes.
//
// Channel-outlier mode: outlier channels carry the zero code, so their columns come out as zero
// in the code tiles and are filled from the side CTAs.  With rotation the kernel contracts the
// un-rotated codes and the rotation is applied to the `rank` output rows afterwards
// (X_hat = Q H  =>  G^T X_hat = (G^T Q) H).
//
// Reference mode (static scale, element outliers; 2/4/8-bit codes).  The same tensor-core kernel
// contracts the integer codes: a per-token or per-tensor scale is first written out as one fp32
// scale per row (r_row_scale_kernel) and folded into the gradient rows exactly like the dynamic
// per-token scale of the channel mode; a per-channel scale multiplies the columns of the summed
// result in wgrad_finish_kernel.  The element outliers (their code is the zero code) are a sparse
// side term, out[n, col] += G[t, n] * value over the pool entries of every row:
// wgrad_pool_kernel accumulates it in shared memory, one CTA per (token slice, group of ranks),
// and adds it into that slice's partial slab before the finish kernel runs.  A low-rank part is
// left to the caller: it adds (sum over the batch of G)^T * lowrank, one small dense product.
#include <stdlib.h>

#include <mutex>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/hyc_b200.h"
#include "hyc_bwd_fast.cuh"

namespace hyc {

constexpr int kChunk = 64;          // tokens per staging buffer
constexpr int kTileM = 128;         // channels per accumulator tile
constexpr int kWgThreads = 512;

// ---- tcgen05 wrappers ------------------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], bf16 x bf16 -> fp32, issued by one thread.  The two shared-memory
// descriptors arrive as (low, high) words.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// the mbarrier gets one arrival when every MMA issued so far by this thread has finished
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void st_shared_u4(uint32_t saddr, uint4 v) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Shared-memory matrix descriptor, no swizzle.  Core matrix = 8 rows of 16 bytes; `lbo` is the
// byte distance between core matrices along K, `sbo` along M/N (MN-major operands).  Low word:
// address >> 4 (14 bits) and lbo >> 4 at bit 16; high word: sbo >> 4 and the version bit (bit 46).
__device__ __forceinline__ uint32_t desc_lo(uint32_t saddr, uint32_t lbo) {
  return ((saddr & 0x3FFFFu) >> 4) | ((lbo >> 4) << 16);
}
__device__ __forceinline__ constexpr uint32_t desc_hi(uint32_t sbo) { return (sbo >> 4) | (1u << 14); }

// instruction descriptor: fp32 accumulate, bf16 A and B, both MN-major, M = 128, N = n
__host__ __device__ constexpr uint32_t instr_desc(int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(kTileM >> 4) << 24);
}

struct WgradArgs {
  PackedDev p;
  const __nv_bfloat16* grad;  // [T, rank]
  int rank, npad;             // npad: rank rounded up to 16
  long long tokens_per_split;
  float* partials;            // [splits][rank][D]
  uint32_t tmem_cols;
  // outlier channels: CTAs with blockIdx.x >= tiles contract the stored bf16 values of 128 outlier
  // channels each instead of dequantised codes
  int tiles;                  // code tiles (blockIdx.x < tiles)
  int side_split;             // side CTAs per outlier tile and token slice (each takes a part of the slice)
  int k;                      // outlier channels
  const __nv_bfloat16* out_value;   // [T, k]
  float* side;                // [splits][k][rank]
};

// A staging: [token group of 8][unit of 8 channels (16)][8 tokens][8 channels] bf16
constexpr uint32_t kASbo = 128, kALbo = 16 * 128, kAStage = (kChunk / 8) * kALbo;  // 16 KiB per segment
// B staging: [token group][npad/8][8 tokens][8 ranks]
constexpr uint32_t kBSbo = 128;

template <int BITS>
__global__ void __launch_bounds__(kWgThreads, 2) lora_wgrad_kernel(const __grid_constant__ WgradArgs a) {
  constexpr int NSEG = 8 / BITS;
  extern __shared__ __align__(1024) unsigned char smem[];
  const PackedDev& p = a.p;
  const int D = p.cols;
  const int segw = D / NSEG;
  const int cb = D * BITS / 8;
  const int G = p.group ? (D >> 7) : 1;
  const int npad = a.npad;
  const uint32_t b_lbo = static_cast<uint32_t>(npad / 8) * 128u;
  const uint32_t b_stage = (kChunk / 8) * b_lbo;
  // shared-memory map
  uint64_t* bar_done = reinterpret_cast<uint64_t*>(smem);          // [2] MMAs of a buffer finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 16);
  uint32_t* fail = reinterpret_cast<uint32_t*>(smem + 20);
  unsigned char* a_buf = smem + 1024;                              // [2][NSEG][kAStage]
  unsigned char* b_buf = a_buf + 2u * NSEG * kAStage;              // [2][B tiles][b_stage]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(&bar_done[0], 1);
    mbar_init(&bar_done[1], 1);
    fence_barrier_init();
    *fail = 0;
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, a.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool is_side = static_cast<int>(blockIdx.x) >= a.tiles;
  const int side_x = is_side ? static_cast<int>(blockIdx.x) - a.tiles : 0;
  const int side_sub = side_x % a.side_split;            // which part of the token slice a side CTA takes
  const int side_j0 = (side_x / a.side_split) * kTileM;  // first outlier of a side CTA
  const int byte0 = is_side ? 0 : blockIdx.x * kTileM;   // first packed byte column of this CTA
  long long t_begin = static_cast<long long>(blockIdx.y) * a.tokens_per_split;
  long long t_end = min(p.rows, t_begin + a.tokens_per_split);
  if (is_side && a.side_split > 1) {
    const long long sub_len = ((a.tokens_per_split + a.side_split - 1) / a.side_split + kChunk - 1) / kChunk * kChunk;
    t_begin += side_sub * sub_len;
    t_end = min(t_end, t_begin + sub_len);
  }
  const int nchunks = t_end > t_begin ? static_cast<int>((t_end - t_begin + kChunk - 1) / kChunk) : 0;
  const uint32_t idesc = instr_desc(npad);
  // conversion mapping: lane = token-in-group (k0) + 8 * (unit & 3); a warp item = (token group, unit >> 2)
  const int k0 = lane & 7, u_lo = lane >> 3;
  constexpr int kAItems = (kChunk / 8) * 4 / (kWgThreads / 32);   // A items per warp and chunk
  const int b_per_tg = (npad / 8 + 3) / 4;                         // 1 or 2 B items per token group
  // B tiles per buffer: the scale is folded into the gradient operand, so group scales (one per
  // 128-channel tile, i.e. per segment) need one scaled copy of the gradient rows per segment
  const int nb = (BITS < 8 && p.group && !is_side) ? NSEG : 1;
  const int nseg_eff = is_side ? 1 : NSEG;               // a side CTA holds one tile of outlier channels
  // Per-thread source pointers and shared-memory offsets are set up once and advanced by a
  // constant per chunk.  Tokens past the end of the slice contribute nothing because their
  // gradient rows are stored as zeros; the code rows only have to be readable, so their
  // pointer is clamped to the last row of the tensor instead of being predicated.
  const unsigned char* a_src[kAItems];
  const unsigned char* a_last[kAItems];
  const float* a_sc[kAItems];             // 8-bit path: scale of the A item
  uint32_t a_dst[kAItems];
#pragma unroll
  for (int i = 0; i < kAItems; ++i) {
    const int item = warp + i * (kWgThreads / 32);
    const int tg = item >> 2, unit = ((item & 3) << 2) + u_lo;
    const long long t = t_begin + tg * 8 + k0;
    const int colb = byte0 + (unit << 3);
    a_src[i] = p.codes + t * cb + colb;
    a_last[i] = p.codes + (p.rows - 1) * cb + colb;
    a_sc[i] = p.scales + t * G + (p.group ? (colb >> 7) : 0);
    a_dst[i] = tg * kALbo + unit * kASbo + k0 * 16;
  }
  // B item of this thread (one per warp and chunk at most)
  const int b_tg = b_per_tg == 2 ? (warp >> 1) : warp;
  const int b_n1 = (b_per_tg == 2 ? (warp & 1) : 0) * 4 + u_lo;
  const bool b_own = warp < (kChunk / 8) * b_per_tg && b_n1 < npad / 8;
  const bool b_real = b_own && (b_n1 << 3) < a.rank;               // ranks past `rank` stay zero
  long long b_t = t_begin + b_tg * 8 + k0;
  const __nv_bfloat16* b_src = a.grad + b_t * a.rank + (b_n1 << 3);
  const float* b_sc = p.scales + b_t * G + (p.group ? (byte0 >> 7) : 0);
  const int b_sc_seg = p.group ? (segw >> 7) : 0;                  // scale index step between segments
  const uint32_t b_dst = b_tg * b_lbo + b_n1 * kBSbo + k0 * 16;
  const long long a_step = static_cast<long long>(kChunk) * cb;
  const float* const sc_last = p.scales + (p.rows - 1) * G;       // last row of scales (clamp for reads)

  uint2 cb_reg[kAItems];
  float sc_reg[kAItems];          // 8-bit path only
  uint4 g_reg;
  float gs_reg[NSEG];
  auto fetch = [&]() {
#pragma unroll
    for (int i = 0; i < kAItems; ++i) {
      const unsigned char* src = a_src[i] < a_last[i] ? a_src[i] : a_last[i];
      cb_reg[i] = is_side ? make_uint2(0u, 0u) : ld_stream_u2(src);
      if (BITS == 8 && !is_side) {
        const float* sp = a_sc[i] < sc_last + G ? a_sc[i] : sc_last;
        sc_reg[i] = __ldg(sp);
        a_sc[i] += kChunk * G;
      }
      a_src[i] += a_step;
    }
    g_reg = make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int s = 0; s < NSEG; ++s) gs_reg[s] = 0.f;
    if (b_real && b_t < t_end) {
      g_reg = *reinterpret_cast<const uint4*>(b_src);
      if (BITS < 8) {
#pragma unroll
        for (int s = 0; s < NSEG; ++s)
          if (s < nb) gs_reg[s] = is_side ? 1.f : __ldg(b_sc + s * b_sc_seg);
      }
    }
    b_t += kChunk;
    b_src += kChunk * a.rank;
    b_sc += kChunk * G;
  };
  if (nchunks > 0) fetch();
  const uint32_t a_smem = smem_u32(a_buf), b_smem = smem_u32(b_buf);
  const uint32_t b_k_step = (2u * b_lbo) >> 4, b_s_step = nb > 1 ? (b_stage >> 4) : 0u;   // descriptor address steps
  for (int c = 0; c < nchunks; ++c) {
    const int buf = c & 1;
    // move this chunk's registers aside and start the next chunk's loads
    uint2 cb_cur[kAItems];
    float sc_cur[kAItems];
    float gs_cur[NSEG];
#pragma unroll
    for (int i = 0; i < kAItems; ++i) { cb_cur[i] = cb_reg[i]; sc_cur[i] = sc_reg[i]; }
    const uint4 g_cur = g_reg;
#pragma unroll
    for (int s = 0; s < NSEG; ++s) gs_cur[s] = gs_reg[s];
    if (c + 1 < nchunks) fetch();
    if (c >= 2) {
      if (!mbar_wait_bounded(&bar_done[buf], ((c >> 1) - 1) & 1)) *fail = 1;
      tc_fence_after();
    }
    const uint32_t abase = a_smem + static_cast<uint32_t>(buf) * NSEG * kAStage;
    const uint32_t bbase = b_smem + static_cast<uint32_t>(buf) * nb * b_stage;
    // ---- A operand.  Below 8 bits: the integer code minus its offset as an exact bf16 (a field is
    // dropped into the mantissa of 128.0 with one byte permute per pair, then 128 + offset is
    // subtracted in packed bf16 arithmetic).  8 bits: dequantised values.
    if (is_side) {
      // outlier values are bf16 already: eight scalar loads per (token, unit) -- the rows of
      // out_value are k elements long, not 16-byte aligned -- packed into one 16-byte store
#pragma unroll
      for (int i = 0; i < kAItems; ++i) {
        const int item = warp + i * (kWgThreads / 32);
        const int tg = item >> 2, unit = ((item & 3) << 2) + u_lo;
        const int j0 = side_j0 + (unit << 3);
        long long t = t_begin + static_cast<long long>(c) * kChunk + tg * 8 + k0;
        if (t > p.rows - 1) t = p.rows - 1;           // readable; such tokens meet zero gradient rows
        const unsigned short* src = reinterpret_cast<const unsigned short*>(a.out_value) + t * a.k + j0;
        uint32_t h[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) h[e] = (j0 + e < a.k) ? static_cast<uint32_t>(__ldg(src + e)) : 0u;
        st_shared_u4(abase + a_dst[i], make_uint4(h[0] | (h[1] << 16), h[2] | (h[3] << 16), h[4] | (h[5] << 16),
                                                  h[6] | (h[7] << 16)));
      }
    } else {
#pragma unroll
    for (int i = 0; i < kAItems; ++i) {
#pragma unroll
      for (int s = 0; s < NSEG; ++s) {
        uint4 v;
        if (BITS == 8) {
          float f[8];
          dequant8<BITS>(cb_cur[i], s, sc_cur[i], f);
          v = pack_bf16x8(f);
        } else {
          constexpr uint32_t m = 0x01010101u * CodeTraits<BITS>::kMask;
          const uint32_t lo = (cb_cur[i].x >> (s * BITS)) & m, hi = (cb_cur[i].y >> (s * BITS)) & m;
          const __nv_bfloat162 bias = __float2bfloat162_rn(128.f + static_cast<float>(CodeTraits<BITS>::kOff));
          auto two = [&](uint32_t w, uint32_t sel) {
            const uint32_t bits = __byte_perm(w, 0x43004300u, sel);      // (128 + field) as bf16x2
            __nv_bfloat162 r = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&bits), bias);
            return *reinterpret_cast<uint32_t*>(&r);
          };
          v = make_uint4(two(lo, 0x7150), two(lo, 0x7352), two(hi, 0x7150), two(hi, 0x7352));
        }
        st_shared_u4(abase + s * kAStage + a_dst[i], v);
      }
    }
    }
    // ---- B operand: gradient rows, times the token (or token-and-tile) scale below 8 bits
    if (b_own) {
      if (BITS == 8) {
        st_shared_u4(bbase + b_dst, g_cur);
      } else {
        float gv[8];
        unpack_bf16x8(g_cur, gv);
#pragma unroll
        for (int s = 0; s < NSEG; ++s) {
          if (s < nb) {
            float sv[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) sv[e] = gv[e] * gs_cur[s];
            st_shared_u4(bbase + s * b_stage + b_dst, pack_bf16x8(sv));
          }
        }
      }
    }
    fence_proxy_async();          // generic-proxy stores -> visible to the tensor-core (async) proxy
    tc_fence_before();
    __syncthreads();
    if (*fail) break;
    if (tid == 0) {
      tc_fence_after();
      // Only the address field (low word) of a descriptor changes between instructions: one
      // add per operand and instruction keeps this single-thread section short -- every other
      // warp meets it again at the next barrier.
      const uint32_t a_lo = desc_lo(abase, kALbo), b_lo = desc_lo(bbase, b_lbo);
      const uint32_t acc0 = c > 0 ? 1u : 0u;
#pragma unroll
      for (int s = 0; s < NSEG; ++s) {
        if (s >= nseg_eff) break;
#pragma unroll
        for (int ks = 0; ks < kChunk / 16; ++ks) {
          umma_bf16(tmem_base + static_cast<uint32_t>(s) * static_cast<uint32_t>(npad),
                    a_lo + ((s * kAStage + ks * 2 * kALbo) >> 4), desc_hi(kASbo),
                    b_lo + static_cast<uint32_t>(s) * b_s_step + static_cast<uint32_t>(ks) * b_k_step, desc_hi(kBSbo),
                    idesc, ks > 0 ? 1u : acc0);
        }
      }
      umma_commit(&bar_done[buf]);
    }
  }
  // ---- wait for the last MMAs, then read the accumulators back
  if (nchunks > 0 && !*fail) {
    const int last = nchunks - 1;
    if (!mbar_wait_bounded(&bar_done[last & 1], (last >> 1) & 1)) *fail = 1;
    if (nchunks > 1) {
      const int prev = nchunks - 2;
      if (!mbar_wait_bounded(&bar_done[prev & 1], (prev >> 1) & 1)) *fail = 1;
    }
  }
  tc_fence_after();
  __syncthreads();
  const bool failed = *fail != 0;
  if (failed && tid == 0 && p.status) atomicOr(p.status, kStatusWaitExpired);
  if (warp < 4 && is_side) {
    // accumulator row = outlier channel; partial [slice][outlier][rank]
    const int j = side_j0 + warp * 32 + lane;
    float* dst = a.side + ((static_cast<long long>(blockIdx.y) * a.side_split + side_sub) * a.k + j) * a.rank;
    for (int n0 = 0; n0 < npad; n0 += 16) {
      uint32_t v[16];
      if (nchunks > 0 && !failed) {
        tmem_ld16(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + static_cast<uint32_t>(n0), v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int q = 0; q < 16; ++q) v[q] = 0u;
      }
      if (j < a.k) {
#pragma unroll
        for (int q = 0; q < 16; ++q)
          if (n0 + q < a.rank) dst[n0 + q] = __uint_as_float(v[q]);
      }
    }
  } else if (warp < 4) {
    float* slab = a.partials + static_cast<long long>(blockIdx.y) * a.rank * D;
#pragma unroll
    for (int s = 0; s < NSEG; ++s) {
      const int d = s * segw + byte0 + warp * 32 + lane;      // channel of this thread's accumulator row
      for (int n0 = 0; n0 < npad; n0 += 16) {
        uint32_t v[16];
        if (nchunks > 0 && !failed) {
          tmem_ld16(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + static_cast<uint32_t>(s * npad + n0), v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int q = 0; q < 16; ++q) v[q] = 0u;
        }
#pragma unroll
        for (int q = 0; q < 16; ++q)
          if (n0 + q < a.rank) slab[static_cast<long long>(n0 + q) * D + d] = __uint_as_float(v[q]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, a.tmem_cols);
}


// ------------------------------------------------------------------------------------------
// Warp-specialised variant for launches in which every CTA is a code tile (reference-mode records and
// channel-mode records without outlier channels; 2- and 4-bit codes; 4096 rows or more).  Measured on
// [65536, 4096] INT4, rank 64: 0.105-0.114 ms against 0.128 ms for the kernel above.  Both kernels are bound by
// shared-memory bandwidth, not by the tensor pipe: every element of the A operand is written to shared memory
// once as bf16 and read from it once by the tensor core (4 bytes of shared-memory traffic per element, about
// 30 us of the 128 bytes per clock and SM for this shape), on top of which come the code tile and the B tiles.
//
// Roles inside one CTA per SM (320 threads):
//   warp 8, one thread    brings the packed code tiles -- 64 tokens x 128 bytes -- into a four-deep ring of
//                         shared-memory tiles with 2-D tensor copies (cp.async.bulk.tensor, 128-byte swizzle,
//                         completion on an mbarrier, no multicast);
//   warps 0-7             turn a code tile into the bf16 A tiles (one per segment) and the scaled gradient
//                         rows into the B tile(s) of a three-deep operand ring, and hand the stage to
//   warp 9, one thread    which issues the tcgen05.mma instructions of the stage and lets tcgen05.commit
//                         release it;
//   warps 0-3             read the accumulators back from tensor memory at the end.
// Every hand-over is an mbarrier (no CTA barrier per chunk), so the copies of chunk c+3, the conversion of
// chunk c+1 and the tensor-core work of chunk c overlap.  The swizzled tile makes both sides of the
// conversion free of bank conflicts: lanes read along tokens (8 tokens x 2 sixteen-byte pieces per
// wavefront) and write the core matrices along tokens too.  Every wait is bounded; a role that gives up
// raises the CTA's flag, the others see it, copies in flight are waited for (bounded) and tensor memory is
// freed before the CTA ends.
constexpr int kWsConvWarps = 8;
constexpr int kWsThreads = (kWsConvWarps + 2) * 32;
constexpr int kWsCodeStages = 4;
constexpr uint32_t kWsCodeTile = kChunk * kTileM;   // 8 KiB
constexpr long long kWsMinRows = 4096;

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 2-D tiled copy global -> this CTA's shared memory (x: byte column, a multiple of 16; y: row)
__device__ __forceinline__ void tma_load_2d(uint32_t dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          dst_smem),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// operand stages: three, or two where four segments of A tiles would not fit three times
__host__ __device__ constexpr int ws_ab_stages(int bits) { return bits == 2 ? 2 : 3; }

template <int BITS>
__global__ void __launch_bounds__(kWsThreads, 1) lora_wgrad_ws_kernel(const __grid_constant__ WgradArgs a,
                                                                      const __grid_constant__ CUtensorMap tmap) {
  constexpr int NSEG = 8 / BITS;
  constexpr int kWsAbStages = ws_ab_stages(BITS);
  extern __shared__ __align__(1024) unsigned char smem[];
  const PackedDev& p = a.p;
  const int D = p.cols;
  const int segw = D / NSEG;
  const int G = p.group ? (D >> 7) : 1;
  const int npad = a.npad;
  const uint32_t b_lbo = static_cast<uint32_t>(npad / 8) * 128u;
  const uint32_t b_stage = (kChunk / 8) * b_lbo;
  const int nb = (BITS < 8 && p.group) ? NSEG : 1;
  // shared-memory map
  uint64_t* code_full = reinterpret_cast<uint64_t*>(smem);          // [4] a code tile has landed
  uint64_t* code_empty = code_full + kWsCodeStages;                 // [4] the converters are done with it
  uint64_t* ab_full = code_empty + kWsCodeStages;                   // [stages] operand stage written
  uint64_t* ab_empty = ab_full + kWsAbStages;                       // [stages] its MMAs have finished
  uint64_t* acc_done = ab_empty + kWsAbStages;                      // every MMA of the CTA has finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 128);
  volatile uint32_t* fail = reinterpret_cast<volatile uint32_t*>(smem + 132);
  unsigned char* code_ring = smem + 1024;                           // [4][8 KiB], 1024-byte aligned (swizzle atom)
  unsigned char* a_buf = code_ring + kWsCodeStages * kWsCodeTile;   // [3][NSEG][kAStage]
  unsigned char* b_buf = a_buf + static_cast<size_t>(kWsAbStages) * NSEG * kAStage;   // [3][nb][b_stage]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    for (int i = 0; i < kWsCodeStages; ++i) { mbar_init(&code_full[i], 1); mbar_init(&code_empty[i], kWsConvWarps); }
    for (int i = 0; i < kWsAbStages; ++i) { mbar_init(&ab_full[i], kWsConvWarps); mbar_init(&ab_empty[i], 1); }
    mbar_init(acc_done, 1);
    fence_barrier_init();
    *fail = 0;
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, a.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int byte0 = blockIdx.x * kTileM;   // first packed byte column of this CTA
  const long long t_begin = static_cast<long long>(blockIdx.y) * a.tokens_per_split;
  const long long t_end = min(p.rows, t_begin + a.tokens_per_split);
  const int nchunks = t_end > t_begin ? static_cast<int>((t_end - t_begin + kChunk - 1) / kChunk) : 0;
  const uint32_t a_smem = smem_u32(a_buf), b_smem = smem_u32(b_buf);

  if (warp == kWsConvWarps) {
    // ---------------------------------------------------------------- copy role
    if (lane == 0) {
      int issued = 0;
      for (int c = 0; c < nchunks; ++c) {
        const int st = c % kWsCodeStages;
        if (c >= kWsCodeStages) {
          if (!mbar_wait_bounded(&code_empty[st], ((c / kWsCodeStages) - 1) & 1)) *fail = 1;
        }
        if (*fail) break;
        mbar_expect_tx(&code_full[st], kWsCodeTile);
        tma_load_2d(smem_u32(code_ring + st * kWsCodeTile), &tmap, byte0, static_cast<int>(t_begin + static_cast<long long>(c) * kChunk),
                    &code_full[st]);
        issued = c + 1;
      }
      if (*fail) {
        // copies still in flight must land before the CTA's shared memory goes away
        for (int c = max(0, issued - kWsCodeStages); c < issued; ++c)
          (void)mbar_wait_bounded(&code_full[c % kWsCodeStages], (c / kWsCodeStages) & 1);
      }
    }
  } else if (warp == kWsConvWarps + 1) {
    // ---------------------------------------------------------------- tensor-core role
    if (lane == 0) {
      const uint32_t idesc = instr_desc(npad);
      const uint32_t b_k_step = (2u * b_lbo) >> 4, b_s_step = nb > 1 ? (b_stage >> 4) : 0u;
      for (int c = 0; c < nchunks; ++c) {
        const int st = c % kWsAbStages;
        if (!mbar_wait_bounded(&ab_full[st], (c / kWsAbStages) & 1)) *fail = 1;
        if (*fail) break;
        tc_fence_after();
        const uint32_t abase = a_smem + static_cast<uint32_t>(st) * NSEG * kAStage;
        const uint32_t bbase = b_smem + static_cast<uint32_t>(st) * nb * b_stage;
        const uint32_t a_lo = desc_lo(abase, kALbo), b_lo = desc_lo(bbase, b_lbo);
        const uint32_t acc0 = c > 0 ? 1u : 0u;
#pragma unroll
        for (int s = 0; s < NSEG; ++s) {
#pragma unroll
          for (int ks = 0; ks < kChunk / 16; ++ks) {
            umma_bf16(tmem_base + static_cast<uint32_t>(s) * static_cast<uint32_t>(npad),
                      a_lo + ((s * kAStage + ks * 2 * kALbo) >> 4), desc_hi(kASbo),
                      b_lo + static_cast<uint32_t>(s) * b_s_step + static_cast<uint32_t>(ks) * b_k_step, desc_hi(kBSbo),
                      idesc, ks > 0 ? 1u : acc0);
          }
        }
        umma_commit(&ab_empty[st]);
      }
      // one more commit covers everything issued; on the give-up path it is also what this thread waits
      // for (bounded) before tensor memory may be freed
      umma_commit(acc_done);
      if (*fail) (void)mbar_wait_bounded(acc_done, 0);
    }
  } else {
    // ---------------------------------------------------------------- conversion role (warps 0-7)
    const int k0 = lane & 7, u_lo = lane >> 3;
    constexpr int kAItems = (kChunk / 8) * 4 / kWsConvWarps;   // 4 per warp and chunk
    const int b_per_tg = (npad / 8 + 3) / 4;                     // 1 or 2 B items per token group
    uint32_t a_src[kAItems], a_dst[kAItems];
#pragma unroll
    for (int i = 0; i < kAItems; ++i) {
      const int item = warp + i * kWsConvWarps;
      const int tg = item >> 2, unit = ((item & 3) << 2) + u_lo;
      const int tl = tg * 8 + k0;                                 // token inside the chunk
      // swizzled tile: sixteen-byte piece c of row t sits at piece c ^ (t & 7)
      a_src[i] = static_cast<uint32_t>(tl) * kTileM + ((((unit >> 1) ^ (tl & 7))) << 4) + ((unit & 1) << 3);
      a_dst[i] = tg * kALbo + unit * kASbo + k0 * 16;
    }
    // B items of this thread: j = warp, warp + 8
    int b_tg[2], b_n1[2];
    bool b_own[2], b_real[2];
    uint32_t b_dst[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int j = warp + i * kWsConvWarps;
      b_tg[i] = b_per_tg == 2 ? (j >> 1) : j;
      b_n1[i] = (b_per_tg == 2 ? (j & 1) : 0) * 4 + u_lo;
      b_own[i] = j < (kChunk / 8) * b_per_tg && b_n1[i] < npad / 8;
      b_real[i] = b_own[i] && (b_n1[i] << 3) < a.rank;
      b_dst[i] = b_tg[i] * b_lbo + b_n1[i] * kBSbo + k0 * 16;
    }
    const int b_sc_seg = p.group ? (segw >> 7) : 0;
    // gradient rows and scales come straight from global memory, two chunks ahead of their use (a chunk is
    // shorter than a global load's latency)
    uint4 g_reg[2], g_nxt[2];
    float gs_reg[2][NSEG], gs_nxt[2][NSEG];
    float a_sc_reg[kAItems], a_sc_nxt[kAItems];   // 8-bit path: scale of the token of every A item
    auto fetch = [&](int c, uint4 (&g_reg)[2], float (&gs_reg)[2][NSEG], float (&a_sc_reg)[kAItems]) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        g_reg[i] = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int s = 0; s < NSEG; ++s) gs_reg[i][s] = 0.f;
        const long long t = t_begin + static_cast<long long>(c) * kChunk + b_tg[i] * 8 + k0;
        if (b_real[i] && t < t_end) {
          g_reg[i] = *reinterpret_cast<const uint4*>(a.grad + t * a.rank + (b_n1[i] << 3));
          if (BITS < 8) {
            const float* sc = p.scales + t * G + (p.group ? (byte0 >> 7) : 0);
#pragma unroll
            for (int s = 0; s < NSEG; ++s)
              if (s < nb) gs_reg[i][s] = __ldg(sc + s * b_sc_seg);
          }
        }
      }
      if (BITS == 8) {
#pragma unroll
        for (int i = 0; i < kAItems; ++i) {
          const int item = warp + i * kWsConvWarps;
          long long t = t_begin + static_cast<long long>(c) * kChunk + (item >> 2) * 8 + k0;
          if (t > p.rows - 1) t = p.rows - 1;
          a_sc_reg[i] = __ldg(p.scales + t * G + (p.group ? ((byte0 + ((((item & 3) << 2) + u_lo) << 3)) >> 7) : 0));
        }
      }
    };
    if (nchunks > 0) fetch(0, g_reg, gs_reg, a_sc_reg);
    if (nchunks > 1) fetch(1, g_nxt, gs_nxt, a_sc_nxt);
    for (int c = 0; c < nchunks; ++c) {
      const int cst = c % kWsCodeStages, ast = c % kWsAbStages;
      uint4 g_cur[2];
      float gs_cur[2][NSEG], a_sc_cur[kAItems];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        g_cur[i] = g_reg[i];
        g_reg[i] = g_nxt[i];
#pragma unroll
        for (int s = 0; s < NSEG; ++s) { gs_cur[i][s] = gs_reg[i][s]; gs_reg[i][s] = gs_nxt[i][s]; }
      }
#pragma unroll
      for (int i = 0; i < kAItems; ++i) { a_sc_cur[i] = a_sc_reg[i]; a_sc_reg[i] = a_sc_nxt[i]; }
      if (c + 2 < nchunks) fetch(c + 2, g_nxt, gs_nxt, a_sc_nxt);
      if (!mbar_wait_bounded(&code_full[cst], (c / kWsCodeStages) & 1)) *fail = 1;
      if (c >= kWsAbStages) {
        if (!mbar_wait_bounded(&ab_empty[ast], ((c / kWsAbStages) - 1) & 1)) *fail = 1;
        tc_fence_after();
      }
      if (*fail) break;
      const unsigned char* tile = code_ring + cst * kWsCodeTile;
      const uint32_t abase = a_smem + static_cast<uint32_t>(ast) * NSEG * kAStage;
      const uint32_t bbase = b_smem + static_cast<uint32_t>(ast) * nb * b_stage;
#pragma unroll
      for (int i = 0; i < kAItems; ++i) {
        const uint2 cw = *reinterpret_cast<const uint2*>(tile + a_src[i]);
#pragma unroll
        for (int s = 0; s < NSEG; ++s) {
          uint4 v;
          if (BITS == 8) {
            float f[8];
            dequant8<BITS>(cw, s, a_sc_cur[i], f);
            v = pack_bf16x8(f);
          } else {
            constexpr uint32_t m = 0x01010101u * CodeTraits<BITS>::kMask;
            const uint32_t lo = (cw.x >> (s * BITS)) & m, hi = (cw.y >> (s * BITS)) & m;
            const __nv_bfloat162 bias = __float2bfloat162_rn(128.f + static_cast<float>(CodeTraits<BITS>::kOff));
            auto two = [&](uint32_t w, uint32_t sel) {
              const uint32_t bits = __byte_perm(w, 0x43004300u, sel);      // (128 + field) as bf16x2
              __nv_bfloat162 r = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&bits), bias);
              return *reinterpret_cast<uint32_t*>(&r);
            };
            v = make_uint4(two(lo, 0x7150), two(lo, 0x7352), two(hi, 0x7150), two(hi, 0x7352));
          }
          st_shared_u4(abase + s * kAStage + a_dst[i], v);
        }
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        if (b_own[i]) {
          if (BITS == 8) {
            st_shared_u4(bbase + b_dst[i], g_cur[i]);
          } else {
            float gv[8];
            unpack_bf16x8(g_cur[i], gv);
#pragma unroll
            for (int s = 0; s < NSEG; ++s) {
              if (s < nb) {
                float sv[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) sv[e] = gv[e] * gs_cur[i][s];
                st_shared_u4(bbase + s * b_stage + b_dst[i], pack_bf16x8(sv));
              }
            }
          }
        }
      }
      fence_proxy_async();          // generic-proxy stores -> visible to the tensor-core (async) proxy
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&code_empty[cst]);
        mbar_arrive(&ab_full[ast]);
      }
    }
    // ---------------------------------------------------------------- read the accumulators back (warps 0-3)
    if (warp < 4) {
      if (nchunks > 0 && !*fail) {
        if (!mbar_wait_bounded(acc_done, 0)) *fail = 1;
      }
      tc_fence_after();
      const bool failed = *fail != 0;
      float* slab = a.partials + static_cast<long long>(blockIdx.y) * a.rank * D;
#pragma unroll
      for (int s = 0; s < NSEG; ++s) {
        const int d = s * segw + byte0 + warp * 32 + lane;      // channel of this thread's accumulator row
        for (int n0 = 0; n0 < npad; n0 += 16) {
          uint32_t v[16];
          if (nchunks > 0 && !failed) {
            tmem_ld16(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + static_cast<uint32_t>(s * npad + n0), v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int q = 0; q < 16; ++q) v[q] = 0u;
          }
#pragma unroll
          for (int q = 0; q < 16; ++q)
            if (n0 + q < a.rank) slab[static_cast<long long>(n0 + q) * D + d] = __uint_as_float(v[q]);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *fail && p.status) atomicOr(p.status, kStatusWaitExpired);
  if (warp == 0) tmem_dealloc(tmem_base, a.tmem_cols);
}

// Last kernel of the call, one CTA per (output row n, part of the row): adds the partial slabs in a
// fixed order, applies the inverse block rotation to the summed row in shared memory (the rotation
// commutes with the contraction over tokens), overwrites the outlier channels' entries with the sums
// of the side partials, and writes the row.
__global__ void wgrad_finish_kernel(const float* __restrict__ partials, int splits, const float* __restrict__ side,
                                    int slices, const int* __restrict__ channels, int k, int rank, int D, int rotate,
                                    const __nv_bfloat16* __restrict__ colscale, float* __restrict__ out,
                                    __nv_bfloat16* __restrict__ out_bf16, int accumulate) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* rowbuf = reinterpret_cast<float*>(smem_raw);
  const int n = blockIdx.x;
  const int len = D / gridDim.y, d0 = blockIdx.y * len;
  const long long slab = static_cast<long long>(rank) * D;
  const float* src = partials + static_cast<long long>(n) * D + d0;
  for (int c = threadIdx.x << 2; c < len; c += blockDim.x << 2) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int q = 0; q < splits; ++q) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(src + q * slab + c));
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    if (colscale) {   // reference mode, per-channel scale: the codes were contracted as integers
      acc.x *= __bfloat162float(colscale[d0 + c]);
      acc.y *= __bfloat162float(colscale[d0 + c + 1]);
      acc.z *= __bfloat162float(colscale[d0 + c + 2]);
      acc.w *= __bfloat162float(colscale[d0 + c + 3]);
    }
    *reinterpret_cast<float4*>(rowbuf + c) = acc;
  }
  __syncthreads();
  if (rotate) fwht_row<float, false>(rowbuf, nullptr, rowbuf, len, rotate);
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    const int ch = channels[j] - d0;
    if (ch >= 0 && ch < len) {
      float sum = 0.f;
      for (int q = 0; q < slices; ++q) sum += side[(static_cast<long long>(q) * k + j) * rank + n];
      rowbuf[ch] = sum;
    }
  }
  __syncthreads();
  // `accumulate`: the result is added to what `out` holds (the sum in fp32, rounded once) -- a gradient buffer that
  // collects several backward passes
  if (out_bf16) {   // the caller's parameter dtype: rounded here instead of by a kernel of its own
    __nv_bfloat16* dst = out_bf16 + static_cast<long long>(n) * D + d0;
    for (int c = threadIdx.x << 2; c < len; c += blockDim.x << 2) {
      float4 v = *reinterpret_cast<const float4*>(rowbuf + c);
      if (accumulate) {
        const uint2 old = *reinterpret_cast<const uint2*>(dst + c);
        v.x += __uint_as_float(old.x << 16); v.y += __uint_as_float(old.x & 0xffff0000u);
        v.z += __uint_as_float(old.y << 16); v.w += __uint_as_float(old.y & 0xffff0000u);
      }
      *reinterpret_cast<uint2*>(dst + c) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
    }
    return;
  }
  float* dst = out + static_cast<long long>(n) * D + d0;
  for (int c = threadIdx.x << 2; c < len; c += blockDim.x << 2) {
    float4 v = *reinterpret_cast<const float4*>(rowbuf + c);
    if (accumulate) {
      const float4 old = *reinterpret_cast<const float4*>(dst + c);
      v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
    }
    *reinterpret_cast<float4*>(dst + c) = v;
  }
}

// Reference mode: the scale of every row as fp32 (per-token scale: by sequence position; per-tensor: the one
// scale; per-channel: 1, the columns are scaled at the end).
__global__ void r_row_scale_kernel(const __nv_bfloat16* __restrict__ scale, int kind, int seq, long long rows,
                                   float* __restrict__ row_scale) {
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (t >= rows) return;
  row_scale[t] = kind == kScaleToken ? __bfloat162float(scale[t % seq])
                 : kind == kScaleTensor ? __bfloat162float(scale[0]) : 1.f;
}

// Reference mode: element outliers as a sparse side term.  CTA (x = group of `rpw` ranks, y = token slice)
// walks the rows of its slice, one warp per row: lane = (entry e of 32/rpw taken at once, rank r of the
// group); every entry (column, value) of the row adds G[t, n0 + r] * value (divided by the column's scale
// when the result will be multiplied by it) to acc[column][r] in shared memory.  At the end the CTA adds its
// accumulator into its own part of the slice's partial slab (one owner per part: no atomics in global
// memory, the result stays reproducible up to the order of the shared-memory additions).
__global__ void __launch_bounds__(512) wgrad_pool_kernel(const uint32_t* __restrict__ pool, const uint2* __restrict__ row_meta,
                                                         const __nv_bfloat16* __restrict__ grad, int rank, int rpw, int D,
                                                         long long rows, long long tokens_per_split,
                                                         const __nv_bfloat16* __restrict__ colscale,
                                                         float* __restrict__ partials) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* acc = reinterpret_cast<float*>(smem_raw);          // [D][rpw]
  const int n0 = blockIdx.x * rpw;
  const long long t0 = static_cast<long long>(blockIdx.y) * tokens_per_split;
  const long long t1 = min(rows, t0 + tokens_per_split);
  for (int i = threadIdx.x; i < D * rpw; i += blockDim.x) acc[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int per = 32 / rpw;                                  // entries taken at once
  const int e = lane / rpw, r = lane % rpw;
  for (long long t = t0 + warp; t < t1; t += nwarps) {
    const uint2 meta = __ldg(row_meta + t);
    if (meta.y == 0) continue;
    const float g = (n0 + r) < rank ? __bfloat162float(grad[t * rank + n0 + r]) : 0.f;
    for (uint32_t i = e; i < meta.y; i += per) {
      const uint32_t ent = __ldg(pool + meta.x + i);
      const int col = static_cast<int>(ent & 0xffffu);
      float v = bf16_bits_to_float(ent >> 16);
      if (colscale) v = __fdividef(v, __bfloat162float(colscale[col]));
      atomicAdd(&acc[col * rpw + r], g * v);
    }
  }
  __syncthreads();
  float* slab = partials + static_cast<long long>(blockIdx.y) * rank * D;
  for (int i = threadIdx.x; i < D * rpw; i += blockDim.x) {
    const int rr = i / D, d = i - rr * D;
    if (n0 + rr < rank) slab[static_cast<long long>(n0 + rr) * D + d] += acc[d * rpw + rr];
  }
}

struct WgradPlan {
  int splits;          // token slices of the tensor-core kernel
  int side_slices;     // token slices holding outlier-channel partials (0: no outlier channels)
  int side_tiles;      // extra CTAs per token slice: tiles of 128 outlier channels x side_split
  int side_split;
  uint32_t smem_bytes, tmem_cols;
  int npad;
  long long scratch_floats;
  long long row_scale_at;   // reference mode: offset (floats) of the per-row scales in the scratch
  int rpw;                  // reference mode: ranks per CTA of the pool kernel
  bool ws;                  // code tiles on the warp-specialised kernel (one CTA per SM)
  uint32_t ws_smem;
};

// cuTensorMapEncodeTiled through the runtime (no link-time dependency on the driver library)
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// the packed codes as a 2-D byte tensor [rows][row bytes], tiles of 64 rows x 128 bytes, 128-byte swizzle
static bool code_tensor_map(const hyc_packed* saved, CUtensorMap* map) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t cb = static_cast<cuuint64_t>(saved->cols) * saved->bits / 8;
  const cuuint64_t dims[2] = {cb, static_cast<cuuint64_t>(saved->rows)};
  const cuuint64_t strides[1] = {cb};
  const cuuint32_t box[2] = {kTileM, kChunk};
  const cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, saved->codes, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Resident CTAs per SM from the kernel's own resource use (registers, shared memory, threads).
template <int BITS>
static int wgrad_ctas_per_sm(uint32_t smem_bytes, int dev) {
  auto kern = lora_wgrad_kernel<BITS>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes) != cudaSuccess) return 0;
  cudaFuncAttributes fa;
  if (cudaFuncGetAttributes(&fa, kern) != cudaSuccess) return 0;
  int smem_sm = 0, regs_sm = 0, thr_sm = 0, reserved = 0;
  if (cudaDeviceGetAttribute(&smem_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&regs_sm, cudaDevAttrMaxRegistersPerMultiprocessor, dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&thr_sm, cudaDevAttrMaxThreadsPerMultiProcessor, dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev) != cudaSuccess)
    return 0;
  const long long per_cta_smem = static_cast<long long>(smem_bytes) + fa.sharedSizeBytes + reserved;
  const int regs_cta = ((fa.numRegs + 7) / 8 * 8) * kWgThreads;
  int n = static_cast<int>(smem_sm / per_cta_smem);
  if (regs_cta > 0 && regs_sm / regs_cta < n) n = regs_sm / regs_cta;
  if (thr_sm / kWgThreads < n) n = thr_sm / kWgThreads;
  return n;
}

// One wave of CTAs: tiles * splits <= SMs * resident CTAs per SM, so that no CTA waits for a slot.
static int wgrad_plan(const hyc_packed* saved, int rank, WgradPlan* pl) {
  const int D = saved->cols, bits = saved->bits, nseg = 8 / bits;
  const int tiles = D * bits / 8 / kTileM;
  pl->npad = (rank + 15) / 16 * 16;
  uint32_t cols = 32;
  while (cols < static_cast<uint32_t>(nseg * pl->npad)) cols *= 2;
  pl->tmem_cols = cols;
  const uint32_t b_stage = (kChunk / 8) * (pl->npad / 8) * 128u;
  const bool ref = saved->mode == HYC_MODE_R;
  const uint32_t nb = (!ref && bits < 8 && saved->group) ? nseg : 1u;
  pl->smem_bytes = 1024 + 2u * nseg * kAStage + 2u * nb * b_stage;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // long inputs: warp-specialised kernel, one CTA per SM (short ones finish before its pipeline fills)
  static const bool ws_off = getenv("HYC_WGRAD_WS") && getenv("HYC_WGRAD_WS")[0] == '0';
  pl->ws_smem = 1024 + kWsCodeStages * kWsCodeTile + static_cast<uint32_t>(ws_ab_stages(bits)) * (nseg * kAStage + nb * b_stage);
  // (used where every CTA is a code tile: with outlier-channel tiles in the launch the shared kernel below,
  // two CTAs per SM, measured faster, and so it did for 8-bit codes)
  const bool has_side = !ref && saved->n_channels > 0;
  pl->ws = !ws_off && !has_side && bits < 8 && pl->ws_smem <= kSmemPerCtaMax && saved->rows >= kWsMinRows && tiles <= sms &&
           encode_tiled_fn() != nullptr;
  // the device queries are cached per (device, bits, shared-memory size)
  struct Known { int dev, bits, per_sm; uint32_t smem; };
  static Known known[32];
  static int n_known = 0;
  static std::mutex mu;
  int per_sm = -1;
  {
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < n_known; ++i)
      if (known[i].dev == dev && known[i].bits == bits && known[i].smem == pl->smem_bytes) per_sm = known[i].per_sm;
    if (per_sm < 0) {
      per_sm = bits == 2 ? wgrad_ctas_per_sm<2>(pl->smem_bytes, dev)
               : bits == 4 ? wgrad_ctas_per_sm<4>(pl->smem_bytes, dev) : wgrad_ctas_per_sm<8>(pl->smem_bytes, dev);
      if (per_sm >= 1 && n_known < 32) known[n_known++] = Known{dev, bits, per_sm, pl->smem_bytes};
    }
  }
  if (per_sm < 1) return HYC_ERR_CUDA;
  // tensor memory: 512 columns per SM shared by the resident CTAs
  if (per_sm * cols > 512u) per_sm = 512 / cols;
  // A side CTA has no register prefetch and takes about as long per chunk as a 4-bit code CTA; with 8-bit codes
  // (one segment per chunk) the code CTAs are faster, so two side CTAs share a token slice.
  pl->side_split = bits == 8 ? 2 : 1;
  const int side_tiles = (!ref && saved->n_channels > 0) ? (saved->n_channels + kTileM - 1) / kTileM * pl->side_split : 0;
  pl->side_tiles = side_tiles;
  long long splits = pl->ws ? sms / tiles : static_cast<long long>(sms) * per_sm / (tiles + side_tiles);
  // every slice costs a partial slab (written, then read by the finish kernel) and a prologue/epilogue:
  // keep at least four chunks per slice
  const long long max_splits = ((saved->rows + kChunk - 1) / kChunk + 3) / 4;
  if (splits > max_splits) splits = max_splits;
  if (splits > 64) splits = 64;
  if (splits < 1) splits = 1;
  pl->splits = static_cast<int>(splits);
  // outlier-channel partials: one [k, rank] block per token slice
  pl->side_slices = side_tiles ? pl->splits * pl->side_split : 0;
  pl->scratch_floats = static_cast<long long>(pl->splits) * rank * D +
                       static_cast<long long>(pl->side_slices) * saved->n_channels * rank;
  // reference mode: one fp32 scale per row behind the slabs, and the ranks a pool CTA accumulates at once
  pl->row_scale_at = pl->scratch_floats;
  pl->rpw = 0;
  if (ref) {
    pl->scratch_floats += (saved->rows + 3) / 4 * 4;
    int rpw = 8;
    while (rpw > 1 && static_cast<long long>(rpw) * D * 4 > 160 * 1024) rpw >>= 1;
    pl->rpw = rpw;
  }
  return HYC_OK;
}

static int wgrad_check(const hyc_packed* saved, int rank) {
  if (!saved) return HYC_ERR_NULL;
  if (saved->mode != HYC_MODE_N && saved->mode != HYC_MODE_R) return HYC_ERR_MODE;
  if (saved->bits != 2 && saved->bits != 4 && saved->bits != 8) return HYC_ERR_BITS;
  const int D = saved->cols;
  if (saved->rows < 0 || D <= 0 || D % 128 != 0 || (D * saved->bits / 8) % kTileM != 0) return HYC_ERR_SHAPE;
  if (rank < 8 || rank > 64 || rank % 8 != 0) return HYC_ERR_SHAPE;
  if (saved->mode == HYC_MODE_R) {
    if (saved->scale_kind < HYC_SCALE_TENSOR || saved->scale_kind > HYC_SCALE_TOKEN) return HYC_ERR_MODE;
    if (saved->scale_dtype != HYC_BF16) return HYC_ERR_DTYPE;
    if (saved->seq < 1 || saved->rows > 0xffffffffLL * 1) return HYC_ERR_SHAPE;
    return HYC_OK;
  }
  if (saved->group != 0 && saved->group != 128) return HYC_ERR_SHAPE;
  if (saved->rotate != 0 && saved->rotate != 16 && saved->rotate != 64 && saved->rotate != 256 &&
      saved->rotate != 1024 && saved->rotate != 4096)
    return HYC_ERR_SHAPE;
  if (saved->rotate && D % saved->rotate != 0) return HYC_ERR_SHAPE;
  if (saved->n_channels < 0 || saved->n_channels > D) return HYC_ERR_SHAPE;
  return HYC_OK;
}

}  // namespace hyc

using namespace hyc;

extern "C" {

int64_t hyc_lora_wgrad_scratch_floats(const hyc_packed* saved, int32_t rank) {
  const int rc = wgrad_check(saved, rank);
  if (rc != HYC_OK) return rc;
  WgradPlan pl;
  const int rp = wgrad_plan(saved, rank, &pl);
  if (rp != HYC_OK) return rp;
  return pl.scratch_floats > 0 ? pl.scratch_floats : 1;
}

int hyc_lora_wgrad(const hyc_packed* saved, const void* grad, int32_t rank, float* out, float* partials,
                   void* stream_) {
  return hyc_lora_wgrad_to(saved, grad, rank, out, HYC_F32, 0, partials, stream_);
}

int hyc_lora_wgrad_to(const hyc_packed* saved, const void* grad, int32_t rank, void* out, int32_t out_dtype,
                      int32_t accumulate, float* partials, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int rc = wgrad_check(saved, rank);
  if (rc != HYC_OK) return rc;
  if (out_dtype != HYC_F32 && out_dtype != HYC_BF16) return HYC_ERR_DTYPE;
  const size_t out_elem = out_dtype == HYC_F32 ? sizeof(float) : sizeof(__nv_bfloat16);
  const bool ref = saved->mode == HYC_MODE_R;
  if (!saved->codes || !grad || !out || !partials) return HYC_ERR_NULL;
  if (ref ? (!saved->scale || !saved->pool || !saved->row_meta) : !saved->scales) return HYC_ERR_NULL;
  if (!ref && saved->n_channels > 0 && (!saved->channels || !saved->out_value)) return HYC_ERR_NULL;
  const int D = saved->cols;
  if ((reinterpret_cast<uintptr_t>(grad) & 15u) || (reinterpret_cast<uintptr_t>(saved->codes) & 15u) ||
      (reinterpret_cast<uintptr_t>(partials) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u))
    return HYC_ERR_ALIGN;
  const long long slab = static_cast<long long>(rank) * D;
  if (saved->rows == 0) {
    if (!accumulate && cudaMemsetAsync(out, 0, slab * out_elem, stream) != cudaSuccess) return HYC_ERR_CUDA;
    return HYC_OK;
  }
  WgradPlan pl;
  const int rp = wgrad_plan(saved, rank, &pl);
  if (rp != HYC_OK) return rp;
  const int splits = pl.splits;
  WgradArgs a;
  memset(&a, 0, sizeof(a));
  a.p.mode = saved->mode; a.p.bits = saved->bits; a.p.rows = saved->rows; a.p.cols = D; a.p.seq = saved->seq;
  a.p.codes = static_cast<unsigned char*>(saved->codes);
  a.p.status = saved->status;
  a.p.group = ref ? 0 : saved->group; a.p.rotate = ref ? 0 : saved->rotate;
  a.p.scales = saved->scales;
  if (ref) {
    float* row_scale = partials + pl.row_scale_at;
    r_row_scale_kernel<<<static_cast<unsigned int>((saved->rows + 255) / 256), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(saved->scale), saved->scale_kind, saved->seq, saved->rows, row_scale);
    HYC_LAUNCHED();
    a.p.scales = row_scale;
  }
  a.grad = static_cast<const __nv_bfloat16*>(grad);
  a.rank = rank;
  a.npad = pl.npad;
  const long long per = (saved->rows + splits - 1) / splits;
  a.tokens_per_split = (per + kChunk - 1) / kChunk * kChunk;
  a.partials = partials;
  a.tmem_cols = pl.tmem_cols;
  a.tiles = D * saved->bits / 8 / kTileM;
  a.side_split = pl.side_split;
  a.k = ref ? 0 : saved->n_channels;
  a.out_value = static_cast<const __nv_bfloat16*>(saved->out_value);
  a.side = partials + static_cast<long long>(splits) * slab;
  const uint32_t smem_bytes = pl.smem_bytes;
  const long long code_tokens_per_split = (per + kChunk - 1) / kChunk * kChunk;
  CUtensorMap tmap;
  if (pl.ws && code_tensor_map(saved, &tmap)) {
    // records without outlier-channel tiles: every CTA is a code tile, on the warp-specialised kernel
    const dim3 wgrid(a.tiles, splits);
#define HYC_WS(B)                                                                                         \
  {                                                                                                       \
    auto kern = lora_wgrad_ws_kernel<B>;                                                                  \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.ws_smem) !=       \
        cudaSuccess)                                                                                      \
      return HYC_ERR_CUDA;                                                                                \
    kern<<<wgrid, kWsThreads, pl.ws_smem, stream>>>(a, tmap); HYC_LAUNCHED();                             \
  }
    if (saved->bits == 2) HYC_WS(2) else HYC_WS(4)
#undef HYC_WS
  } else {
    const dim3 grid(a.tiles + pl.side_tiles, splits);
#define HYC_WG(B)                                                                                         \
  {                                                                                                       \
    auto kern = lora_wgrad_kernel<B>;                                                                     \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes) !=       \
        cudaSuccess)                                                                                      \
      return HYC_ERR_CUDA;                                                                                \
    kern<<<grid, kWgThreads, smem_bytes, stream>>>(a); HYC_LAUNCHED();                                    \
  }
    if (saved->bits == 2) HYC_WG(2) else if (saved->bits == 4) HYC_WG(4) else HYC_WG(8)
#undef HYC_WG
  }
  if (cudaGetLastError() != cudaSuccess) return HYC_ERR_CUDA;
  const __nv_bfloat16* colscale =
      (ref && saved->scale_kind == HYC_SCALE_CHANNEL) ? static_cast<const __nv_bfloat16*>(saved->scale) : nullptr;
  if (ref) {
    // element outliers into the slabs
    const size_t sm = static_cast<size_t>(pl.rpw) * D * 4;
    if (cudaFuncSetAttribute(wgrad_pool_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm) != cudaSuccess)
      return HYC_ERR_CUDA;
    wgrad_pool_kernel<<<dim3((rank + pl.rpw - 1) / pl.rpw, splits), 512, sm, stream>>>(
        saved->pool, reinterpret_cast<const uint2*>(saved->row_meta), a.grad, rank, pl.rpw, D, saved->rows,
        code_tokens_per_split, colscale, partials);
    HYC_LAUNCHED();
    if (cudaGetLastError() != cudaSuccess) return HYC_ERR_CUDA;
  }
  const int k = ref ? 0 : saved->n_channels;
  const float* side = partials + static_cast<long long>(splits) * slab;
  {
    // parts of a row are independent when they hold whole rotation blocks
    const int unit = (!ref && saved->rotate) ? saved->rotate : 128;
    int parts = 8;
    while (parts > 1 && (D % parts != 0 || (D / parts) % unit != 0 || (D / parts) % 128 != 0)) parts >>= 1;
    const size_t sm = static_cast<size_t>(D / parts) * 4;
    if (sm > 48 * 1024)
      if (cudaFuncSetAttribute(wgrad_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm) != cudaSuccess)
        return HYC_ERR_CUDA;
    wgrad_finish_kernel<<<dim3(rank, parts), 256, sm, stream>>>(partials, splits, side, pl.side_slices, saved->channels,
                                                               pl.side_slices > 0 ? k : 0, rank, D,
                                                               ref ? 0 : saved->rotate, colscale,
                                                               out_dtype == HYC_F32 ? static_cast<float*>(out) : nullptr,
                                                               out_dtype == HYC_BF16 ? static_cast<__nv_bfloat16*>(out) : nullptr,
                                                               accumulate != 0);
    HYC_LAUNCHED();
  }
  return cudaGetLastError() == cudaSuccess ? HYC_OK : HYC_ERR_CUDA;
}

}  // extern "C"
