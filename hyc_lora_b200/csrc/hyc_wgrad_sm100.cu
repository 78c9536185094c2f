// LoRA-A weight gradient straight from packed codes on the 5th-generation tensor cores:
//
//     dA[n, d] = sum_t G[t, n] * X_hat[t, d]        (n < rank, d < D, t < T)
//
// X_hat is never written to HBM.  A CTA owns 128 packed byte columns of the code rows (that is
// 8/bits tiles of 128 channels, one per row segment) and a slice of the tokens.  For every
// chunk of 64 tokens all threads rebuild the bf16 values from the codes (integer -> float
// through the mantissa of 2^23, times the token / group scale, one rounding to bf16 -- the
// same values the decompress kernel produces) and store them, 16 bytes per token and 8
// channels, into shared memory in the MN-major no-swizzle core-matrix layout tcgen05 reads;
// the gradient rows are copied into the same layout.  One thread then issues
// tcgen05.mma (M = 128 channels, N = rank, K = 16 tokens per instruction) with the
// accumulators in tensor memory, and commits to an mbarrier that tells everybody when the
// staging buffer may be overwritten (two buffers, so conversion of chunk c+1 overlaps the
// MMAs of chunk c).  At the end four warps read the accumulators back with tcgen05.ld and
// store one partial [rank, D] slab per token slice; a second kernel adds the slabs.
//
// Channel-outlier mode only.  Outlier channels carry the zero code, so their columns come out
// as zero here; the caller adds G^T * out_value there.  With rotation the kernel contracts the
// un-rotated codes and the rotation is applied to the `rank` output rows afterwards
// (X_hat = Q H  =>  G^T X_hat = (G^T Q) H).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/hyc_b200.h"
#include "hyc_bwd_fast.cuh"

namespace hyc {

constexpr int kChunk = 64;          // tokens per staging buffer
constexpr int kTileM = 128;         // channels per accumulator tile
constexpr int kWgThreads = 256;

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

// D[tmem] (+)= A[smem] * B[smem], bf16 x bf16 -> fp32, issued by one thread
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
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

// Shared-memory matrix descriptor, no swizzle.  Core matrix = 8 rows of 16 bytes; `lbo` is the
// byte distance between core matrices along K, `sbo` along M/N (MN-major operands).
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (static_cast<uint64_t>(lbo >> 4) << 16) |
         (static_cast<uint64_t>(sbo >> 4) << 32) | (1ull << 46);
}

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
  unsigned char* b_buf = a_buf + 2u * NSEG * kAStage;              // [2][b_stage]
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
  const int byte0 = blockIdx.x * kTileM;                 // first packed byte column of this CTA
  const long long t_begin = static_cast<long long>(blockIdx.y) * a.tokens_per_split;
  const long long t_end = min(p.rows, t_begin + a.tokens_per_split);
  const int nchunks = t_end > t_begin ? static_cast<int>((t_end - t_begin + kChunk - 1) / kChunk) : 0;
  const uint32_t idesc = instr_desc(npad);
  // conversion mapping: lane = token-in-group (k0) + 8 * (unit & 3); a warp item = (token group, unit >> 2)
  const int k0 = lane & 7, u_lo = lane >> 3;
  constexpr int kAItems = (kChunk / 8) * 4 / (kWgThreads / 32);   // A items per warp and chunk (4)
  constexpr int kBItems = 2;                                      // B items per warp and chunk (at most)
  const int b_per_tg = (npad / 8 + 3) / 4;
  // The packed bytes, scales and gradient vectors of chunk c+1 are loaded into registers before
  // chunk c is converted, so their latency hides behind the conversion and the MMAs.
  uint2 cb_reg[kAItems];
  float sc_reg[kAItems];
  uint4 g_reg[kBItems];
  auto fetch = [&](int c) {
    const long long t0 = t_begin + static_cast<long long>(c) * kChunk;
#pragma unroll
    for (int i = 0; i < kAItems; ++i) {
      const int item = warp + i * (kWgThreads / 32);
      const int tg = item >> 2, unit = ((item & 3) << 2) + u_lo;
      const long long t = t0 + tg * 8 + k0;
      cb_reg[i] = make_uint2(0, 0);
      sc_reg[i] = 0.f;
      if (t < t_end) {
        cb_reg[i] = ld_stream_u2(p.codes + t * cb + byte0 + (unit << 3));
        if (!p.group) sc_reg[i] = __ldg(p.scales + t);
      }
    }
#pragma unroll
    for (int i = 0; i < kBItems; ++i) {
      const int item = warp + i * (kWgThreads / 32);
      const int tg = item / b_per_tg, n1 = (item % b_per_tg) * 4 + u_lo;
      const long long t = t0 + tg * 8 + k0;
      g_reg[i] = make_uint4(0, 0, 0, 0);
      if (item < (kChunk / 8) * b_per_tg && n1 < npad / 8 && t < t_end && (n1 << 3) < a.rank)
        g_reg[i] = *reinterpret_cast<const uint4*>(a.grad + t * a.rank + (n1 << 3));
    }
  };
  if (nchunks > 0) fetch(0);
  for (int c = 0; c < nchunks; ++c) {
    const int buf = c & 1;
    // move this chunk's registers aside and start the next chunk's loads
    uint2 cb_cur[kAItems];
    float sc_cur[kAItems];
    uint4 g_cur[kBItems];
#pragma unroll
    for (int i = 0; i < kAItems; ++i) { cb_cur[i] = cb_reg[i]; sc_cur[i] = sc_reg[i]; }
#pragma unroll
    for (int i = 0; i < kBItems; ++i) g_cur[i] = g_reg[i];
    if (c + 1 < nchunks) fetch(c + 1);
    if (c >= 2) {
      if (!mbar_wait_bounded(&bar_done[buf], ((c >> 1) - 1) & 1)) *fail = 1;
      tc_fence_after();
    }
    const long long t0 = t_begin + static_cast<long long>(c) * kChunk;
    unsigned char* abase = a_buf + static_cast<uint32_t>(buf) * NSEG * kAStage;
    unsigned char* bbase = b_buf + static_cast<uint32_t>(buf) * b_stage;
    // ---- A: codes -> bf16 values
#pragma unroll
    for (int i = 0; i < kAItems; ++i) {
      const int item = warp + i * (kWgThreads / 32);
      const int tg = item >> 2, unit = ((item & 3) << 2) + u_lo;
      const long long t = t0 + tg * 8 + k0;
      const bool live = t < t_end;
#pragma unroll
      for (int s = 0; s < NSEG; ++s) {
        uint4 packed_vals = make_uint4(0, 0, 0, 0);
        if (live) {
          float f[8];
          const int col = s * segw + byte0 + (unit << 3);
          const float sc = p.group ? __ldg(p.scales + t * G + (col >> 7)) : sc_cur[i];
          dequant8<BITS>(cb_cur[i], s, sc, f);
          packed_vals = pack_bf16x8(f);
        }
        *reinterpret_cast<uint4*>(abase + s * kAStage + tg * kALbo + unit * kASbo + k0 * 16) = packed_vals;
      }
    }
    // ---- B: gradient rows
#pragma unroll
    for (int i = 0; i < kBItems; ++i) {
      const int item = warp + i * (kWgThreads / 32);
      const int tg = item / b_per_tg, n1 = (item % b_per_tg) * 4 + u_lo;
      if (item < (kChunk / 8) * b_per_tg && n1 < npad / 8)
        *reinterpret_cast<uint4*>(bbase + tg * b_lbo + n1 * kBSbo + k0 * 16) = g_cur[i];
    }
    fence_proxy_async();          // generic-proxy stores -> visible to the tensor-core (async) proxy
    tc_fence_before();
    __syncthreads();
    if (*fail) break;
    if (tid == 0) {
      tc_fence_after();
      const uint32_t a_addr = smem_u32(abase), b_addr = smem_u32(bbase);
#pragma unroll
      for (int s = 0; s < NSEG; ++s) {
        for (int ks = 0; ks < kChunk / 16; ++ks) {
          const uint64_t da = smem_desc(a_addr + s * kAStage + ks * 2 * kALbo, kALbo, kASbo);
          const uint64_t db = smem_desc(b_addr + ks * 2 * b_lbo, b_lbo, kBSbo);
          umma_bf16(tmem_base + static_cast<uint32_t>(s * npad), da, db, idesc, (c > 0 || ks > 0) ? 1u : 0u);
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
  if (warp < 4) {
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

// out[n, d] = sum over slabs
__global__ void wgrad_reduce_kernel(const float* partials, int splits, long long slab, float* out) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= slab) return;
  float s = 0.f;
  for (int q = 0; q < splits; ++q) s += partials[q * slab + i];
  out[i] = s;
}

// block rotation of every output row (rows are short: one CTA per row, row staged in shared memory)
__global__ void wgrad_rotate_rows_kernel(float* out, int D, int n) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* rowbuf = reinterpret_cast<float*>(smem_raw);
  float* row = out + static_cast<long long>(blockIdx.x) * D;
  for (int c = threadIdx.x; c < D; c += blockDim.x) rowbuf[c] = row[c];
  __syncthreads();
  fwht_row<float, false>(rowbuf, nullptr, rowbuf, D, n);
  for (int c = threadIdx.x; c < D; c += blockDim.x) row[c] = rowbuf[c];
}

static int wgrad_splits(long long rows, int cols, int bits) {
  const int tiles = cols * bits / 8 / kTileM;
  if (tiles <= 0) return 1;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long splits = (2 * sms + tiles - 1) / tiles;  // two CTAs per SM
  const long long max_splits = (rows + kChunk - 1) / kChunk;
  if (splits > max_splits) splits = max_splits;
  if (splits < 1) splits = 1;
  if (splits > 64) splits = 64;
  return static_cast<int>(splits);
}

}  // namespace hyc

using namespace hyc;

extern "C" {

int hyc_lora_wgrad_splits(int64_t rows, int32_t cols, int32_t bits) {
  if (rows < 0 || cols <= 0 || (bits != 2 && bits != 4 && bits != 8)) return HYC_ERR_SHAPE;
  return wgrad_splits(rows, cols, bits);
}

int hyc_lora_wgrad(const hyc_packed* saved, const void* grad, int32_t rank, float* out, float* partials,
                   void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!saved || !saved->codes || !grad || !out || !partials) return HYC_ERR_NULL;
  if (saved->mode != HYC_MODE_N) return HYC_ERR_MODE;
  if (saved->bits != 2 && saved->bits != 4 && saved->bits != 8) return HYC_ERR_BITS;
  const int D = saved->cols;
  if (saved->rows < 0 || D <= 0 || D % 128 != 0 || (D * saved->bits / 8) % kTileM != 0) return HYC_ERR_SHAPE;
  if (rank < 8 || rank > 64 || rank % 8 != 0) return HYC_ERR_SHAPE;
  if (saved->group != 0 && saved->group != 128) return HYC_ERR_SHAPE;
  if (saved->rotate != 0 && saved->rotate != 16 && saved->rotate != 64 && saved->rotate != 256 &&
      saved->rotate != 1024 && saved->rotate != 4096)
    return HYC_ERR_SHAPE;
  if (saved->rotate && D % saved->rotate != 0) return HYC_ERR_SHAPE;
  if (!saved->scales) return HYC_ERR_NULL;
  if ((reinterpret_cast<uintptr_t>(grad) & 15u) || (reinterpret_cast<uintptr_t>(saved->codes) & 15u)) return HYC_ERR_ALIGN;
  const long long slab = static_cast<long long>(rank) * D;
  if (saved->rows == 0) {
    if (cudaMemsetAsync(out, 0, slab * sizeof(float), stream) != cudaSuccess) return HYC_ERR_CUDA;
    return HYC_OK;
  }
  const int nseg = 8 / saved->bits;
  const int splits = wgrad_splits(saved->rows, D, saved->bits);
  WgradArgs a;
  memset(&a, 0, sizeof(a));
  a.p.mode = saved->mode; a.p.bits = saved->bits; a.p.rows = saved->rows; a.p.cols = D; a.p.seq = saved->seq;
  a.p.codes = static_cast<unsigned char*>(saved->codes);
  a.p.status = saved->status;
  a.p.group = saved->group; a.p.rotate = saved->rotate;
  a.p.scales = saved->scales;
  a.grad = static_cast<const __nv_bfloat16*>(grad);
  a.rank = rank;
  a.npad = (rank + 15) / 16 * 16;
  const long long per = (saved->rows + splits - 1) / splits;
  a.tokens_per_split = (per + kChunk - 1) / kChunk * kChunk;
  a.partials = partials;
  uint32_t cols = 32;
  while (cols < static_cast<uint32_t>(nseg * a.npad)) cols *= 2;
  a.tmem_cols = cols;
  const uint32_t b_stage = (kChunk / 8) * (a.npad / 8) * 128u;
  const uint32_t smem_bytes = 1024 + 2u * nseg * kAStage + 2u * b_stage;
  const dim3 grid(D * saved->bits / 8 / kTileM, splits);
#define HYC_WG(B)                                                                                         \
  {                                                                                                       \
    auto kern = lora_wgrad_kernel<B>;                                                                     \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes) !=       \
        cudaSuccess)                                                                                      \
      return HYC_ERR_CUDA;                                                                                \
    kern<<<grid, kWgThreads, smem_bytes, stream>>>(a);                                                    \
  }
  if (saved->bits == 2) HYC_WG(2) else if (saved->bits == 4) HYC_WG(4) else HYC_WG(8)
#undef HYC_WG
  if (cudaGetLastError() != cudaSuccess) return HYC_ERR_CUDA;
  wgrad_reduce_kernel<<<static_cast<int>((slab + 255) / 256), 256, 0, stream>>>(partials, splits, slab, out);
  if (saved->rotate) {
    const size_t sm = static_cast<size_t>(D) * 4;
    if (sm > 48 * 1024)
      cudaFuncSetAttribute(wgrad_rotate_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
    wgrad_rotate_rows_kernel<<<rank, 256, sm, stream>>>(out, D, saved->rotate);
  }
  return cudaGetLastError() == cudaSuccess ? HYC_OK : HYC_ERR_CUDA;
}

}  // extern "C"
