// Calibration kernels for the channel-outlier mode: column absmax of an
// activation and deterministic top-k channel selection (ties to the lower
// index, ascending output).  They run on the first calls of a site only.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>

#include "../../include/hyc_b200.h"
#include "hyc_common.cuh"

namespace hyc {

// Each CTA walks rows blockIdx.x, +gridDim.x, ...; thread t owns the 8-channel
// vectors t, t+blockDim, ... of every row and keeps their running maxima in
// shared memory (one owner per column, so no atomics there).  The CTA's maxima
// are merged into the global score with integer atomicMax, which orders
// non-negative floats correctly.
template <typename XT>
__global__ void __launch_bounds__(256) channel_absmax_kernel(const XT* x, long long rows, int D, int seq, int chunks,
                                                             long long row_stride, long long batch_stride,
                                                             long long chunk_stride, float* score) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* acc = reinterpret_cast<float*>(smem_raw);
  const int nvec = D >> 3;
  const int clen = D / chunks;
  for (int c = threadIdx.x; c < D; c += blockDim.x) acc[c] = 0.f;
  __syncthreads();  // columns are re-partitioned by 8-channel vector below
  for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
    const XT* src = chunks == 1 ? x + row * row_stride : x + (row / seq) * batch_stride + (row % seq) * row_stride;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const int col = v << 3;
      const int c = col / clen;
      float f[8];
      load8<XT>(src + c * chunk_stride, col - c * clen, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[col + e] = fmaxf(acc[col + e], fabsf(f[e]));
    }
  }
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int col = (v << 3) + e;
      atomicMax(reinterpret_cast<unsigned int*>(score) + col, __float_as_uint(acc[col]));
    }
  }
}

// Scores are ordered through an integer key so that the order is total whatever the bits are:
// finite values and infinities keep their numeric order, -0 counts as +0, and every NaN sits
// above +inf (where a descending sort puts it).  With a total order exactly k channels have a
// rank below k, which is what lets the gather below write a k-entry list.
__device__ __forceinline__ unsigned int score_key(float s) {
  if (s != s) return 0xFFFFFFFFu;
  const unsigned int u = __float_as_uint(s + 0.f);  // -0 + 0 = +0
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// rank[c] = number of channels that come before c when ordering by
// (score descending, index ascending)
__global__ void __launch_bounds__(256) channel_rank_kernel(const float* score, int D, int* rank) {
  __shared__ unsigned int tile[1024];
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const unsigned int mine = c < D ? score_key(score[c]) : 0u;
  int before = 0;
  for (int j0 = 0; j0 < D; j0 += 1024) {
    __syncthreads();
    for (int j = threadIdx.x; j < 1024; j += blockDim.x) tile[j] = (j0 + j < D) ? score_key(score[j0 + j]) : 0u;
    __syncthreads();
    const int n = min(1024, D - j0);
    for (int j = 0; j < n; ++j) {
      const unsigned int s = tile[j];
      before += (s > mine || (s == mine && (j0 + j) < c)) ? 1 : 0;
    }
  }
  if (c < D) rank[c] = before;
}

// Ascending list of the channels whose rank is below k.  One CTA: thread t owns a contiguous
// run of channels, counts its selected ones, a block-wide exclusive scan of the counts gives
// the run's first output slot, and the run is walked once more to write.  A slot at or beyond
// k is never written (it cannot occur with the ranks of channel_rank_kernel; the check keeps
// the store inside the caller's list for any rank array).
constexpr int kGatherThreads = 1024;
__global__ void __launch_bounds__(kGatherThreads) channel_gather_kernel(const int* rank, int D, int k, int* channels) {
  __shared__ int warp_sum[kGatherThreads / 32];
  const int per = (D + kGatherThreads - 1) / kGatherThreads;
  const int c0 = min(D, static_cast<int>(threadIdx.x) * per), c1 = min(D, c0 + per);
  int mine = 0;
  for (int c = c0; c < c1; ++c) mine += rank[c] < k ? 1 : 0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  if (lane == 31) warp_sum[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = warp_sum[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += up;
    }
    warp_sum[lane] = w;  // inclusive over warps
  }
  __syncthreads();
  int pos = incl - mine + (warp ? warp_sum[warp - 1] : 0);
  for (int c = c0; c < c1; ++c) {
    if (rank[c] < k) {
      if (pos < k) channels[pos] = c;
      ++pos;
    }
  }
}

// Scratch of the allocation-free selection entry point: one rank per channel.  The array
// lives in every GPU context that loads this library, until the process exits.
constexpr int kStaticSelectMaxCols = 16384;
static __device__ __align__(256) int g_select_rank_scratch[kStaticSelectMaxCols];

}  // namespace hyc

using namespace hyc;

extern "C" {

int hyc_channel_absmax(const hyc_dense* x, int64_t rows, int32_t cols, int32_t seq, float* score, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!x || !x->base || !score) return HYC_ERR_NULL;
  if (rows < 0 || cols <= 0 || cols % 128 != 0 || cols > 65408 || seq < 1) return HYC_ERR_SHAPE;
  if (x->dtype != HYC_F32 && x->dtype != HYC_BF16) return HYC_ERR_DTYPE;
  if (x->chunks < 1 || cols % x->chunks != 0 || (cols / x->chunks) % 8 != 0) return HYC_ERR_SHAPE;
  const int es = x->dtype == HYC_BF16 ? 2 : 4;
  if ((reinterpret_cast<uintptr_t>(x->base) & 15u) || (x->row_stride * es) % 16 != 0 ||
      (x->chunks > 1 && ((x->batch_stride * es) % 16 != 0 || (x->chunk_stride * es) % 16 != 0)))
    return HYC_ERR_ALIGN;
  if (rows == 0) return HYC_OK;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long grid = static_cast<long long>(sms) * 4;
  if (grid > rows) grid = rows;
  const size_t smem = static_cast<size_t>(cols) * 4;
  if (x->dtype == HYC_BF16) {
    auto kern = channel_absmax_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kern<<<static_cast<int>(grid), 256, smem, stream>>>(static_cast<const __nv_bfloat16*>(x->base), rows, cols, seq,
                                                        x->chunks, x->row_stride, x->batch_stride, x->chunk_stride,
                                                        score); HYC_LAUNCHED();
  } else {
    auto kern = channel_absmax_kernel<float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kern<<<static_cast<int>(grid), 256, smem, stream>>>(static_cast<const float*>(x->base), rows, cols, seq, x->chunks,
                                                        x->row_stride, x->batch_stride, x->chunk_stride, score); HYC_LAUNCHED();
  }
  return cudaGetLastError() == cudaSuccess ? HYC_OK : HYC_ERR_CUDA;
}

int hyc_select_channels(const float* score, int32_t cols, int32_t k, int32_t* channels, int32_t* rank_scratch,
                        void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!score || !rank_scratch || (k > 0 && !channels)) return HYC_ERR_NULL;
  if (cols <= 0 || k < 0 || k > cols) return HYC_ERR_SHAPE;
  if (k == 0) return HYC_OK;
  const int blocks = (cols + 255) / 256;
  channel_rank_kernel<<<blocks, 256, 0, stream>>>(score, cols, rank_scratch); HYC_LAUNCHED();
  channel_gather_kernel<<<1, kGatherThreads, 0, stream>>>(rank_scratch, cols, k, channels); HYC_LAUNCHED();
  return cudaGetLastError() == cudaSuccess ? HYC_OK : HYC_ERR_CUDA;
}

int hyc_select_channels_static_max_cols(void) { return kStaticSelectMaxCols; }

int hyc_select_channels_noalloc(const float* score, int32_t cols, int32_t k, int32_t* channels, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!score || (k > 0 && !channels)) return HYC_ERR_NULL;
  if (cols <= 0 || k < 0 || k > cols) return HYC_ERR_SHAPE;
  if (cols > kStaticSelectMaxCols) return HYC_ERR_CAPACITY;
  if (k == 0) return HYC_OK;
  // In host code the array's name is only a handle: the device address has to be asked for,
  // once per device, with that device current.  The first call on a device does it.
  // The cache is read and written by any host thread: entries are atomics, and two threads that
  // both miss simply look the same address up twice.  cudaDeviceReset() invalidates the address;
  // a process that resets a device must not call this entry point on it afterwards.
  static std::atomic<int*> scratch_of_device[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return HYC_ERR_CUDA;
  int* rank = scratch_of_device[dev].load(std::memory_order_acquire);
  if (!rank) {
    int* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_select_rank_scratch) != cudaSuccess || !ptr)
      return HYC_ERR_CUDA;
    scratch_of_device[dev].store(ptr, std::memory_order_release);
    rank = ptr;
  }
  const int blocks = (cols + 255) / 256;
  // every rank in [0, cols) is rewritten by the first kernel, so nothing has to start at zero
  channel_rank_kernel<<<blocks, 256, 0, stream>>>(score, cols, rank); HYC_LAUNCHED();
  channel_gather_kernel<<<1, kGatherThreads, 0, stream>>>(rank, cols, k, channels); HYC_LAUNCHED();
  return cudaGetLastError() == cudaSuccess ? HYC_OK : HYC_ERR_CUDA;
}

}  // extern "C"
