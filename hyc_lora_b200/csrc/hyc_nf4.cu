// Blockwise 4-bit codebook weights for the frozen base linears of the host models:
// 64 consecutive values share one fp32 absmax; a byte holds two 4-bit indices into a
// 16-entry codebook (high nibble first).  Only the dequantiser runs on the training path
// (the bf16 weight is rebuilt for the forward GEMM and again for the backward GEMM, so the
// frozen layer keeps nothing but the packed weight).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hyc_b200.h"
#include "hyc_common.cuh"

namespace hyc {

// One thread rebuilds 8 values (4 bytes) per step -> one 16-byte store; a warp reads 128 and writes 512
// contiguous bytes per instruction.  Four independent steps per loop trip keep several loads in flight.
constexpr int kNf4Unroll = 4;

__device__ __forceinline__ uint4 nf4_expand8(uint32_t c, float s, const float* cbk) {
  float f[8];
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const uint32_t byte = (c >> (8 * b)) & 0xffu;
    f[2 * b] = cbk[byte >> 4] * s;
    f[2 * b + 1] = cbk[byte & 15u] * s;
  }
  return pack_bf16x8(f);
}

__global__ void __launch_bounds__(256) nf4_dequant_kernel(const uint32_t* codes, const float* absmax,
                                                          const float* codebook, long long n8, uint4* out) {
  __shared__ float cbk[16];
  if (threadIdx.x < 16) cbk[threadIdx.x] = codebook[threadIdx.x];
  __syncthreads();
  const long long span = static_cast<long long>(blockDim.x) * kNf4Unroll;
  for (long long base = blockIdx.x * span + threadIdx.x; base < n8; base += gridDim.x * span) {
    uint32_t c[kNf4Unroll];
    float s[kNf4Unroll];
#pragma unroll
    for (int u = 0; u < kNf4Unroll; ++u) {
      const long long i = base + static_cast<long long>(u) * blockDim.x;
      c[u] = i < n8 ? __ldg(codes + i) : 0u;
      s[u] = i < n8 ? __ldg(absmax + (i >> 3)) : 0.f;   // 8 values per step, 64 per scale
    }
#pragma unroll
    for (int u = 0; u < kNf4Unroll; ++u) {
      const long long i = base + static_cast<long long>(u) * blockDim.x;
      if (i < n8) out[i] = nf4_expand8(c[u], s[u], cbk);
    }
  }
}

}  // namespace hyc

extern "C" int hyc_nf4_dequant(const void* codes, const float* absmax, const float* codebook, int64_t n,
                               void* out_bf16, void* stream) {
  if (!codes || !absmax || !codebook || !out_bf16) return HYC_ERR_NULL;
  if (n < 0 || n % 64 != 0) return HYC_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(codes) & 3u) || (reinterpret_cast<uintptr_t>(out_bf16) & 15u)) return HYC_ERR_ALIGN;
  if (n == 0) return HYC_OK;
  const long long n8 = n / 8;
  const long long per_block = 256LL * hyc::kNf4Unroll;
  long long blocks = (n8 + per_block - 1) / per_block;
  if (blocks > 148 * 16) blocks = 148 * 16;
  hyc::nf4_dequant_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(codes), absmax, codebook, n8, static_cast<uint4*>(out_bf16)); HYC_LAUNCHED();
  return cudaGetLastError() == cudaSuccess ? HYC_OK : HYC_ERR_CUDA;
}
