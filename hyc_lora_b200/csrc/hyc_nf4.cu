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

// one thread rebuilds 16 values (8 bytes) -> two 16-byte stores
__global__ void nf4_dequant_kernel(const uint2* codes, const float* absmax, const float* codebook, long long n16,
                                   uint4* out) {
  __shared__ float cbk[16];
  if (threadIdx.x < 16) cbk[threadIdx.x] = codebook[threadIdx.x];
  __syncthreads();
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const uint2 c = codes[i];
    const float s = absmax[i >> 2];  // 16 values per thread, 64 per block
    float f[16];
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const uint32_t byte = ((b < 4 ? c.x >> (8 * b) : c.y >> (8 * (b - 4))) & 0xffu);
      f[2 * b] = cbk[byte >> 4] * s;
      f[2 * b + 1] = cbk[byte & 15u] * s;
    }
    float lo[8], hi[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { lo[e] = f[e]; hi[e] = f[8 + e]; }
    out[2 * i] = pack_bf16x8(lo);
    out[2 * i + 1] = pack_bf16x8(hi);
  }
}

}  // namespace hyc

extern "C" int hyc_nf4_dequant(const void* codes, const float* absmax, const float* codebook, int64_t n,
                               void* out_bf16, void* stream) {
  if (!codes || !absmax || !codebook || !out_bf16) return HYC_ERR_NULL;
  if (n < 0 || n % 64 != 0) return HYC_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(codes) & 7u) || (reinterpret_cast<uintptr_t>(out_bf16) & 15u)) return HYC_ERR_ALIGN;
  if (n == 0) return HYC_OK;
  const long long n16 = n / 16;
  long long blocks = (n16 + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  hyc::nf4_dequant_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint2*>(codes), absmax, codebook, n16, static_cast<uint4*>(out_bf16));
  return cudaGetLastError() == cudaSuccess ? HYC_OK : HYC_ERR_CUDA;
}
