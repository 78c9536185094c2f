// Rotary position embedding applied in place to the query and key projections of the host
// models, [tokens, heads, head_dim] bf16 each, in one launch (the models of the reference
// apply it with eager tensor ops: rotate_half / apply_rotary_pos_emb, models/modeling_llama.py:228-260).
// Pair (i, i + head_dim/2) of every head is rotated by the angle of (position, i):
//     y[i]       = x[i] cos - x[i + h/2] sin
//     y[i + h/2] = x[i + h/2] cos + x[i] sin
// computed in fp32 and rounded once.  `inverse` rotates by the negative angle, which is the
// backward of the forward rotation (the transform is orthogonal).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hyc_b200.h"
#include "hyc_common.cuh"

namespace hyc {

// one thread: 8 consecutive pair indices of one head of one token
__global__ void rope_kernel(__nv_bfloat16* q, __nv_bfloat16* k, const float* __restrict__ cos_sin, long long tokens,
                            int seq, int heads_q, int heads_k, int head_dim, float sign) {
  const int half = head_dim >> 1, vec = half >> 3;           // 16-byte pieces per half head
  const int heads = heads_q + heads_k;
  const long long total = tokens * heads * vec;
  for (long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; t < total;
       t += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int v = static_cast<int>(t % vec);
    const long long th = t / vec;
    const int h = static_cast<int>(th % heads);
    const long long tok = th / heads;
    const int pos = static_cast<int>(tok % seq);
    __nv_bfloat16* base = h < heads_q ? q + (tok * heads_q + h) * head_dim : k + (tok * heads_k + (h - heads_q)) * head_dim;
    float a[8], b[8];
    load8<__nv_bfloat16>(base, v << 3, a);
    load8<__nv_bfloat16>(base, half + (v << 3), b);
    const float4* cs = reinterpret_cast<const float4*>(cos_sin + (static_cast<long long>(pos) * half + (v << 3)) * 2);
    float ya[8], yb[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float4 c2 = __ldg(cs + e);                       // cos, sin of two consecutive pair indices
      const float s0 = sign * c2.y, s1 = sign * c2.w;
      ya[2 * e] = a[2 * e] * c2.x - b[2 * e] * s0;
      yb[2 * e] = b[2 * e] * c2.x + a[2 * e] * s0;
      ya[2 * e + 1] = a[2 * e + 1] * c2.z - b[2 * e + 1] * s1;
      yb[2 * e + 1] = b[2 * e + 1] * c2.z + a[2 * e + 1] * s1;
    }
    store8<__nv_bfloat16>(base, v << 3, ya);
    store8<__nv_bfloat16>(base, half + (v << 3), yb);
  }
}

}  // namespace hyc

extern "C" int hyc_rope(void* q, void* k, const float* cos_sin, int64_t tokens, int32_t seq, int32_t heads_q,
                        int32_t heads_k, int32_t head_dim, int32_t inverse, void* stream) {
  if (!q || !k || !cos_sin) return HYC_ERR_NULL;
  if (tokens < 0 || seq < 1 || heads_q < 1 || heads_k < 1 || head_dim < 16 || head_dim % 16 != 0) return HYC_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q) & 15u) || (reinterpret_cast<uintptr_t>(k) & 15u) ||
      (reinterpret_cast<uintptr_t>(cos_sin) & 15u))
    return HYC_ERR_ALIGN;
  if (tokens == 0) return HYC_OK;
  const long long total = tokens * (heads_q + heads_k) * (head_dim / 16);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  hyc::rope_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(k), cos_sin, tokens, seq, heads_q, heads_k, head_dim,
      inverse ? -1.f : 1.f); HYC_LAUNCHED();
  return cudaGetLastError() == cudaSuccess ? HYC_OK : HYC_ERR_CUDA;
}
