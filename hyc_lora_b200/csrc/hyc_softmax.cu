// Sparse copy of attention probabilities: keep the entries above a threshold as a compact
// per-row list (no host synchronisation), expand it back to a dense tensor, and the softmax
// backward evaluated from the list.  One warp per row; rows are short (the sequence length).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hyc_b200.h"
#include "hyc_common.cuh"

namespace hyc {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T of_f(float v);
template <> __device__ __forceinline__ float of_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 of_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Entries of a row are written in ascending column order: ballot + popcount give every kept
// element its place; one atomic per row reserves the row's range in the pool.
template <typename T>
__global__ void softmax_compact_kernel(const T* p, long long rows, int cols, const float* thr_ptr, T* val,
                                       uint16_t* col, uint32_t cap, uint32_t* used, uint2* row_meta,
                                       uint32_t* status) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  float thr = *thr_ptr;
  if (sizeof(T) == 2) thr = bf16_round(thr);  // the compare runs in the tensor's dtype
  for (long long row = warp; row < rows; row += nwarps) {
    const T* prow = p + row * cols;
    uint32_t cnt = 0;
    for (int c0 = 0; c0 < cols; c0 += 32) {
      const int c = c0 + lane;
      const bool keep = c < cols && to_f<T>(prow[c]) > thr;
      cnt += __popc(__ballot_sync(0xffffffffu, keep));
    }
    uint32_t base = 0;
    if (lane == 0 && cnt > 0) {
      base = atomicAdd(used, cnt);
      if (base > cap || cnt > cap - base) {
        cnt = 0;
        if (status) atomicOr(status, kStatusPoolOverflow);
      }
    }
    base = __shfl_sync(0xffffffffu, base, 0);
    cnt = __shfl_sync(0xffffffffu, cnt, 0);
    if (lane == 0) row_meta[row] = make_uint2(base, cnt);
    if (cnt == 0) continue;
    uint32_t at = base;
    for (int c0 = 0; c0 < cols; c0 += 32) {
      const int c = c0 + lane;
      const T v = c < cols ? prow[c] : of_f<T>(0.f);
      const bool keep = c < cols && to_f<T>(v) > thr;
      const uint32_t m = __ballot_sync(0xffffffffu, keep);
      if (keep) {
        const uint32_t k = at + __popc(m & ((1u << lane) - 1u));
        val[k] = v;
        col[k] = static_cast<uint16_t>(c);
      }
      at += __popc(m);
    }
  }
}

template <typename T>
__global__ void softmax_expand_kernel(const T* val, const uint16_t* col, const uint2* row_meta, long long rows,
                                      int cols, T* dense) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long row = warp; row < rows; row += nwarps) {
    T* drow = dense + row * cols;
    for (int c = lane; c < cols; c += 32) drow[c] = of_f<T>(0.f);
    __syncwarp();
    const uint2 meta = row_meta[row];
    for (uint32_t j = lane; j < meta.y; j += 32) drow[col[meta.x + j]] = val[meta.x + j];
  }
}

// dx = (g - sum_j g_j y_j) * y  with y zero outside the kept entries
template <typename T, typename GT, typename OT>
__global__ void softmax_bwd_kernel(const T* val, const uint16_t* col, const uint2* row_meta, long long rows, int cols,
                                   const GT* g, OT* dx) {
  const int lane = threadIdx.x & 31;
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  for (long long row = warp; row < rows; row += nwarps) {
    const GT* grow = g + row * cols;
    OT* drow = dx + row * cols;
    const uint2 meta = row_meta[row];
    float s = 0.f;
    for (uint32_t j = lane; j < meta.y; j += 32) s += to_f<GT>(grow[col[meta.x + j]]) * to_f<T>(val[meta.x + j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    for (int c = lane; c < cols; c += 32) drow[c] = of_f<OT>(0.f);
    __syncwarp();
    for (uint32_t j = lane; j < meta.y; j += 32) {
      const int c = col[meta.x + j];
      drow[c] = of_f<OT>((to_f<GT>(grow[c]) - s) * to_f<T>(val[meta.x + j]));
    }
  }
}

static int check_sparse(const hyc_sparse_rows* s) {
  if (!s || !s->val || !s->col || !s->used || !s->row_meta) return HYC_ERR_NULL;
  if (s->rows < 0 || s->cols <= 0 || s->cols > 65535) return HYC_ERR_SHAPE;
  if (s->dtype != HYC_F32 && s->dtype != HYC_BF16) return HYC_ERR_DTYPE;
  return HYC_OK;
}

static int grid_for(long long rows) {
  long long blocks = (rows + 7) / 8;  // 8 warps per block
  if (blocks > 148 * 16) blocks = 148 * 16;
  return static_cast<int>(blocks < 1 ? 1 : blocks);
}

}  // namespace hyc

using namespace hyc;

extern "C" {

int hyc_softmax_compact(const void* p, const float* thr, const hyc_sparse_rows* out, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int rc = check_sparse(out);
  if (rc) return rc;
  if (!p || !thr) return HYC_ERR_NULL;
  if (cudaMemsetAsync(out->used, 0, sizeof(uint32_t), stream) != cudaSuccess) return HYC_ERR_CUDA;
  if (out->rows == 0) return HYC_OK;
  uint2* meta = reinterpret_cast<uint2*>(out->row_meta);
  if (out->dtype == HYC_F32)
    softmax_compact_kernel<float><<<grid_for(out->rows), 256, 0, stream>>>(
        static_cast<const float*>(p), out->rows, out->cols, thr, static_cast<float*>(out->val), out->col, out->cap,
        out->used, meta, out->status);
  else
    softmax_compact_kernel<__nv_bfloat16><<<grid_for(out->rows), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(p), out->rows, out->cols, thr, static_cast<__nv_bfloat16*>(out->val),
        out->col, out->cap, out->used, meta, out->status);
  HYC_LAUNCHED();
  return cudaGetLastError() == cudaSuccess ? HYC_OK : HYC_ERR_CUDA;
}

int hyc_softmax_expand(const hyc_sparse_rows* in, void* dense, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int rc = check_sparse(in);
  if (rc) return rc;
  if (!dense) return HYC_ERR_NULL;
  if (in->rows == 0) return HYC_OK;
  const uint2* meta = reinterpret_cast<const uint2*>(in->row_meta);
  if (in->dtype == HYC_F32)
    softmax_expand_kernel<float><<<grid_for(in->rows), 256, 0, stream>>>(
        static_cast<const float*>(in->val), in->col, meta, in->rows, in->cols, static_cast<float*>(dense));
  else
    softmax_expand_kernel<__nv_bfloat16><<<grid_for(in->rows), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(in->val), in->col, meta, in->rows, in->cols,
        static_cast<__nv_bfloat16*>(dense));
  HYC_LAUNCHED();
  return cudaGetLastError() == cudaSuccess ? HYC_OK : HYC_ERR_CUDA;
}

int hyc_softmax_bwd(const hyc_sparse_rows* in, const void* g, int g_dtype, void* dx, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int rc = check_sparse(in);
  if (rc) return rc;
  if (!g || !dx) return HYC_ERR_NULL;
  if (g_dtype != HYC_F32 && g_dtype != HYC_BF16) return HYC_ERR_DTYPE;
  if (in->rows == 0) return HYC_OK;
  const uint2* meta = reinterpret_cast<const uint2*>(in->row_meta);
  const int grid = grid_for(in->rows);
#define HYC_SM_BWD(T, GT, OT)                                                                              \
  softmax_bwd_kernel<T, GT, OT><<<grid, 256, 0, stream>>>(static_cast<const T*>(in->val), in->col, meta,   \
                                                          in->rows, in->cols, static_cast<const GT*>(g),   \
                                                          static_cast<OT*>(dx))
  // the result has the promoted dtype of the probabilities and the gradient
  if (in->dtype == HYC_F32 && g_dtype == HYC_F32) HYC_SM_BWD(float, float, float);
  else if (in->dtype == HYC_F32) HYC_SM_BWD(float, __nv_bfloat16, float);
  else if (g_dtype == HYC_F32) HYC_SM_BWD(__nv_bfloat16, float, float);
  else HYC_SM_BWD(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
#undef HYC_SM_BWD
  HYC_LAUNCHED();
  return cudaGetLastError() == cudaSuccess ? HYC_OK : HYC_ERR_CUDA;
}

}  // extern "C"
