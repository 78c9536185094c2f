// Compress-only and fused norm + compress: kernel and launcher, instantiated per
// input dtype in hyc_fwd_bf16.cu / hyc_fwd_f32.cu.
#pragma once
#include "hyc_host.cuh"

namespace hyc {

// ------------------------------------------------------------------ forward: (norm +) compress

struct FwdArgs {
  PackedDev p;
  const unsigned char* x;
  long long row_stride, batch_stride, chunk_stride;  // elements
  int chunks;
  int kind;
  float eps;
  const void* weight;
  const void* bias;
  int param_bf16;
  void* y;
  float* rstd;
  float* mean;
  SmemLayout L;
};

template <typename XT>
__device__ __forceinline__ void issue_x_row(const FwdArgs& a, RowRing& ring, int stage, long long row) {
  const int D = a.p.cols;
  uint64_t* bar = &ring.bars[stage];
  XT* dst = reinterpret_cast<XT*>(ring.slot(stage));
  const XT* base = reinterpret_cast<const XT*>(a.x);
  mbar_expect_tx(bar, static_cast<uint32_t>(D * sizeof(XT)));
  if (a.chunks == 1) {
    bulk_g2s(dst, base + row * a.row_stride, static_cast<uint32_t>(D * sizeof(XT)), bar);
  } else {
    const long long b = row / a.p.seq, s = row % a.p.seq;
    const int clen = D / a.chunks;
    const XT* src = base + b * a.batch_stride + s * a.row_stride;
    for (int c = 0; c < a.chunks; ++c)
      bulk_g2s(dst + c * clen, src + c * a.chunk_stride, static_cast<uint32_t>(clen * sizeof(XT)), bar);
  }
}

template <typename PT>
__device__ __forceinline__ void norm_apply8(const float (&x)[8], const PT* weight, const PT* bias, int col, float mean,
                                            float rstd, bool gemma, float (&y)[8]) {
  float wv[8];
  load8<PT>(weight, col, wv);
  if (bias) {
    float bv[8];
    load8<PT>(bias, col, bv);
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = (x[e] - mean) * rstd * wv[e] + bv[e];
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) y[e] = (x[e] - mean) * rstd * (gemma ? wv[e] + 1.f : wv[e]);
  }
}

template <typename XT, int MODE, int BITS, bool NORM>
__global__ void __launch_bounds__(256) fwd_kernel(const __grid_constant__ FwdArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  const int D = p.cols;
  const int nvec = D >> 3;
  RowRing ring{reinterpret_cast<uint64_t*>(smem), smem + a.L.off_slots, a.L.slot_bytes, a.L.stages};
  ring.init();
  const Work w = make_work(smem, a.L);
  setup_packed(p, w);
  float thr = 0.f;
  if (MODE == kModeR) {
    thr = *p.thr;
    if (sizeof(XT) == 2) thr = bf16_round(thr);
  }
  const long long rows = p.rows, stride = gridDim.x;
  long long row = blockIdx.x;
  if (threadIdx.x == 0) {
    for (int s = 0; s < ring.stages; ++s) {
      const long long r = row + s * stride;
      if (r < rows) issue_x_row<XT>(a, ring, s, r);
    }
  }
  for (int i = 0; row < rows; ++i, row += stride) {
    const int st = i % ring.stages;
    if (!mbar_wait_bounded(&ring.bars[st], (i / ring.stages) & 1)) w.misc[2] = 1;
    const XT* xs = reinterpret_cast<const XT*>(ring.slot(st));
    if (NORM) {
      float mean = 0.f;
      if (a.kind == HYC_NORM_LAYER) {
        float s[1] = {0.f};
        for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
          float f[8];
          load8<XT>(xs, v << 3, f);
#pragma unroll
          for (int e = 0; e < 8; ++e) s[0] += f[e];
        }
        block_reduce<1>(s, w.red + 128, OpSum());
        mean = s[0] / static_cast<float>(D);
      }
      float ss[1] = {0.f};
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        float f[8];
        load8<XT>(xs, v << 3, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) { const float c = f[e] - mean; ss[0] = fmaf(c, c, ss[0]); }
      }
      block_reduce<1>(ss, w.red + 192, OpSum());
      const float rstd = 1.0f / sqrtf(ss[0] / static_cast<float>(D) + a.eps);
      if (threadIdx.x == 0) {
        a.rstd[row] = rstd;
        if (a.kind == HYC_NORM_LAYER) a.mean[row] = mean;
      }
      XT* yrow = reinterpret_cast<XT*>(a.y) + row * a.row_stride;
      const bool gemma = a.kind == HYC_NORM_RMS_GEMMA;
      const void* bias = a.kind == HYC_NORM_LAYER ? a.bias : nullptr;
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        float f[8], y[8];
        load8<XT>(xs, v << 3, f);
        if (a.param_bf16)
          norm_apply8<__nv_bfloat16>(f, static_cast<const __nv_bfloat16*>(a.weight),
                                     static_cast<const __nv_bfloat16*>(bias), v << 3, mean, rstd, gemma, y);
        else
          norm_apply8<float>(f, static_cast<const float*>(a.weight), static_cast<const float*>(bias), v << 3, mean,
                             rstd, gemma, y);
        store8<XT>(yrow, v << 3, y);
      }
    }
    if (MODE == kModeN) n_compress_row<XT, BITS>(p, w, xs, row);
    else r_compress_row<XT, BITS>(p, w, xs, row, thr);
    __syncthreads();  // every read of this slot is done
    if (w.misc[2]) {
      if (threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusWaitExpired);
      drain_ring(ring, i, row + stride, rows, stride);
      return;
    }
    if (threadIdx.x == 0) {
      const long long next = row + ring.stages * stride;
      if (next < rows) {
        fence_proxy_async();
        issue_x_row<XT>(a, ring, st, next);
      }
    }
  }
}

template <typename XT, bool NORM>
static int launch_fwd(const FwdArgs& a, const LaunchPlan& plan, cudaStream_t stream) {
#define HYC_FWD_CASE(MODE, BITS)                                                                     \
  {                                                                                                  \
    auto kern = fwd_kernel<XT, MODE, BITS, NORM>;                                                    \
    int rc = set_smem(kern, plan.L.total);                                                           \
    if (rc) return rc;                                                                               \
    kern<<<plan.grid, plan.threads, plan.L.total, stream>>>(a); HYC_LAUNCHED();                                      \
    break;                                                                                           \
  }
  if (a.p.mode == kModeN) {
    switch (a.p.bits) {
      case 2: HYC_FWD_CASE(kModeN, 2)
      case 4: HYC_FWD_CASE(kModeN, 4)
      default: HYC_FWD_CASE(kModeN, 8)
    }
  } else {
    switch (a.p.bits) {
      case 1: HYC_FWD_CASE(kModeR, 1)
      case 2: HYC_FWD_CASE(kModeR, 2)
      case 4: HYC_FWD_CASE(kModeR, 4)
      default: HYC_FWD_CASE(kModeR, 8)
    }
  }
#undef HYC_FWD_CASE
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? HYC_OK : cuda_fail(e, "fwd_kernel launch");
}

// defined once per input dtype (hyc_fwd_bf16.cu, hyc_fwd_f32.cu)
int launch_fwd_bf16(const FwdArgs& a, const LaunchPlan& plan, bool norm, cudaStream_t stream);
int launch_fwd_f32(const FwdArgs& a, const LaunchPlan& plan, bool norm, cudaStream_t stream);

}  // namespace hyc
