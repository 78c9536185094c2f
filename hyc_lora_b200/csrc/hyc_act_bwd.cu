// Decompress + SiLU / GELU(tanh) / product backward.
#include "hyc_bwd_fast.cuh"
#include "hyc_bwd_warp.cuh"

namespace hyc {

// ------------------------------------------------------------------ decompress + activation backward

struct ActBwdArgs {
  PackedDev p1, p2;
  int op;
  const unsigned char* g;
  unsigned char* dx1;
  unsigned char* dx2;
  SmemLayout L;
};

__device__ __forceinline__ float silu_grad(float x) {
  const float s = __fdividef(1.f, 1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float gamma = 0.7978845608028654f, kappa = 0.044715f;
  const float y = gamma * (x + kappa * x * x * x);
  const float t = 1.f - __fdividef(2.f, 1.f + __expf(2.f * y));  // tanh(y)
  return 0.5f * ((1.f + t) + x * ((1.f - t * t) * gamma * (1.f + 3.f * kappa * x * x)));
}

template <int MODE, int BITS, typename GT, int OP>
__global__ void __launch_bounds__(256) act_bwd_kernel(const __grid_constant__ ActBwdArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p1;
  const int D = p.cols;
  const int nvec = D >> 3;
  const uint32_t cb = static_cast<uint32_t>(D) * BITS / 8;
  const uint32_t gb = static_cast<uint32_t>(D) * sizeof(GT);
  const uint32_t off_c2 = (cb + 127u) & ~127u;
  const uint32_t off_g = OP == HYC_ACT_PRODUCT ? 2 * off_c2 : off_c2;
  RowRing ring{reinterpret_cast<uint64_t*>(smem), smem + a.L.off_slots, a.L.slot_bytes, a.L.stages};
  ring.init();
  const Work w = make_work(smem, a.L);
  Work w2 = w;
  setup_packed(p, w);
  if (OP == HYC_ACT_PRODUCT) {
    w2.omask = reinterpret_cast<uint32_t*>(smem + a.L.off_omask2);
    w2.chan = reinterpret_cast<int*>(smem + a.L.off_chan2);
    w2.cscale = reinterpret_cast<float*>(smem + a.L.off_cscale2);
    w2.xr = reinterpret_cast<__nv_bfloat16*>(smem + a.L.off_xr2);
    setup_packed(a.p2, w2);
  }
  const long long rows = p.rows, stride = gridDim.x;
  long long row = blockIdx.x;
  auto issue = [&](int s, long long r) {
    mbar_expect_tx(&ring.bars[s], (OP == HYC_ACT_PRODUCT ? 2 * cb : cb) + gb);
    issue_bytes(ring, s, 0, p.codes + r * cb, cb);
    if (OP == HYC_ACT_PRODUCT) issue_bytes(ring, s, off_c2, a.p2.codes + r * cb, cb);
    issue_bytes(ring, s, off_g, a.g + r * gb, gb);
  };
  if (threadIdx.x == 0)
    for (int s = 0; s < ring.stages; ++s)
      if (row + s * stride < rows) issue(s, row + s * stride);
  for (int i = 0; row < rows; ++i, row += stride) {
    const int st = i % ring.stages;
    if (!mbar_wait_bounded(&ring.bars[st], (i / ring.stages) & 1)) w.misc[2] = 1;
    dequant_row<MODE, BITS>(p, w, ring.slot(st), row);
    if (OP == HYC_ACT_PRODUCT) dequant_row<MODE, BITS>(a.p2, w2, ring.slot(st) + off_c2, row);
    const GT* gs = reinterpret_cast<const GT*>(ring.slot(st) + off_g);
    GT* d1 = reinterpret_cast<GT*>(a.dx1) + row * static_cast<long long>(D);
    GT* d2 = reinterpret_cast<GT*>(a.dx2) + row * static_cast<long long>(D);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float x[8], g[8], o[8];
      load8<__nv_bfloat16>(w.xr, v << 3, x);
      load8<GT>(gs, v << 3, g);
      if (OP == HYC_ACT_PRODUCT) {
        float x2[8], o2[8];
        load8<__nv_bfloat16>(w2.xr, v << 3, x2);
#pragma unroll
        for (int e = 0; e < 8; ++e) { o[e] = g[e] * x2[e]; o2[e] = x[e] * g[e]; }
        store8<GT>(d2, v << 3, o2);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = (OP == HYC_ACT_SILU ? silu_grad(x[e]) : gelu_tanh_grad(x[e])) * g[e];
      }
      store8<GT>(d1, v << 3, o);
    }
    __syncthreads();
    if (w.misc[2]) {
      if (threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusWaitExpired);
      drain_ring(ring, i, row + stride, rows, stride);
      return;
    }
    if (threadIdx.x == 0) {
      const long long next = row + ring.stages * stride;
      if (next < rows) { fence_proxy_async(); issue(st, next); }
    }
  }
}

}  // namespace hyc

using namespace hyc;

extern "C" {

int hyc_act_bwd(int op, const hyc_packed* s1, const hyc_packed* s2, const void* g, int g_dtype, void* dx1, void* dx2,
                void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (op < HYC_ACT_SILU || op > HYC_ACT_PRODUCT) return HYC_ERR_MODE;
  const int empty = packed_is_empty(s1);
  if (empty) return empty < 0 ? empty : HYC_OK;
  int rc = check_packed(s1, false);
  if (rc) return rc;
  if (!g || !dx1) return HYC_ERR_NULL;
  if (g_dtype != HYC_F32 && g_dtype != HYC_BF16) return HYC_ERR_DTYPE;
  if (!aligned16(g) || !aligned16(dx1)) return HYC_ERR_ALIGN;
  const bool prod = op == HYC_ACT_PRODUCT;
  if (prod) {
    rc = check_packed(s2, false);
    if (rc) return rc;
    if (!dx2) return HYC_ERR_NULL;
    if (!aligned16(dx2)) return HYC_ERR_ALIGN;
    if (s2->rows != s1->rows || s2->cols != s1->cols || s2->mode != s1->mode || s2->bits != s1->bits ||
        s2->rotate != s1->rotate || s2->group != s1->group)
      return HYC_ERR_SHAPE;
  }
  if (s1->rows == 0) return HYC_OK;
  const int D = s1->cols;
  if (!prod && g_dtype == HYC_BF16 && !s1->rotate) {
    // SiLU / GELU, bf16 gradient, rows of up to 4096 channels without rotation: one warp per row
    WarpBwdPlan wp = plan_warp_bwd(s1, nullptr, true, false, kNormBwdWarpThreads, 1);
    if (!wp.ok) wp = plan_warp_bwd(s1, nullptr, true, false, 512, 1);
    if (!wp.ok) wp = plan_warp_bwd(s1, nullptr, true, false, 384, 1);
    if (wp.ok) {
      WarpBwdArgs wa;
      fill_warp_bwd(&wa, wp, s1, nullptr);
      wa.g = static_cast<const __nv_bfloat16*>(g);
      wa.out1 = static_cast<__nv_bfloat16*>(dx1);
      return launch_act_bwd_warp(wa, wp, op == HYC_ACT_GELU_TANH, stream);
    }
  }
  {
    const BwdPlan bp = plan_bwd_fast(s1, prod ? s2 : nullptr, 4, false, 0, 512, 0,
                                     align_up(static_cast<uint32_t>(D) * s1->bits / 8, 128) * (prod ? 2 : 1) +
                                         static_cast<uint32_t>(D) * (g_dtype == HYC_BF16 ? 2 : 4),
                                     256, 2);
    if (bp.ok) {
      ActFastArgs fa;
      memset(&fa, 0, sizeof(fa));
      fa.p1 = to_dev(s1);
      if (prod) fa.p2 = to_dev(s2);
      fa.g = static_cast<const unsigned char*>(g);
      fa.dx1 = static_cast<unsigned char*>(dx1);
      fa.dx2 = static_cast<unsigned char*>(dx2);
      fa.L = bp.L;
      // These CTAs set up no tables, and on long inputs four short waves measured 5 % faster than one
      // persistent wave (65 536 rows of 4096 channels: 0.234 against 0.246 ms); each CTA keeps 8 rows or more.
      const int grid_l = (!g_tune_ctas && s1->rows >= 32LL * bp.grid) ? bp.grid * 4 : bp.grid;
#define HYC_ACTF_OP(B, UP, RT, GT, OPV)                                                         \
  {                                                                                             \
    auto kern = act_bwd_n_fast_kernel<B, UP, RT, GT, OPV>;                                      \
    rc = set_smem(kern, bp.L.total);                                                            \
    if (rc) return rc;                                                                          \
    kern<<<grid_l, bp.threads, bp.L.total, stream>>>(fa); HYC_LAUNCHED();                                       \
  }
#define HYC_ACTF(B, UP, RT)                                                                     \
  {                                                                                             \
    if (g_dtype == HYC_BF16) {                                                                  \
      if (op == HYC_ACT_SILU) HYC_ACTF_OP(B, UP, RT, __nv_bfloat16, HYC_ACT_SILU)               \
      else if (op == HYC_ACT_GELU_TANH) HYC_ACTF_OP(B, UP, RT, __nv_bfloat16, HYC_ACT_GELU_TANH) \
      else HYC_ACTF_OP(B, UP, RT, __nv_bfloat16, HYC_ACT_PRODUCT)                               \
    } else {                                                                                    \
      if (op == HYC_ACT_SILU) HYC_ACTF_OP(B, UP, RT, float, HYC_ACT_SILU)                       \
      else if (op == HYC_ACT_GELU_TANH) HYC_ACTF_OP(B, UP, RT, float, HYC_ACT_GELU_TANH)        \
      else HYC_ACTF_OP(B, UP, RT, float, HYC_ACT_PRODUCT)                                       \
    }                                                                                           \
  }
      HYC_BWD_DISPATCH(bp, s1->bits, 4, HYC_ACTF)
#undef HYC_ACTF
#undef HYC_ACTF_OP
      cudaError_t e = cudaGetLastError();
      return e == cudaSuccess ? HYC_OK : cuda_fail(e, "act_bwd_n_fast_kernel launch");
    }
  }
  const uint32_t cb = static_cast<uint32_t>(D) * s1->bits / 8;
  LayoutReq req;
  fill_req_packed(&req, s1, false);
  req.xr = true;
  if (prod) {
    req.second = true;
    req.nmode2 = s2->mode == HYC_MODE_N;
    req.k2 = s2->n_channels;
    req.cscale2 = s2->mode == HYC_MODE_R && s2->scale_kind == HYC_SCALE_CHANNEL;
  }
  req.slot_bytes = align_up(cb, 128) * (prod ? 2 : 1) + static_cast<uint32_t>(D) * (g_dtype == HYC_BF16 ? 2 : 4);
  LaunchPlan plan;
  rc = plan_launch(req, s1->rows, &plan);
  if (rc) return rc;
  ActBwdArgs a;
  memset(&a, 0, sizeof(a));
  a.p1 = to_dev(s1);
  if (prod) a.p2 = to_dev(s2);
  a.op = op;
  a.g = static_cast<const unsigned char*>(g);
  a.dx1 = static_cast<unsigned char*>(dx1);
  a.dx2 = static_cast<unsigned char*>(dx2);
  a.L = plan.L;
#define HYC_ACT_LAUNCH(MODE, BITS, GT, OP)                                  \
  {                                                                         \
    auto kern = act_bwd_kernel<MODE, BITS, GT, OP>;                         \
    rc = set_smem(kern, plan.L.total);                                      \
    if (rc) return rc;                                                      \
    kern<<<plan.grid, plan.threads, plan.L.total, stream>>>(a); HYC_LAUNCHED();             \
  }
#define HYC_ACT_CASE(MODE, BITS)                                            \
  {                                                                         \
    if (g_dtype == HYC_BF16) {                                              \
      if (op == HYC_ACT_SILU) HYC_ACT_LAUNCH(MODE, BITS, __nv_bfloat16, HYC_ACT_SILU)            \
      else if (op == HYC_ACT_GELU_TANH) HYC_ACT_LAUNCH(MODE, BITS, __nv_bfloat16, HYC_ACT_GELU_TANH) \
      else HYC_ACT_LAUNCH(MODE, BITS, __nv_bfloat16, HYC_ACT_PRODUCT)       \
    } else {                                                                \
      if (op == HYC_ACT_SILU) HYC_ACT_LAUNCH(MODE, BITS, float, HYC_ACT_SILU)                    \
      else if (op == HYC_ACT_GELU_TANH) HYC_ACT_LAUNCH(MODE, BITS, float, HYC_ACT_GELU_TANH)     \
      else HYC_ACT_LAUNCH(MODE, BITS, float, HYC_ACT_PRODUCT)               \
    }                                                                       \
  }
  HYC_DISPATCH_MODE_BITS(a.p1.mode, a.p1.bits, HYC_ACT_CASE)
#undef HYC_ACT_CASE
#undef HYC_ACT_LAUNCH
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? HYC_OK : cuda_fail(e, "act_bwd_kernel launch");
}

}  // extern "C"
