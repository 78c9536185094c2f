// Warp-per-row reference-mode forward kernel: instantiations and launcher.
#include "hyc_fwd_r_warp.cuh"

namespace hyc {
int launch_fwd_r_warp(const RWarpArgs& a, const RWarpPlan& w, bool norm, cudaStream_t stream) {
  const int nk = !norm ? 0 : a.kind == HYC_NORM_LAYER ? 2 : 1;
#define HYC_K(B, NKV)                                                          \
  {                                                                            \
    auto kern = fwd_r_warp_kernel<B, NKV>;                                     \
    int rc = set_smem(kern, w.total);                                          \
    if (rc) return rc;                                                         \
    kern<<<w.grid, w.threads, w.total, stream>>>(a); HYC_LAUNCHED();           \
  }
#define HYC_B(B)                                                               \
  {                                                                            \
    if (nk == 2) HYC_K(B, 2) else if (nk == 1) HYC_K(B, 1) else HYC_K(B, 0)    \
  }
  if (a.p.bits == 2) HYC_B(2) else if (a.p.bits == 4) HYC_B(4) else HYC_B(8)
#undef HYC_B
#undef HYC_K
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? HYC_OK : cuda_fail(e, "fwd_r_warp_kernel launch");
}
}  // namespace hyc
