// Warp-per-row norm backward: instantiations and launcher.
#include "hyc_bwd_warp.cuh"

namespace hyc {
int launch_norm_bwd_warp(const WarpBwdArgs& a, const WarpBwdPlan& w, cudaStream_t stream) {
  const bool ref = a.p.mode == HYC_MODE_R;
  const bool ln = a.kind == HYC_NORM_LAYER;
#define HYC_K(B, NGV, RT, LNV)                                                                   \
  {                                                                                              \
    auto kern = norm_bwd_n_warp_kernel<B, RT, LNV>;                                              \
    int rc = set_smem(kern, w.total);                                                            \
    if (rc) return rc;                                                                           \
    kern<<<w.grid, w.threads, w.total, stream>>>(a); HYC_LAUNCHED();                    \
  }
#define HYC_L(B, NGV)                                                                            \
  {                                                                                              \
    if (ref) { if (ln) HYC_K(B, NGV, true, true) else HYC_K(B, NGV, true, false) }               \
    else { if (ln) HYC_K(B, NGV, false, true) else HYC_K(B, NGV, false, false) }                 \
  }
  HYC_WARP_BWD_DISPATCH(a.p.bits, w.ng, HYC_L)
#undef HYC_L
#undef HYC_K
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? HYC_OK : cuda_fail(e, "norm_bwd_n_warp_kernel launch");
}
}  // namespace hyc
