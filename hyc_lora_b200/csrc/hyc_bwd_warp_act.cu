// Warp-per-row activation backward (SiLU / GELU): instantiations and launcher.
#include "hyc_bwd_warp.cuh"

namespace hyc {
int launch_act_bwd_warp(const WarpBwdArgs& a, const WarpBwdPlan& w, bool gelu, cudaStream_t stream) {
  const bool ref = a.p.mode == HYC_MODE_R;
#define HYC_K(B, RF, GL)                                                                         \
  {                                                                                              \
    auto kern = act_bwd_n_warp_kernel<B, RF, GL>;                                                \
    int rc = set_smem(kern, w.total);                                                            \
    if (rc) return rc;                                                                           \
    kern<<<w.grid, w.threads, w.total, stream>>>(a); HYC_LAUNCHED();                             \
  }
#define HYC_L(B, NGV)                                                                            \
  {                                                                                              \
    if (ref) { if (gelu) HYC_K(B, true, true) else HYC_K(B, true, false) }                       \
    else { if (gelu) HYC_K(B, false, true) else HYC_K(B, false, false) }                         \
  }
  HYC_WARP_BWD_DISPATCH(a.p.bits, w.ng, HYC_L)
#undef HYC_L
#undef HYC_K
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? HYC_OK : cuda_fail(e, "act_bwd_n_warp_kernel launch");
}
}  // namespace hyc
