// Warp-per-row decompress: instantiations and launcher.
#include "hyc_bwd_warp.cuh"

namespace hyc {
int launch_decompress_warp(const WarpBwdArgs& a, const WarpBwdPlan& w, cudaStream_t stream) {
  const bool rot = a.p.rotate != 0, ref = a.p.mode == HYC_MODE_R;
#define HYC_L(B, NGV)                                                                            \
  {                                                                                              \
    if (ref) {                                                                                   \
      auto kern = decompress_n_warp_kernel<B, NGV, 2>;                                           \
      int rc = set_smem(kern, w.total);                                                          \
      if (rc) return rc;                                                                         \
      kern<<<w.grid, w.threads, w.total, stream>>>(a); HYC_LAUNCHED();                  \
    } else if (rot) {                                                                            \
      auto kern = decompress_n_warp_kernel<B, NGV, 1>;                                           \
      int rc = set_smem(kern, w.total);                                                          \
      if (rc) return rc;                                                                         \
      kern<<<w.grid, w.threads, w.total, stream>>>(a); HYC_LAUNCHED();                  \
    } else {                                                                                     \
      auto kern = decompress_n_warp_kernel<B, NGV, 0>;                                           \
      int rc = set_smem(kern, w.total);                                                          \
      if (rc) return rc;                                                                         \
      kern<<<w.grid, w.threads, w.total, stream>>>(a); HYC_LAUNCHED();                  \
    }                                                                                            \
  }
  HYC_WARP_BWD_DISPATCH(a.p.bits, w.ng, HYC_L)
#undef HYC_L
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? HYC_OK : cuda_fail(e, "decompress_n_warp_kernel launch");
}
}  // namespace hyc
