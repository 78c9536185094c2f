// Warp-per-row forward kernel, 2-bit codes (one translation unit per bit width so they compile in parallel).
#include "hyc_fwd_warp.cuh"

namespace hyc {
int launch_fwd_warp_b2(const WarpFwdArgs& a, const WarpPlan& w, bool norm, cudaStream_t stream) {
  return launch_fwd_warp_bits<2>(a, w, norm, stream);
}
}  // namespace hyc
