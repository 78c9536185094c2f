// f32-input instantiations of the register-resident forward kernel.
#include "hyc_fwd_fast.cuh"

namespace hyc {
int launch_fwd_fast_f32(const FwdArgs& a, const LaunchPlan& plan, const FastPlan& f, bool norm, cudaStream_t stream) {
  return norm ? launch_fwd_fast<float, true>(a, plan, f, stream) : launch_fwd_fast<float, false>(a, plan, f, stream);
}
}  // namespace hyc
