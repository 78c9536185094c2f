// fp32-input instantiations of the compress / norm+compress kernel.
#include "hyc_fwd.cuh"

namespace hyc {
int launch_fwd_f32(const FwdArgs& a, const LaunchPlan& plan, bool norm, cudaStream_t stream) {
  return norm ? launch_fwd<float, true>(a, plan, stream) : launch_fwd<float, false>(a, plan, stream);
}
}  // namespace hyc
