// bf16-input instantiations of the compress / norm+compress kernel.
#include "hyc_fwd.cuh"

namespace hyc {
int launch_fwd_bf16(const FwdArgs& a, const LaunchPlan& plan, bool norm, cudaStream_t stream) {
  return norm ? launch_fwd<__nv_bfloat16, true>(a, plan, stream) : launch_fwd<__nv_bfloat16, false>(a, plan, stream);
}
}  // namespace hyc
