// bf16-input instantiations of the register-resident forward kernel.
#include "hyc_fwd_fast.cuh"

namespace hyc {
int launch_fwd_fast_bf16(const FwdArgs& a, const LaunchPlan& plan, const FastPlan& f, bool norm, cudaStream_t stream) {
  return norm ? launch_fwd_fast<__nv_bfloat16, true>(a, plan, f, stream) : launch_fwd_fast<__nv_bfloat16, false>(a, plan, f, stream);
}
}  // namespace hyc
