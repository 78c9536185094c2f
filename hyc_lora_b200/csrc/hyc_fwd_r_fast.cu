// Instantiations of the reference-mode fast forward kernel.
#include "hyc_fwd_r_fast.cuh"

namespace hyc {

int launch_fwd_r_fast_bf16(const RFastArgs& a, const RFastPlan& f, bool norm, cudaStream_t stream) {
  return norm ? launch_fwd_r_fast<__nv_bfloat16, true>(a, f, stream) : launch_fwd_r_fast<__nv_bfloat16, false>(a, f, stream);
}

int launch_fwd_r_fast_f32(const RFastArgs& a, const RFastPlan& f, bool norm, cudaStream_t stream) {
  return norm ? launch_fwd_r_fast<float, true>(a, f, stream) : launch_fwd_r_fast<float, false>(a, f, stream);
}

}  // namespace hyc
