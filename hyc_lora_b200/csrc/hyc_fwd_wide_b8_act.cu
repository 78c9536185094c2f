// Wide-row forward kernel, 8-bit codes: SiLU / GELU + compress.
#include "hyc_fwd_wide.cuh"

namespace hyc {
int launch_wide_b8_act(const WideArgs& a, const WidePlan& w, int op, const CUtensorMap& m0, const CUtensorMap& m1,
                        const CUtensorMap& m2, cudaStream_t s) {
  return op == kWideGelu ? launch_wide_op<8, kWideGelu>(a, w, m0, m1, m2, s)
                         : launch_wide_op<8, kWideSilu>(a, w, m0, m1, m2, s);
}
}  // namespace hyc
