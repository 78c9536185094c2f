// Wide-row forward kernel, 8-bit codes: compress-only and product + compress.
#include "hyc_fwd_wide.cuh"

namespace hyc {
int launch_wide_b8_cp(const WideArgs& a, const WidePlan& w, int op, const CUtensorMap& m0, const CUtensorMap& m1,
                       const CUtensorMap& m2, cudaStream_t s) {
  return op == kWideProduct ? launch_wide_op<8, kWideProduct>(a, w, m0, m1, m2, s)
                            : launch_wide_op<8, kWideCompress>(a, w, m0, m1, m2, s);
}
}  // namespace hyc
