// Chunk-per-lane rotating forward kernel, 2-bit codes: 4096 channels (32 per lane and segment).
#include "hyc_fwd_chunk.cuh"

namespace hyc {
int launch_fwd_chunk_b2(const ChunkFwdArgs& a, const ChunkPlan& w, bool norm, const CUtensorMap& in_map,
                        const CUtensorMap& y_map, cudaStream_t stream) {
  if (w.ch == 32) return launch_fwd_chunk_one<2, 32>(a, w, norm, in_map, y_map, stream);
  return HYC_ERR_SHAPE;
}
}  // namespace hyc
