// Chunk-per-lane rotating forward kernel, 4-bit codes (one translation unit per bit width so they compile in
// parallel): 4096 channels (64 per lane and segment) and 2048 channels (32).
#include "hyc_fwd_chunk.cuh"

namespace hyc {
int launch_fwd_chunk_b4(const ChunkFwdArgs& a, const ChunkPlan& w, bool norm, const CUtensorMap& in_map,
                        const CUtensorMap& y_map, cudaStream_t stream) {
  if (w.ch == 64) return launch_fwd_chunk_one<4, 64>(a, w, norm, in_map, y_map, stream);
  if (w.ch == 32) return launch_fwd_chunk_one<4, 32>(a, w, norm, in_map, y_map, stream);
  return HYC_ERR_SHAPE;
}
}  // namespace hyc
