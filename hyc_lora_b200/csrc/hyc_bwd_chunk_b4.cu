// Chunk-per-lane consumer kernels for rotated records (decompress, decompress + norm backward), 4-bit codes.
#include "hyc_bwd_chunk.cuh"

namespace hyc {
int launch_bwd_chunk_b4(const ChunkBwdArgs& a, const ChunkBwdPlan& w, int op, const CUtensorMap& dy_map,
                        const CUtensorMap& out_map, cudaStream_t stream) {
  if (w.ch == 64) return launch_bwd_chunk_one<4, 64>(a, w, op, dy_map, out_map, stream);
  if (w.ch == 32) return launch_bwd_chunk_one<4, 32>(a, w, op, dy_map, out_map, stream);
  return HYC_ERR_SHAPE;
}
}  // namespace hyc
