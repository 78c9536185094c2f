// Chunk-per-lane consumer kernels for rotated records (decompress, decompress + norm backward), 8-bit codes.
#include "hyc_bwd_chunk.cuh"

namespace hyc {
int launch_bwd_chunk_b8(const ChunkBwdArgs& a, const ChunkBwdPlan& w, int op, const CUtensorMap& dy_map,
                        const CUtensorMap& out_map, cudaStream_t stream) {
  if (w.ch == 128) return launch_bwd_chunk_one<8, 128>(a, w, op, dy_map, out_map, stream);
  if (w.ch == 64) return launch_bwd_chunk_one<8, 64>(a, w, op, dy_map, out_map, stream);
  if (w.ch == 32) return launch_bwd_chunk_one<8, 32>(a, w, op, dy_map, out_map, stream);
  return HYC_ERR_SHAPE;
}
}  // namespace hyc
