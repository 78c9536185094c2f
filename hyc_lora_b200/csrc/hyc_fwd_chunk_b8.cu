// Chunk-per-lane rotating forward kernel, 8-bit codes: 4096 channels (128 per lane), 2048 (64) and 1024 (32).
#include <mutex>

#include "hyc_fwd_chunk.cuh"

namespace hyc {
int launch_fwd_chunk_b8(const ChunkFwdArgs& a, const ChunkPlan& w, bool norm, const CUtensorMap& in_map,
                        const CUtensorMap& y_map, cudaStream_t stream) {
  if (w.ch == 128) return launch_fwd_chunk_one<8, 128>(a, w, norm, in_map, y_map, stream);
  if (w.ch == 64) return launch_fwd_chunk_one<8, 64>(a, w, norm, in_map, y_map, stream);
  if (w.ch == 32) return launch_fwd_chunk_one<8, 32>(a, w, norm, in_map, y_map, stream);
  return HYC_ERR_SHAPE;
}

TensorMapEncodeFn tensor_map_encoder() {
  static TensorMapEncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<TensorMapEncodeFn>(ptr);
  });
  return fn;
}
}  // namespace hyc
