// Packed activation -> bf16 rows.
#include "hyc_bwd_warp.cuh"
#include "hyc_bwd_chunk.cuh"

namespace hyc {

// ------------------------------------------------------------------ decompress to bf16 rows

struct DecArgs {
  PackedDev p;
  __nv_bfloat16* out;
  long long row_stride, batch_stride, chunk_stride;
  int chunks;
  SmemLayout L;
};

template <int MODE, int BITS>
__global__ void __launch_bounds__(256) decompress_kernel(const __grid_constant__ DecArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  const int D = p.cols;
  const uint32_t cb = static_cast<uint32_t>(D) * BITS / 8;
  RowRing ring{reinterpret_cast<uint64_t*>(smem), smem + a.L.off_slots, a.L.slot_bytes, a.L.stages};
  ring.init();
  const Work w = make_work(smem, a.L);
  setup_packed(p, w);
  const long long rows = p.rows, stride = gridDim.x;
  long long row = blockIdx.x;
  auto issue = [&](int s, long long r) {
    mbar_expect_tx(&ring.bars[s], cb);
    issue_bytes(ring, s, 0, p.codes + r * cb, cb);
  };
  if (threadIdx.x == 0)
    for (int s = 0; s < ring.stages; ++s)
      if (row + s * stride < rows) issue(s, row + s * stride);
  for (int i = 0; row < rows; ++i, row += stride) {
    const int st = i % ring.stages;
    if (!mbar_wait_bounded(&ring.bars[st], (i / ring.stages) & 1)) w.misc[2] = 1;
    dequant_row<MODE, BITS>(p, w, ring.slot(st), row);
    __nv_bfloat16* orow;
    const int clen = D / a.chunks;
    if (a.chunks == 1) orow = a.out + row * a.row_stride;
    else orow = a.out + (row / p.seq) * a.batch_stride + (row % p.seq) * a.row_stride;
    for (int v = threadIdx.x; v < (D >> 3); v += blockDim.x) {
      const int col = v << 3;
      const uint4 val = *reinterpret_cast<const uint4*>(w.xr + col);
      const int c = col / clen;
      *reinterpret_cast<uint4*>(orow + c * a.chunk_stride + (col - c * clen)) = val;
    }
    __syncthreads();
    if (w.misc[2]) {
      if (threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusWaitExpired);
      drain_ring(ring, i, row + stride, rows, stride);
      return;
    }
    if (threadIdx.x == 0) {
      const long long next = row + ring.stages * stride;
      if (next < rows) { fence_proxy_async(); issue(st, next); }
    }
  }
}

}  // namespace hyc

using namespace hyc;

extern "C" {

int hyc_decompress(const hyc_packed* in, const hyc_dense* o, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int empty = packed_is_empty(in);
  if (empty) return empty < 0 ? empty : HYC_OK;
  int rc = check_packed(in, false);
  if (rc) return rc;
  rc = check_dense(o, in->cols, false);
  if (rc) return rc;
  if (o->dtype != HYC_BF16) return HYC_ERR_DTYPE;
  if (in->rows == 0) return HYC_OK;
  if (o->chunks == 1) {
    // rotated records whose segment is 32 chunks wide: one warp per row, a chunk of every segment per lane
    const ChunkBwdPlan cp = plan_chunk_bwd(in, false);
    if (cp.ok && (o->row_stride * 2) % 16 == 0) {
      const int rcb = run_chunk_bwd(in, cp, nullptr, o->base, o->row_stride, 0, nullptr, 0, nullptr, nullptr, 0, stream);
      if (rcb != HYC_ERR_SHAPE) return rcb;
    }
    // plain output rows of up to 4096 channels: one warp per row
    const WarpBwdPlan wp = plan_warp_bwd(in, nullptr, false, false);
    if (wp.ok) {
      WarpBwdArgs wa;
      fill_warp_bwd(&wa, wp, in, nullptr);
      wa.out1 = static_cast<__nv_bfloat16*>(o->base);
      wa.out_stride = o->row_stride;
      return launch_decompress_warp(wa, wp, stream);
    }
  }
  {
    // register-resident kernel for the channel-outlier mode
    const BwdPlan bp = plan_bwd_fast(in, nullptr, 4, false, 0, 512, 0, static_cast<uint32_t>(in->cols) * in->bits / 8, 0, 2);
    if (bp.ok) {
      DecFastArgs fa;
      memset(&fa, 0, sizeof(fa));
      fa.p = to_dev(in);
      fa.out = static_cast<__nv_bfloat16*>(o->base);
      fa.row_stride = o->row_stride; fa.batch_stride = o->batch_stride; fa.chunk_stride = o->chunk_stride;
      fa.chunks = o->chunks;
      fa.L = bp.L;
#define HYC_DECF(B, UP, RT)                                                                     \
  {                                                                                             \
    auto kern = decompress_n_fast_kernel<B, UP, RT>;                                            \
    rc = set_smem(kern, bp.L.total);                                                            \
    if (rc) return rc;                                                                          \
    const int g = bp.rot == 2 ? bp.grid : resident_grid(kern, bp.threads, bp.L.total, bp.grid);    \
    kern<<<g, bp.threads, bp.L.total, stream>>>(fa); HYC_LAUNCHED();                                            \
  }
      HYC_BWD_DISPATCH(bp, in->bits, 4, HYC_DECF)
#undef HYC_DECF
      cudaError_t e = cudaGetLastError();
      return e == cudaSuccess ? HYC_OK : cuda_fail(e, "decompress_n_fast_kernel launch");
    }
  }
  LayoutReq req;
  fill_req_packed(&req, in, false);
  req.xr = true;
  req.slot_bytes = static_cast<uint32_t>(in->cols) * in->bits / 8;
  LaunchPlan plan;
  rc = plan_launch(req, in->rows, &plan);
  if (rc) return rc;
  DecArgs a;
  memset(&a, 0, sizeof(a));
  a.p = to_dev(in);
  a.out = static_cast<__nv_bfloat16*>(o->base);
  a.row_stride = o->row_stride; a.batch_stride = o->batch_stride; a.chunk_stride = o->chunk_stride;
  a.chunks = o->chunks;
  a.L = plan.L;
#define HYC_DEC_CASE(MODE, BITS)                                            \
  {                                                                         \
    auto kern = decompress_kernel<MODE, BITS>;                              \
    rc = set_smem(kern, plan.L.total);                                      \
    if (rc) return rc;                                                      \
    kern<<<plan.grid, plan.threads, plan.L.total, stream>>>(a); HYC_LAUNCHED();             \
  }
  HYC_DISPATCH_MODE_BITS(a.p.mode, a.p.bits, HYC_DEC_CASE)
#undef HYC_DEC_CASE
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? HYC_OK : cuda_fail(e, "decompress_kernel launch");
}

}  // extern "C"
