// Decompress + RMSNorm / LayerNorm backward, with the optional weight / bias gradient.
#include "hyc_bwd_warp.cuh"
#include "hyc_bwd_chunk.cuh"

namespace hyc {

// ------------------------------------------------------------------ decompress + norm backward

struct NormBwdArgs {
  PackedDev p;
  int kind, ref_compat_c2, param_bf16;
  const void* weight;
  const unsigned char* dy;
  const float* rstd;
  const float* mean;
  __nv_bfloat16* dx;
  float* partials;  // [gridDim][D] dw, then [gridDim][D] db
  int need_dw, need_db;
  SmemLayout L;
};

template <int MODE, int BITS, typename GT>
__global__ void __launch_bounds__(256) norm_bwd_kernel(const __grid_constant__ NormBwdArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  const PackedDev& p = a.p;
  const int D = p.cols;
  const int nvec = D >> 3;
  const uint32_t cb = static_cast<uint32_t>(D) * BITS / 8;
  const uint32_t gb = static_cast<uint32_t>(D) * sizeof(GT);
  const uint32_t off_g = (cb + 127u) & ~127u;
  RowRing ring{reinterpret_cast<uint64_t*>(smem), smem + a.L.off_slots, a.L.slot_bytes, a.L.stages};
  ring.init();
  const Work w = make_work(smem, a.L);
  setup_packed(p, w);
  float* acc_w = reinterpret_cast<float*>(smem + a.L.off_acc);
  float* acc_b = acc_w + D;
  if (a.need_dw) {
    for (int c = threadIdx.x; c < D * (a.need_db ? 2 : 1); c += blockDim.x) acc_w[c] = 0.f;
    __syncthreads();
  }
  const long long rows = p.rows, stride = gridDim.x;
  long long row = blockIdx.x;
  auto issue = [&](int s, long long r) {
    mbar_expect_tx(&ring.bars[s], cb + gb);
    issue_bytes(ring, s, 0, p.codes + r * cb, cb);
    issue_bytes(ring, s, off_g, a.dy + r * gb, gb);
  };
  if (threadIdx.x == 0)
    for (int s = 0; s < ring.stages; ++s)
      if (row + s * stride < rows) issue(s, row + s * stride);
  const bool ln = a.kind == HYC_NORM_LAYER;
  const bool gemma = a.kind == HYC_NORM_RMS_GEMMA;
  const float inv_d = 1.0f / static_cast<float>(D);
  for (int i = 0; row < rows; ++i, row += stride) {
    const int st = i % ring.stages;
    if (!mbar_wait_bounded(&ring.bars[st], (i / ring.stages) & 1)) w.misc[2] = 1;
    dequant_row<MODE, BITS>(p, w, ring.slot(st), row);
    const GT* gs = reinterpret_cast<const GT*>(ring.slot(st) + off_g);
    const float rstd = a.rstd[row];
    const float mean = ln ? a.mean[row] : 0.f;
    float c[2] = {0.f, 0.f};
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float x[8], g[8], wv[8];
      load8<__nv_bfloat16>(w.xr, v << 3, x);
      load8<GT>(gs, v << 3, g);
      if (a.param_bf16) load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(a.weight), v << 3, wv);
      else load8<float>(static_cast<const float*>(a.weight), v << 3, wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float gy = sizeof(GT) == 4 ? bf16_round(g[e]) : g[e];
        const float wdy = (gemma ? wv[e] + 1.f : wv[e]) * gy;
        const float xh = (x[e] - mean) * rstd;
        c[0] = fmaf(xh, wdy, c[0]);
        c[1] += wdy;
      }
    }
    block_reduce<2>(c, w.red + 128, OpSum());
    const float c1 = c[0] * inv_d;
    const float c2 = (ln || a.ref_compat_c2) ? c[1] * inv_d : 0.f;
    __nv_bfloat16* dxrow = a.dx + row * static_cast<long long>(D);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float x[8], g[8], wv[8], d[8];
      load8<__nv_bfloat16>(w.xr, v << 3, x);
      load8<GT>(gs, v << 3, g);
      if (a.param_bf16) load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(a.weight), v << 3, wv);
      else load8<float>(static_cast<const float*>(a.weight), v << 3, wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float gy = sizeof(GT) == 4 ? bf16_round(g[e]) : g[e];
        const float wdy = (gemma ? wv[e] + 1.f : wv[e]) * gy;
        const float xh = (x[e] - mean) * rstd;
        d[e] = (wdy - (xh * c1 + c2)) * rstd;
        if (a.need_dw) {
          acc_w[(v << 3) + e] += gy * xh;
          if (a.need_db) acc_b[(v << 3) + e] += gy;
        }
      }
      store8<__nv_bfloat16>(dxrow, v << 3, d);
    }
    __syncthreads();
    if (w.misc[2]) {
      if (threadIdx.x == 0 && p.status) atomicOr(p.status, kStatusWaitExpired);
      drain_ring(ring, i, row + stride, rows, stride);
      break;
    }
    if (threadIdx.x == 0) {
      const long long next = row + ring.stages * stride;
      if (next < rows) { fence_proxy_async(); issue(st, next); }
    }
  }
  if (a.need_dw) {
    // each thread wrote only its own columns; no further sync needed to read them back
    float* pw = a.partials + static_cast<long long>(blockIdx.x) * D;
    float* pb = a.partials + (static_cast<long long>(gridDim.x) + blockIdx.x) * D;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        pw[(v << 3) + e] = acc_w[(v << 3) + e];
        if (a.need_db) pb[(v << 3) + e] = acc_b[(v << 3) + e];
      }
    }
  }
}

// column sums of the per-CTA partial rows -> dweight / dbias
__global__ void reduce_partials_kernel(const float* partials, int nparts, int D, float* dweight, float* dbias) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float sw = 0.f, sb = 0.f;
  for (int r = 0; r < nparts; ++r) sw += partials[static_cast<long long>(r) * D + c];
  dweight[c] = sw;
  if (dbias) {
    for (int r = 0; r < nparts; ++r) sb += partials[static_cast<long long>(nparts + r) * D + c];
    dbias[c] = sb;
  }
}

}  // namespace hyc

using namespace hyc;

extern "C" {

int hyc_norm_bwd_partial_rows(void) { return kPartialRowsMax; }

int hyc_norm_bwd(const hyc_packed* saved, const hyc_norm_bwd_args* g, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int empty = packed_is_empty(saved);
  if (empty < 0) return empty;
  if (empty) {
    // no rows: the parameter gradients are zero
    if (g && g->dweight && cudaMemsetAsync(g->dweight, 0, sizeof(float) * saved->cols, stream) != cudaSuccess) return HYC_ERR_CUDA;
    if (g && g->dbias && cudaMemsetAsync(g->dbias, 0, sizeof(float) * saved->cols, stream) != cudaSuccess) return HYC_ERR_CUDA;
    return HYC_OK;
  }
  int rc = check_packed(saved, false);
  if (rc) return rc;
  if (!g || !g->weight || !g->dy || !g->rstd || !g->dx) return HYC_ERR_NULL;
  if (g->kind < HYC_NORM_RMS || g->kind > HYC_NORM_LAYER) return HYC_ERR_MODE;
  if (g->kind == HYC_NORM_LAYER && !g->mean) return HYC_ERR_NULL;
  if ((g->param_dtype != HYC_F32 && g->param_dtype != HYC_BF16) || (g->dy_dtype != HYC_F32 && g->dy_dtype != HYC_BF16))
    return HYC_ERR_DTYPE;
  if ((g->dweight || g->dbias) && !g->partials) return HYC_ERR_NULL;
  if (g->dbias && !g->dweight) return HYC_ERR_NULL;
  if (!aligned16(g->dy) || !aligned16(g->dx) || !aligned16(g->weight)) return HYC_ERR_ALIGN;
  if (saved->rows == 0) {
    if (g->dweight) cudaMemsetAsync(g->dweight, 0, sizeof(float) * saved->cols, stream);
    if (g->dbias) cudaMemsetAsync(g->dbias, 0, sizeof(float) * saved->cols, stream);
    return HYC_OK;
  }
  const int D = saved->cols;
  if (g->dy_dtype == HYC_BF16 && !g->dweight && saved->rotate) {
    // frozen norm weight, bf16 gradient, rotated record whose segment is 32 chunks wide: one warp per row, a
    // chunk of every segment per lane (six of the eight butterfly stages inside the lane)
    const ChunkBwdPlan cp = plan_chunk_bwd(saved, true);
    if (cp.ok) {
      const int rcb = run_chunk_bwd(saved, cp, g->dy, g->dx, D, g->kind, g->weight, g->param_dtype == HYC_BF16, g->rstd,
                                    g->mean, g->ref_compat_c2, stream);
      if (rcb != HYC_ERR_SHAPE) return rcb;
    }
  }
  if (g->dy_dtype == HYC_BF16 && !g->dweight && !saved->rotate) {
    // frozen norm weight (the adapter case), bf16 gradient, no rotation: one warp per row (a rotated record
    // would be rotated back in both of that kernel's passes; the shuffle pipe is its bound, so it stays on
    // the kernel below, which rotates once and keeps the row in registers)
    // twenty warps where their slots fit the shared memory (2- and 4-bit codes of 4096 channels), else sixteen
    // or twelve (8-bit codes: 12 KB per row)
    WarpBwdPlan wp = plan_warp_bwd(saved, nullptr, true, true, kNormBwdWarpThreads, 1);
    if (!wp.ok) wp = plan_warp_bwd(saved, nullptr, true, true, 512, 1);
    if (!wp.ok) wp = plan_warp_bwd(saved, nullptr, true, true, 384, 1);
    if (wp.ok) {
      WarpBwdArgs wa;
      fill_warp_bwd(&wa, wp, saved, nullptr);
      wa.g = static_cast<const __nv_bfloat16*>(g->dy);
      wa.out1 = static_cast<__nv_bfloat16*>(g->dx);
      wa.kind = g->kind; wa.ref_compat_c2 = g->ref_compat_c2; wa.param_bf16 = g->param_dtype == HYC_BF16;
      wa.weight = g->weight; wa.rstd = g->rstd; wa.mean = g->mean;
      return launch_norm_bwd_warp(wa, wp, stream);
    }
  }
  {
    const BwdPlan bp = plan_bwd_fast(saved, nullptr, 4, true, g->dweight ? (g->dbias ? 2 : 1) : 0, 256, kPartialRowsMax,
                                     align_up(static_cast<uint32_t>(D) * saved->bits / 8, 128) +
                                         static_cast<uint32_t>(D) * (g->dy_dtype == HYC_BF16 ? 2 : 4),
                                     256, 4);
    if (bp.ok) {
      NormBwdFastArgs fa;
      memset(&fa, 0, sizeof(fa));
      fa.p = to_dev(saved);
      fa.kind = g->kind; fa.ref_compat_c2 = g->ref_compat_c2; fa.param_bf16 = g->param_dtype == HYC_BF16;
      fa.weight = g->weight; fa.dy = static_cast<const unsigned char*>(g->dy);
      fa.rstd = g->rstd; fa.mean = g->mean; fa.dx = static_cast<__nv_bfloat16*>(g->dx);
      fa.partials = g->partials; fa.need_dw = g->dweight != nullptr; fa.need_db = g->dbias != nullptr;
      fa.L = bp.L;
      int grid_used = bp.grid;   // partial rows of the weight gradient: one per CTA
#define HYC_NBF(B, UP, RT)                                                                      \
  {                                                                                             \
    if (g->dy_dtype == HYC_BF16) {                                                              \
      auto kern = norm_bwd_n_fast_kernel<B, UP, RT, __nv_bfloat16>;                             \
      rc = set_smem(kern, bp.L.total);                                                          \
      if (rc) return rc;                                                                        \
      grid_used = resident_grid(kern, bp.threads, bp.L.total, bp.grid);                         \
      kern<<<grid_used, bp.threads, bp.L.total, stream>>>(fa); HYC_LAUNCHED();                                  \
    } else {                                                                                    \
      auto kern = norm_bwd_n_fast_kernel<B, UP, RT, float>;                                     \
      rc = set_smem(kern, bp.L.total);                                                          \
      if (rc) return rc;                                                                        \
      grid_used = resident_grid(kern, bp.threads, bp.L.total, bp.grid);                         \
      kern<<<grid_used, bp.threads, bp.L.total, stream>>>(fa); HYC_LAUNCHED();                                  \
    }                                                                                           \
  }
      HYC_BWD_DISPATCH(bp, saved->bits, 4, HYC_NBF)
#undef HYC_NBF
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return cuda_fail(e, "norm_bwd_n_fast_kernel launch");
      if (g->dweight) {
        reduce_partials_kernel<<<(D + 127) / 128, 128, 0, stream>>>(g->partials, grid_used, D, g->dweight, g->dbias); HYC_LAUNCHED();
        e = cudaGetLastError();
        if (e != cudaSuccess) return cuda_fail(e, "reduce_partials_kernel launch");
      }
      return HYC_OK;
    }
  }
  const uint32_t cb = static_cast<uint32_t>(D) * saved->bits / 8;
  LayoutReq req;
  fill_req_packed(&req, saved, false);
  req.xr = true;
  req.slot_bytes = align_up(cb, 128) + static_cast<uint32_t>(D) * (g->dy_dtype == HYC_BF16 ? 2 : 4);
  req.acc_rows = g->dweight ? (g->dbias ? 2 : 1) : 0;
  LaunchPlan plan;
  rc = plan_launch(req, saved->rows, &plan, kPartialRowsMax);
  if (rc) return rc;
  NormBwdArgs a;
  memset(&a, 0, sizeof(a));
  a.p = to_dev(saved);
  a.kind = g->kind; a.ref_compat_c2 = g->ref_compat_c2; a.param_bf16 = g->param_dtype == HYC_BF16;
  a.weight = g->weight; a.dy = static_cast<const unsigned char*>(g->dy);
  a.rstd = g->rstd; a.mean = g->mean; a.dx = static_cast<__nv_bfloat16*>(g->dx);
  a.partials = g->partials; a.need_dw = g->dweight != nullptr; a.need_db = g->dbias != nullptr;
  a.L = plan.L;
#define HYC_NB_CASE(MODE, BITS)                                             \
  {                                                                         \
    if (g->dy_dtype == HYC_BF16) {                                          \
      auto kern = norm_bwd_kernel<MODE, BITS, __nv_bfloat16>;               \
      rc = set_smem(kern, plan.L.total);                                    \
      if (rc) return rc;                                                    \
      kern<<<plan.grid, plan.threads, plan.L.total, stream>>>(a); HYC_LAUNCHED();           \
    } else {                                                                \
      auto kern = norm_bwd_kernel<MODE, BITS, float>;                       \
      rc = set_smem(kern, plan.L.total);                                    \
      if (rc) return rc;                                                    \
      kern<<<plan.grid, plan.threads, plan.L.total, stream>>>(a); HYC_LAUNCHED();           \
    }                                                                       \
  }
  HYC_DISPATCH_MODE_BITS(a.p.mode, a.p.bits, HYC_NB_CASE)
#undef HYC_NB_CASE
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "norm_bwd_kernel launch");
  if (g->dweight) {
    reduce_partials_kernel<<<(D + 127) / 128, 128, 0, stream>>>(g->partials, plan.grid, D, g->dweight, g->dbias); HYC_LAUNCHED();
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "reduce_partials_kernel launch");
  }
  return HYC_OK;
}

}  // extern "C"
