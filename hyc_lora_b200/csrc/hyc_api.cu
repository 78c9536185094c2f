// Library-wide state, error strings, tuning knobs and the forward entry points
// (argument checks + launch planning; the kernels are instantiated elsewhere).
#include <stdlib.h>

#include "hyc_fwd_r_fast.cuh"
#include "hyc_fwd_warp.cuh"
#include "hyc_fwd_chunk.cuh"
#include "hyc_fwd_wide.cuh"
#include "hyc_fwd_r_warp.cuh"

namespace hyc {

thread_local char g_cuda_error[256] = "";
int g_tune_threads = 0, g_tune_stages = 0, g_tune_ctas = 0;
std::atomic<unsigned long long> g_launch_count{0};
long long g_debug_wait_cycles = 0;
unsigned int g_debug_tx_pad = 0;


// The wide-row kernels (hyc_fwd_wide.cuh): compress-only of rows wider than 4096 channels, activation + compress,
// product + compress.  HYC_ERR_SHAPE: this combination is not built; the caller takes the separate calls.
static int run_wide(int op, const hyc_dense* x, const hyc_dense* x2, void* y, const hyc_packed* out, const hyc_packed* out_y,
                    cudaStream_t stream) {
  static const bool wide_off = getenv("HYC_FWD_WIDE") && getenv("HYC_FWD_WIDE")[0] == '0';
  if (wide_off) return HYC_ERR_SHAPE;
  const WidePlan wp = plan_wide(out, x, out_y);
  if (!wp.ok) return HYC_ERR_SHAPE;
  CUtensorMap m0, m1, m2;
  if (!row_tensor_map(&m0, x->base, out->rows, out->cols, x->row_stride)) return HYC_ERR_SHAPE;
  m1 = m0;
  m2 = m0;
  if (x2 && !row_tensor_map(&m1, x2->base, out->rows, out->cols, x2->row_stride)) return HYC_ERR_SHAPE;
  if (y && !row_tensor_map(&m2, y, out->rows, out->cols, out->cols)) return HYC_ERR_SHAPE;
  WideArgs wa;
  memset(&wa, 0, sizeof(wa));
  wa.p = to_dev(out);
  if (out_y) { wa.p2 = to_dev(out_y); wa.has_p2 = 1; }
  wa.lanes = wp.lanes;
  wa.off_chan = wp.off_chan; wa.off_chan2 = wp.off_chan2; wa.off_red = wp.off_red;
  wa.off_slots = wp.off_slots; wa.slot_stride = wp.slot_stride;
  wa.wait_cycles = g_debug_wait_cycles > 0 ? g_debug_wait_cycles : kWaitCycles;
  wa.tx_pad = g_debug_tx_pad;
  return launch_wide(wa, wp, op, m0, m1, m2, stream);
}

static int run_fwd(const hyc_dense* x, const hyc_norm_fwd* norm, const hyc_packed* out, cudaStream_t stream,
                   const hyc_packed* out_y = nullptr) {
  const int empty = packed_is_empty(out);
  if (empty) return empty < 0 ? empty : HYC_OK;
  int rc = check_packed(out, true);
  if (rc) return rc;
  rc = check_dense(x, out->cols, norm != nullptr);
  if (rc) return rc;
  if (norm) {
    if (!norm->weight || !norm->y || !norm->rstd) return HYC_ERR_NULL;
    if (norm->kind < HYC_NORM_RMS || norm->kind > HYC_NORM_LAYER) return HYC_ERR_MODE;
    if (norm->kind == HYC_NORM_LAYER && (!norm->bias || !norm->mean)) return HYC_ERR_NULL;
    if (norm->param_dtype != HYC_F32 && norm->param_dtype != HYC_BF16) return HYC_ERR_DTYPE;
    if (!aligned16(norm->weight) || !aligned16(norm->y) || (norm->bias && !aligned16(norm->bias))) return HYC_ERR_ALIGN;
  }
  if (out->rows == 0) return HYC_OK;
  const int es = x->dtype == HYC_BF16 ? 2 : 4;
  if (out_y && out->mode != HYC_MODE_N) return HYC_ERR_SHAPE;
  if (out->mode == HYC_MODE_R) {
    // bf16 rows of up to 4096 channels: one warp per row
    const RWarpPlan rw = plan_r_warp(out, x, norm != nullptr, norm && norm->kind == HYC_NORM_LAYER);
    if (rw.ok) {
      RWarpArgs wa;
      memset(&wa, 0, sizeof(wa));
      wa.p = to_dev(out);
      wa.x = static_cast<const __nv_bfloat16*>(x->base);
      wa.row_stride = x->row_stride;
      if (norm) {
        wa.kind = norm->kind; wa.eps = norm->eps; wa.weight = norm->weight; wa.bias = norm->bias;
        wa.param_bf16 = norm->param_dtype == HYC_BF16;
        wa.y = static_cast<__nv_bfloat16*>(norm->y); wa.rstd = norm->rstd; wa.mean = norm->mean;
      }
      wa.off_csc = rw.off_csc; wa.off_crcp = rw.off_crcp; wa.off_wsm = rw.off_wsm; wa.off_bsm = rw.off_bsm;
      wa.off_slots = rw.off_slots; wa.slot_bytes = rw.slot_bytes; wa.off_lr = rw.off_lr;
      wa.wait_cycles = g_debug_wait_cycles > 0 ? g_debug_wait_cycles : kWaitCycles;
      cudaError_t e = cudaMemsetAsync(out->pool_used, 0, sizeof(uint32_t), stream);
      if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(pool_used)");
      return launch_fwd_r_warp(wa, rw, norm != nullptr, stream);
    }
    // register-resident kernel for 2/4/8-bit codes; 1-bit codes and rows too wide for it take the generic kernel
    const RFastPlan rf = plan_r_fast(out, es, norm != nullptr, norm && norm->kind == HYC_NORM_LAYER);
    if (rf.ok) {
      RFastArgs ra;
      memset(&ra, 0, sizeof(ra));
      ra.p = to_dev(out);
      ra.x = static_cast<const unsigned char*>(x->base);
      ra.row_stride = x->row_stride; ra.batch_stride = x->batch_stride; ra.chunk_stride = x->chunk_stride;
      ra.chunks = x->chunks;
      if (norm) {
        ra.kind = norm->kind; ra.eps = norm->eps; ra.weight = norm->weight; ra.bias = norm->bias;
        ra.param_bf16 = norm->param_dtype == HYC_BF16;
        ra.y = norm->y; ra.rstd = norm->rstd; ra.mean = norm->mean;
      }
      ra.L = rf.L;
      cudaError_t e = cudaMemsetAsync(out->pool_used, 0, sizeof(uint32_t), stream);
      if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(pool_used)");
      return x->dtype == HYC_BF16 ? launch_fwd_r_fast_bf16(ra, rf, norm != nullptr, stream)
                                  : launch_fwd_r_fast_f32(ra, rf, norm != nullptr, stream);
    }
  }
  if (out->mode == HYC_MODE_N) {
    // rows wider than one warp holds: up to four warps per row, a chunk of every segment per lane
    // (measured: with a rotation the chunk layout wins, 23 against 26 us at 2048 x 11008; without one the
    // CTA-per-row kernel below does, 15 against 18 us)
    if (!norm && !out_y && out->cols > 4096 && out->rotate && x->dtype == HYC_BF16) {
      const int rw = run_wide(kWideCompress, x, nullptr, nullptr, out, nullptr, stream);
      if (rw != HYC_ERR_SHAPE) return rw;
    }
    // rotated rows whose segment is 32 chunks wide: one warp per row, a chunk of every segment per lane
    static const bool chunk_off = getenv("HYC_FWD_CHUNK") && getenv("HYC_FWD_CHUNK")[0] == '0';
    const ChunkPlan cp = chunk_off ? ChunkPlan{} : plan_chunk_fwd(out, x, norm != nullptr, norm && norm->kind == HYC_NORM_LAYER, out_y);
    CUtensorMap in_map, y_map;
    if (cp.ok && row_tensor_map(&in_map, x->base, out->rows, out->cols, x->row_stride) &&
        (norm ? row_tensor_map(&y_map, norm->y, out->rows, out->cols, x->row_stride) : (y_map = in_map, true))) {
      ChunkFwdArgs ca;
      memset(&ca, 0, sizeof(ca));
      ca.p = to_dev(out);
      if (out_y) ca.p2 = to_dev(out_y);
      if (norm) {
        ca.kind = norm->kind; ca.eps = norm->eps; ca.weight = norm->weight; ca.bias = norm->bias;
        ca.param_bf16 = norm->param_dtype == HYC_BF16;
        ca.rstd = norm->rstd; ca.mean = norm->mean;
      }
      ca.off_chan = cp.off_chan; ca.off_chan2 = cp.off_chan2; ca.off_wsm = cp.off_wsm; ca.off_bsm = cp.off_bsm;
      ca.off_slots = cp.off_slots; ca.slot_bytes = cp.slot_bytes;
      ca.wait_cycles = g_debug_wait_cycles > 0 ? g_debug_wait_cycles : kWaitCycles;
      ca.tx_pad = g_debug_tx_pad;
      return out->bits == 2 ? launch_fwd_chunk_b2(ca, cp, norm != nullptr, in_map, y_map, stream)
           : out->bits == 4 ? launch_fwd_chunk_b4(ca, cp, norm != nullptr, in_map, y_map, stream)
                            : launch_fwd_chunk_b8(ca, cp, norm != nullptr, in_map, y_map, stream);
    }
    // rows of up to 4096 bf16 channels: one warp per row, no CTA barrier in the row loop
    static const bool warp_off = getenv("HYC_FWD_WARP") && getenv("HYC_FWD_WARP")[0] == '0';
    const WarpPlan wp = warp_off ? WarpPlan{} : plan_warp_fwd(out, x, norm != nullptr, norm && norm->kind == HYC_NORM_LAYER, out_y);
    if (out_y && !wp.ok) return HYC_ERR_SHAPE;     // the two-record variant exists on the warp-per-row kernel only
    if (wp.ok) {
      WarpFwdArgs wa;
      memset(&wa, 0, sizeof(wa));
      wa.p = to_dev(out);
      if (out_y) wa.p2 = to_dev(out_y);
      wa.off_chan2 = wp.off_chan2;
      wa.x = static_cast<const __nv_bfloat16*>(x->base);
      wa.row_stride = x->row_stride;
      if (norm) {
        wa.kind = norm->kind; wa.eps = norm->eps; wa.weight = norm->weight; wa.bias = norm->bias;
        wa.param_bf16 = norm->param_dtype == HYC_BF16;
        wa.y = static_cast<__nv_bfloat16*>(norm->y); wa.rstd = norm->rstd; wa.mean = norm->mean;
      }
      wa.off_chan = wp.off_chan; wa.off_wsm = wp.off_wsm; wa.off_bsm = wp.off_bsm;
      wa.off_slots = wp.off_slots; wa.slot_bytes = wp.slot_bytes;
      wa.wait_cycles = g_debug_wait_cycles > 0 ? g_debug_wait_cycles : kWaitCycles;
      return out->bits == 2 ? launch_fwd_warp_b2(wa, wp, norm != nullptr, stream)
           : out->bits == 4 ? launch_fwd_warp_b4(wa, wp, norm != nullptr, stream)
                            : launch_fwd_warp_b8(wa, wp, norm != nullptr, stream);
    }
  }
  FastPlan fast = plan_fast(out, es);
  LayoutReq req;
  fill_req_packed(&req, out, true);
  req.slot_bytes = static_cast<uint32_t>(out->cols) * es;
  if (fast.ok) {
    req.rot = fast.rot == 1;
    req.osm = true;
    req.wsm = norm != nullptr;
    req.bsm = norm != nullptr && norm->kind == HYC_NORM_LAYER;
  }
  LaunchPlan plan;
  // the register-resident kernel frees a slot right after pass 1: two stages suffice and
  // leave room for more resident CTAs
  // (three when the norm output re-reads the staged row after the in-register rotation)
  const bool late_refill = fast.ok && fast.rot == 2 && norm;
  rc = plan_launch(req, out->rows, &plan, 0, fast.ok ? fast.threads : 0, fast.ok ? (late_refill ? 3 : 2) : 3,
                   late_refill ? 3 : 1);
  if (rc == HYC_ERR_SMEM && fast.ok) {
    // the row is too wide for the register-resident kernel's staging: take the generic kernel
    fast.ok = false;
    LayoutReq g;
    fill_req_packed(&g, out, true);
    g.slot_bytes = req.slot_bytes;
    req = g;
    rc = plan_launch(req, out->rows, &plan, 0, 0, 3);
  }
  if (rc) return rc;
  FwdArgs a;
  memset(&a, 0, sizeof(a));
  a.p = to_dev(out);
  a.x = static_cast<const unsigned char*>(x->base);
  a.row_stride = x->row_stride; a.batch_stride = x->batch_stride; a.chunk_stride = x->chunk_stride;
  a.chunks = x->chunks;
  if (norm) {
    a.kind = norm->kind; a.eps = norm->eps; a.weight = norm->weight; a.bias = norm->bias;
    a.param_bf16 = norm->param_dtype == HYC_BF16;
    a.y = norm->y; a.rstd = norm->rstd; a.mean = norm->mean;
  }
  a.L = plan.L;
  if (out->mode == HYC_MODE_R) {
    cudaError_t e = cudaMemsetAsync(out->pool_used, 0, sizeof(uint32_t), stream);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemsetAsync(pool_used)");
  }
  if (fast.ok)
    return x->dtype == HYC_BF16 ? launch_fwd_fast_bf16(a, plan, fast, norm != nullptr, stream)
                                : launch_fwd_fast_f32(a, plan, fast, norm != nullptr, stream);
  return x->dtype == HYC_BF16 ? launch_fwd_bf16(a, plan, norm != nullptr, stream)
                              : launch_fwd_f32(a, plan, norm != nullptr, stream);
}

}  // namespace hyc

using namespace hyc;

extern "C" {

const char* hyc_strerror(int code) {
  switch (code) {
    case HYC_OK: return "ok";
    case HYC_ERR_NULL: return "a required pointer is NULL";
    case HYC_ERR_SHAPE: return "unsupported shape (cols must be a multiple of 128; group 0 or 128; rotate block must divide cols)";
    case HYC_ERR_BITS: return "unsupported bit width";
    case HYC_ERR_DTYPE: return "unsupported dtype";
    case HYC_ERR_MODE: return "unknown mode, scale kind, norm kind or op";
    case HYC_ERR_ALIGN: return "pointer or stride not 16-byte aligned";
    case HYC_ERR_CAPACITY: return "size exceeds a stated maximum";
    case HYC_ERR_CUDA: return "CUDA runtime error";
    case HYC_ERR_SMEM: return "row too large for shared-memory staging";
    default: return "unknown error code";
  }
}

const char* hyc_last_cuda_error(void) { return g_cuda_error; }

int hyc_version(void) { return 100; }

uint64_t hyc_launch_count(void) { return g_launch_count.load(std::memory_order_relaxed); }

int hyc_set_tuning(int threads, int stages, int ctas_per_sm) {
  if (threads != 0 && (threads < 32 || threads > 512 || threads % 32 != 0)) return HYC_ERR_SHAPE;
  if (stages < 0 || stages > kMaxStages || ctas_per_sm < 0 || ctas_per_sm > 16) return HYC_ERR_SHAPE;
  g_tune_threads = threads; g_tune_stages = stages; g_tune_ctas = ctas_per_sm;
  return HYC_OK;
}

int hyc_debug_wait(int64_t wait_cycles, uint32_t tx_pad_bytes) {
  if (wait_cycles < 0 || wait_cycles > kWaitCycles || tx_pad_bytes > 4096 || tx_pad_bytes % 16 != 0) return HYC_ERR_SHAPE;
  g_debug_wait_cycles = wait_cycles;
  g_debug_tx_pad = tx_pad_bytes;
  return HYC_OK;
}

int hyc_compress(const hyc_dense* x, const hyc_packed* out, void* stream) {
  return run_fwd(x, nullptr, out, static_cast<cudaStream_t>(stream));
}

int hyc_norm_compress(const hyc_dense* x, const hyc_norm_fwd* norm, const hyc_packed* out, void* stream) {
  if (!norm) return HYC_ERR_NULL;
  return run_fwd(x, norm, out, static_cast<cudaStream_t>(stream));
}

static int check_wide_call(const hyc_dense* x, void* y, const hyc_packed* out, const hyc_packed* out_y) {
  if (!x || !y || !out) return HYC_ERR_NULL;
  const int empty = packed_is_empty(out);
  if (empty) return empty < 0 ? empty : 1;        // 1: nothing to do
  int rc = check_packed(out, true);
  if (rc) return rc;
  if (out_y && (rc = check_packed(out_y, true))) return rc;
  rc = check_dense(x, out->cols, true);
  if (rc) return rc;
  if (!aligned16(y)) return HYC_ERR_ALIGN;
  if (out->mode != HYC_MODE_N || x->dtype != HYC_BF16) return HYC_ERR_SHAPE;
  return out->rows == 0 ? 1 : HYC_OK;
}

int hyc_act_compress(const hyc_dense* x, int op, void* y, const hyc_packed* out_x, const hyc_packed* out_y, void* stream) {
  if (op != HYC_ACT_SILU && op != HYC_ACT_GELU_TANH) return HYC_ERR_MODE;
  const int rc = check_wide_call(x, y, out_x, out_y);
  if (rc) return rc == 1 ? HYC_OK : rc;
  return run_wide(op == HYC_ACT_SILU ? kWideSilu : kWideGelu, x, nullptr, y, out_x, out_y, static_cast<cudaStream_t>(stream));
}

int hyc_product_compress(const hyc_dense* x1, const hyc_dense* x2, void* y, const hyc_packed* out_x2, const hyc_packed* out_y,
                         void* stream) {
  int rc = check_wide_call(x2, y, out_x2, out_y);
  if (rc) return rc == 1 ? HYC_OK : rc;
  rc = check_dense(x1, out_x2->cols, true);
  if (rc) return rc;
  if (x1->dtype != HYC_BF16) return HYC_ERR_SHAPE;
  return run_wide(kWideProduct, x1, x2, y, out_x2, out_y, static_cast<cudaStream_t>(stream));
}

int hyc_norm_compress2(const hyc_dense* x, const hyc_norm_fwd* norm, const hyc_packed* out_x, const hyc_packed* out_y,
                       void* stream) {
  if (!norm || !out_y) return HYC_ERR_NULL;
  int rc = check_packed(out_y, true);
  if (rc) return rc;
  return run_fwd(x, norm, out_x, static_cast<cudaStream_t>(stream), out_y);
}

}  // extern "C"
