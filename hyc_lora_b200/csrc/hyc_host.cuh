// Host-side launch planning / argument validation and the device-side CTA setup
// shared by the row-streaming kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/hyc_b200.h"
#include "hyc_rows.cuh"

namespace hyc {

// ------------------------------------------------------------------ host-side state

extern thread_local char g_cuda_error[256];
extern int g_tune_threads, g_tune_stages, g_tune_ctas;
extern long long g_debug_wait_cycles;   // 0: default limit
extern unsigned int g_debug_tx_pad;     // bytes added to what a staged row announces (test of the give-up path)

inline int cuda_fail(cudaError_t e, const char* what) {
  snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", what, cudaGetErrorString(e));
  return HYC_ERR_CUDA;
}

inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

constexpr uint32_t kSmemBudget = 220 * 1024;  // per SM, leaves room for the per-CTA reserve
constexpr uint32_t kSmemPerCtaMax = 227 * 1024;
constexpr int kPartialRowsMax = 148 * 8;

struct SmemLayout {
  int stages;
  uint32_t slot_bytes;
  uint32_t off_slots, off_red, off_misc, off_omask, off_chan, off_gamax, off_ginv, off_rot, off_list, off_cscale,
      off_xr, off_omask2, off_chan2, off_cscale2, off_xr2, off_acc, off_wsm, off_bsm, off_osm;
  uint32_t total;
};

struct LayoutReq {
  int D = 0;
  uint32_t slot_bytes = 0;
  int k = 0, k2 = 0;
  bool nmode = false, group = false, rot = false, list = false, cscale = false, xr = false;
  bool second = false, nmode2 = false, cscale2 = false;
  bool wsm = false, bsm = false;  // fp32 norm weight / bias rows
  bool osm = false;               // fp32 originals of the outlier channels, ring of 3 rows
  int acc_rows = 0;  // fp32 [acc_rows][D] accumulators
};

inline uint32_t align_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

inline SmemLayout make_layout(const LayoutReq& r, int stages) {
  SmemLayout L;
  memset(&L, 0, sizeof(L));
  uint32_t off = 64;  // mbarriers
  L.off_red = off; off += 6 * 64 * 4;
  L.off_misc = off; off += 64;
  auto take = [&](uint32_t bytes) { uint32_t o = off; off = align_up(off + bytes, 16); return o; };
  if (r.nmode) { L.off_omask = take(r.D / 32 * 4); L.off_chan = take((r.k > 0 ? r.k : 1) * 4); }
  if (r.group) { L.off_gamax = take(r.D / 128 * 4 * 2); L.off_ginv = take(r.D / 128 * 4); }  // gamax: two row parities
  if (r.rot) L.off_rot = take(r.D * 4);
  if (r.list) L.off_list = take(r.D * 4);
  if (r.cscale) L.off_cscale = take(r.D * 4);
  if (r.xr) L.off_xr = take(r.D * 2);
  if (r.second) {
    if (r.nmode2) { L.off_omask2 = take(r.D / 32 * 4); L.off_chan2 = take((r.k2 > 0 ? r.k2 : 1) * 4); }
    if (r.cscale2) L.off_cscale2 = take(r.D * 4);
    L.off_xr2 = take(r.D * 2);
  }
  if (r.wsm) L.off_wsm = take(r.D * 4);
  if (r.bsm) L.off_bsm = take(r.D * 4);
  if (r.osm) L.off_osm = take(3u * (r.k > 0 ? r.k : 1) * 4);
  if (r.acc_rows) L.off_acc = take(static_cast<uint32_t>(r.acc_rows) * r.D * 4);
  off = align_up(off, 128);
  L.off_slots = off;
  L.slot_bytes = align_up(r.slot_bytes, 128);
  L.stages = stages;
  L.total = off + L.slot_bytes * stages;
  return L;
}

struct LaunchPlan {
  SmemLayout L;
  int threads, grid;
};

// Pick threads, staging depth and CTAs per SM so that the staging rings of the
// resident CTAs fill most of an SM's shared memory; the grid is that many CTAs
// on every SM (or one CTA per row when there are fewer rows).
// `min_stages`: the fewest staging slots the kernel works with (a kernel that hands a slot back one row late
// waits forever with fewer than three).
inline int plan_launch(const LayoutReq& r, long long rows, LaunchPlan* out, int grid_cap = 0, int force_threads = 0,
                       int default_stages = 3, int min_stages = 1) {
  int threads = force_threads ? force_threads : g_tune_threads ? g_tune_threads : (r.D <= 1024 ? 64 : r.D <= 4096 ? 128 : 256);
  int stages = g_tune_stages ? g_tune_stages : default_stages;
  if (stages < min_stages) stages = min_stages;
  if (stages > kMaxStages) stages = kMaxStages;
  SmemLayout L = make_layout(r, stages);
  while (L.total > kSmemPerCtaMax && stages > min_stages) L = make_layout(r, --stages);
  if (L.total > kSmemPerCtaMax) return HYC_ERR_SMEM;
  int ctas = g_tune_ctas ? g_tune_ctas : 8;
  while (ctas > 1 && (static_cast<uint32_t>(ctas) * (L.total + 1024) > kSmemBudget || ctas * threads > 2048)) --ctas;
  // with few resident CTAs prefer more threads and fewer stages of a fat row
  if (!g_tune_stages && ctas < 4 && stages > 2 && min_stages <= 2) {
    SmemLayout L2 = make_layout(r, 2);
    int c2 = 8;
    while (c2 > 1 && (static_cast<uint32_t>(c2) * (L2.total + 1024) > kSmemBudget || c2 * threads > 2048)) --c2;
    if (c2 > ctas) { L = L2; ctas = c2; }
  }
  long long grid = static_cast<long long>(sm_count()) * ctas;
  if (grid_cap && grid > grid_cap) grid = grid_cap;
  if (grid > rows) grid = rows;
  out->L = L;
  out->threads = threads;
  out->grid = static_cast<int>(grid);
  return HYC_OK;
}

// The planners size the grid from shared memory and thread counts; registers can allow fewer CTAs on an SM,
// and the CTAs that are not resident at once run as a second, partial wave of the persistent row walk.
// Keeping the grid to what is resident took up to 20 % off the compress kernel (rows of 5120 and 8192
// channels), the norm backward (768 x 4 channels) and the reference-mode decompress; a late partial wave
// measured slightly faster for the activation backward and the decompress with rotation in registers (it
// evens out SMs of unequal speed), which therefore launch the planned grid.
template <typename K>
inline int resident_grid(K kernel, int threads, uint32_t smem_bytes, int grid) {
  if (g_tune_ctas) return grid;   // an explicit tuning request is taken as given
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem_bytes) != cudaSuccess || per_sm < 1) {
    cudaGetLastError();
    return grid;
  }
  const long long cap = static_cast<long long>(sm_count()) * per_sm;
  return grid > cap ? static_cast<int>(cap) : grid;
}

template <typename K>
inline int set_smem(K kernel, uint32_t bytes) {
  if (bytes <= 48 * 1024) return HYC_OK;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute");
  return HYC_OK;
}

// ------------------------------------------------------------------ device: common CTA setup

__device__ __forceinline__ Work make_work(unsigned char* smem, const SmemLayout& L) {
  Work w;
  w.red = reinterpret_cast<float*>(smem + L.off_red);
  w.misc = reinterpret_cast<uint32_t*>(smem + L.off_misc);
  w.omask = reinterpret_cast<uint32_t*>(smem + L.off_omask);
  w.chan = reinterpret_cast<int*>(smem + L.off_chan);
  w.gamax = reinterpret_cast<float*>(smem + L.off_gamax);
  w.ginv = reinterpret_cast<float*>(smem + L.off_ginv);
  w.rot = reinterpret_cast<float*>(smem + L.off_rot);
  w.list = reinterpret_cast<uint32_t*>(smem + L.off_list);
  w.cscale = reinterpret_cast<float*>(smem + L.off_cscale);
  w.xr = reinterpret_cast<__nv_bfloat16*>(smem + L.off_xr);
  return w;
}

// Once per CTA: outlier-channel bitmap and list (north-star mode), per-channel
// scale cache (reference mode).  Ends with a __syncthreads().
__device__ inline void setup_packed(const PackedDev& p, const Work& w) {
  const int D = p.cols;
  if (threadIdx.x < 8) w.misc[threadIdx.x] = 0;
  if (p.mode == kModeN) {
    for (int i = threadIdx.x; i < D / 32; i += blockDim.x) w.omask[i] = 0;
    __syncthreads();
    for (int j = threadIdx.x; j < p.n_channels; j += blockDim.x) {
      const int c = max(0, min(D - 1, p.channels[j]));  // never index outside the row
      w.chan[j] = c;
      atomicOr(&w.omask[c >> 5], 1u << (c & 31));
    }
  } else if (p.scale_kind == kScaleChannel) {
    for (int c = threadIdx.x; c < D; c += blockDim.x) w.cscale[c] = __bfloat162float(p.scale[c]);
  }
  __syncthreads();
}

// after an expired wait: give this CTA's other copies a bounded chance to land
__device__ inline void drain_ring(RowRing& ring, int i_done, long long next_row, long long rows, long long stride,
                                  int in_flight = -1) {
  if (threadIdx.x != 0) return;
  const int last = in_flight < 0 ? ring.stages - 1 : in_flight;
  for (int s = 1; s <= last; ++s) {
    const int i = i_done + s;
    if (next_row + static_cast<long long>(s - 1) * stride >= rows) break;
    (void)mbar_wait_bounded(&ring.bars[i % ring.stages], (i / ring.stages) & 1, ring.wait_cycles);
  }
}

__device__ __forceinline__ void issue_bytes(RowRing& ring, int stage, uint32_t offset, const void* src, uint32_t bytes) {
  bulk_g2s(ring.slot(stage) + offset, src, bytes, &ring.bars[stage]);
}

template <int MODE, int BITS>
__device__ __forceinline__ void dequant_row(const PackedDev& p, const Work& w, const unsigned char* codes_row,
                                            long long row) {
  if (MODE == kModeN) n_dequant_row<BITS>(p, w, codes_row, row);
  else r_dequant_row<BITS>(p, w, codes_row, row);
}

// ------------------------------------------------------------------ host: validation and conversion

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// An empty activation (rows == 0) has no buffers to speak of: the caller's pointers may be null.  Returns 1 when
// the record is a well-formed empty one (nothing to do), 0 when it is not empty, a negative code when malformed.
inline int packed_is_empty(const hyc_packed* q) {
  if (!q) return HYC_ERR_NULL;
  if (q->rows != 0) return 0;
  if (q->mode != HYC_MODE_R && q->mode != HYC_MODE_N) return HYC_ERR_MODE;
  if (q->cols <= 0 || q->cols % 128 != 0 || q->cols > 65408) return HYC_ERR_SHAPE;
  if (q->bits != 1 && q->bits != 2 && q->bits != 4 && q->bits != 8) return HYC_ERR_BITS;
  if (q->mode == HYC_MODE_N && q->bits == 1) return HYC_ERR_BITS;
  return 1;
}

inline int check_packed(const hyc_packed* q, bool for_compress) {
  if (!q || !q->codes) return HYC_ERR_NULL;
  if (q->mode != HYC_MODE_R && q->mode != HYC_MODE_N) return HYC_ERR_MODE;
  if (q->rows < 0 || q->cols <= 0 || q->cols % 128 != 0 || q->cols > 65408 || q->seq < 1) return HYC_ERR_SHAPE;
  if (!aligned16(q->codes)) return HYC_ERR_ALIGN;
  if (q->mode == HYC_MODE_R) {
    if (q->bits != 1 && q->bits != 2 && q->bits != 4 && q->bits != 8) return HYC_ERR_BITS;
    if (q->scale_kind < HYC_SCALE_TENSOR || q->scale_kind > HYC_SCALE_TOKEN) return HYC_ERR_MODE;
    if (q->scale_dtype != HYC_BF16) return HYC_ERR_DTYPE;
    if (!q->scale || !q->pool_used || !q->row_meta || (!q->pool && q->pool_cap)) return HYC_ERR_NULL;
    if (for_compress && !q->thr) return HYC_ERR_NULL;
    if (q->lowrank && !aligned16(q->lowrank)) return HYC_ERR_ALIGN;
  } else {
    if (q->bits != 2 && q->bits != 4 && q->bits != 8) return HYC_ERR_BITS;
    if (q->n_channels < 0 || q->n_channels > q->cols) return HYC_ERR_SHAPE;
    if (q->n_channels > 0 && (!q->channels || !q->out_value)) return HYC_ERR_NULL;
    if (!q->scales) return HYC_ERR_NULL;
    if (q->group != 0 && q->group != 128) return HYC_ERR_SHAPE;
    if (q->rotate != 0) {
      const int n = q->rotate;
      if (n != 16 && n != 64 && n != 256 && n != 1024 && n != 4096) return HYC_ERR_SHAPE;
      if (q->cols % n != 0) return HYC_ERR_SHAPE;
    }
  }
  return HYC_OK;
}

inline PackedDev to_dev(const hyc_packed* q) {
  PackedDev d;
  memset(&d, 0, sizeof(d));
  d.mode = q->mode; d.bits = q->bits; d.rows = q->rows; d.cols = q->cols; d.seq = q->seq;
  d.codes = static_cast<unsigned char*>(q->codes);
  d.status = q->status;
  if (q->mode == HYC_MODE_R) {
    d.scale_kind = q->scale_kind;
    d.scale = static_cast<const __nv_bfloat16*>(q->scale);
    d.thr = q->thr;
    d.lowrank = static_cast<const __nv_bfloat16*>(q->lowrank);
    d.pool = q->pool; d.pool_cap = q->pool_cap; d.pool_used = q->pool_used;
    d.row_meta = reinterpret_cast<uint2*>(q->row_meta);
  } else {
    d.channels = q->channels; d.n_channels = q->n_channels; d.group = q->group; d.rotate = q->rotate;
    d.out_value = static_cast<__nv_bfloat16*>(q->out_value);
    d.scales = q->scales;
  }
  return d;
}

inline int check_dense(const hyc_dense* x, int cols, bool need_plain) {
  if (!x || !x->base) return HYC_ERR_NULL;
  if (x->dtype != HYC_F32 && x->dtype != HYC_BF16) return HYC_ERR_DTYPE;
  const int es = x->dtype == HYC_BF16 ? 2 : 4;
  if (x->chunks < 1 || cols % x->chunks != 0) return HYC_ERR_SHAPE;
  if (need_plain && x->chunks != 1) return HYC_ERR_SHAPE;
  if (!aligned16(x->base) || (x->row_stride * es) % 16 != 0) return HYC_ERR_ALIGN;
  if (x->chunks > 1) {
    const int clen = cols / x->chunks;
    if (clen % 8 != 0 || (clen * es) % 16 != 0) return HYC_ERR_SHAPE;
    if ((x->batch_stride * es) % 16 != 0 || (x->chunk_stride * es) % 16 != 0) return HYC_ERR_ALIGN;
  }
  return HYC_OK;
}

inline void fill_req_packed(LayoutReq* r, const hyc_packed* q, bool compress) {
  r->D = q->cols;
  if (q->mode == HYC_MODE_N) {
    r->nmode = true; r->k = q->n_channels;
    r->group = q->group != 0;
    r->rot = q->rotate != 0;
  } else {
    r->list = compress;
    r->cscale = q->scale_kind == HYC_SCALE_CHANNEL;
  }
}

#define HYC_DISPATCH_MODE_BITS(MODE_V, BITS_V, MACRO)                       \
  if ((MODE_V) == kModeN) {                                                 \
    switch (BITS_V) {                                                       \
      case 2: MACRO(kModeN, 2) break;                                       \
      case 4: MACRO(kModeN, 4) break;                                       \
      default: MACRO(kModeN, 8) break;                                      \
    }                                                                       \
  } else {                                                                  \
    switch (BITS_V) {                                                       \
      case 1: MACRO(kModeR, 1) break;                                       \
      case 2: MACRO(kModeR, 2) break;                                       \
      case 4: MACRO(kModeR, 4) break;                                       \
      default: MACRO(kModeR, 8) break;                                      \
    }                                                                       \
  }

}  // namespace hyc
