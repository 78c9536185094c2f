/*
 * hyc_b200.h -- C ABI of the B200 (sm_100a) activation compress / decompress+grad
 * kernels that stand behind the HyC-LoRA operator layer.
 *
 * Conventions (all entry points):
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer unless
 *     the comment says "host";
 *   - the caller allocates every buffer (inputs, outputs, scratch); no entry
 *     point allocates, frees or synchronises unless its comment says so;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued on it;
 *   - the return value is HYC_OK (0) or a negative hyc_status; argument errors
 *     are returned BEFORE anything is enqueued; hyc_strerror() names a code;
 *   - conditions only the device can see (outlier pool overflow, an expired
 *     wait) are OR-ed into the caller-owned `status` word of the hyc_packed
 *     record, never trapped;
 *   - an activation of zero rows is valid input everywhere: the call returns
 *     HYC_OK without enqueueing anything (norm backward zeroes the parameter
 *     gradients it was given) and the record's buffer pointers may be NULL.
 *
 * Citations name the reference implementation each entry replaces
 * (paths inside thu-ee-acts-lab/HyC-LoRA).
 */
#ifndef HYC_B200_H
#define HYC_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  HYC_OK = 0,
  HYC_ERR_NULL = -1,        /* a required pointer is NULL                         */
  HYC_ERR_SHAPE = -2,       /* rows/cols/seq/group/rotate not supported           */
  HYC_ERR_BITS = -3,        /* bits not in {1,2,4,8} (R) / {2,4,8} (N)            */
  HYC_ERR_DTYPE = -4,       /* dtype enum out of range or combination unsupported */
  HYC_ERR_MODE = -5,        /* unknown mode / scale kind / op                     */
  HYC_ERR_ALIGN = -6,       /* a pointer or stride is not 16-byte aligned         */
  HYC_ERR_CAPACITY = -7,    /* a size exceeds a stated maximum                    */
  HYC_ERR_CUDA = -8,        /* a CUDA runtime call failed (see hyc_last_cuda_error) */
  HYC_ERR_SMEM = -9         /* the row does not fit the shared-memory staging     */
} hyc_status;

typedef enum { HYC_F32 = 0, HYC_BF16 = 1 } hyc_dtype;

/* Semantic mode of a packed activation.
 *  HYC_MODE_R  the reference's arithmetic: optional low-rank subtraction, scalar
 *              threshold on |x| selecting ELEMENT outliers, static calibrated
 *              scale (per tensor / channel / sequence position), round-half-even
 *              of x/scale, clamp, offset-binary segment packing
 *              (operators/compress_function.py:136-200).
 *  HYC_MODE_N  channel outliers (a fixed ascending channel list kept in bf16),
 *              optional block Walsh-Hadamard rotation, dynamic absmax scale per
 *              row or per 128-channel group; same rounding/clamp/packing.     */
typedef enum { HYC_MODE_R = 0, HYC_MODE_N = 1 } hyc_mode;

typedef enum { HYC_SCALE_TENSOR = 0, HYC_SCALE_CHANNEL = 1, HYC_SCALE_TOKEN = 2 } hyc_scale_kind;

/* bits of the caller-owned status word */
#define HYC_STATUS_POOL_OVERFLOW 1u /* some rows were stored without their element outliers */
#define HYC_STATUS_WAIT_EXPIRED 2u  /* a bounded wait on a staged copy ran out              */

/* The compressed form of one activation of `rows` x `cols` (rows = B*S tokens).
 * Packed codes: byte j of a row holds channel j of each of the 8/bits contiguous
 * row segments, segment s in bit field s*bits (compress_function.py:176-197);
 * 8-bit codes are int8 without offset.  cols must be a multiple of 128.        */
typedef struct {
  int32_t mode;          /* hyc_mode */
  int32_t bits;          /* 1,2,4,8 (R) ; 2,4,8 (N) */
  int64_t rows;          /* T */
  int32_t cols;          /* D, multiple of 128, <= 65408 */
  int32_t seq;           /* rows per batch element: row t uses position t % seq of [seq,*] statics; >= 1 */
  void* codes;           /* u8 [rows, cols*bits/8] */
  uint32_t* status;      /* one word, OR-ed by kernels; may be NULL */

  /* ---- HYC_MODE_R ---- */
  int32_t scale_kind;    /* hyc_scale_kind */
  int32_t scale_dtype;   /* hyc_dtype of `scale` */
  const void* scale;     /* [] / [cols] / [seq] */
  const float* thr;      /* one fp32 threshold (device memory) */
  const void* lowrank;   /* bf16 [seq, cols] = L@R already multiplied, or NULL (rank 0) */
  uint32_t* pool;        /* outlier entries: (bf16 value bits << 16) | column */
  uint32_t pool_cap;     /* entries in pool */
  uint32_t* pool_used;   /* one word: entries reserved so far (compress zeroes it) */
  uint32_t* row_meta;    /* [rows, 2]: (first entry, count) of each row */

  /* ---- HYC_MODE_N ---- */
  const int32_t* channels; /* [n_channels] ascending outlier channels */
  int32_t n_channels;
  int32_t group;         /* 0: one scale per row; 128: one per 128 channels */
  int32_t rotate;        /* 0 or the Hadamard block size in {16,64,256,1024,4096}, dividing cols */
  int32_t _pad;
  void* out_value;       /* bf16 [rows, n_channels] */
  float* scales;         /* f32 [rows, cols/group or 1] */
} hyc_packed;

/* A dense activation as rows of `cols` elements.  chunks == 1: row t starts at
 * base + t*row_stride.  chunks > 1 ([B,H,S,hd] head layout seen as [B,S,H*hd],
 * compress_function.py:4-12): row t = (b,s) with b = t / seq, s = t % seq is the
 * concatenation of `chunks` pieces of cols/chunks elements, piece c starting at
 * base + b*batch_stride + s*row_stride + c*chunk_stride (strides in elements). */
typedef struct {
  void* base;
  int32_t dtype;         /* hyc_dtype */
  int32_t chunks;
  int64_t row_stride;
  int64_t batch_stride;
  int64_t chunk_stride;
} hyc_dense;

typedef enum { HYC_NORM_RMS = 0, HYC_NORM_RMS_GEMMA = 1, HYC_NORM_LAYER = 2 } hyc_norm_kind;
typedef enum { HYC_ACT_SILU = 0, HYC_ACT_GELU_TANH = 1, HYC_ACT_PRODUCT = 2 } hyc_act_op;

const char* hyc_strerror(int code);
/* text of the last CUDA error seen by this library on the calling thread */
const char* hyc_last_cuda_error(void);
int hyc_version(void);
/* Number of kernels this library has launched in this process so far (all threads, all streams;
 * a launch recorded into a CUDA graph counts once, its replays do not).  Diagnostic only. */
uint64_t hyc_launch_count(void);

/* Optional launch tuning for experiments (0 = library default): threads per row-CTA, staging
 * depth, resident CTAs per SM.  The setting is PROCESS-GLOBAL and unsynchronised: it changes the
 * launches of every thread and stream from then on, so set it before the threads that launch are
 * started (or not at all); every other entry point keeps no mutable state. */
int hyc_set_tuning(int threads, int stages, int ctas_per_sm);

/* Test hook for the give-up path of the bounded waits, PROCESS-GLOBAL like hyc_set_tuning and 0/0 in
 * normal use.  It applies to the register-resident consumer kernels (hyc_decompress, hyc_act_bwd,
 * hyc_norm_bwd on 2/4/8-bit records): every staged row announces `tx_pad_bytes` (a multiple of 16,
 * at most 4096) more bytes than are copied, so its barrier never completes, and the wait gives up
 * after `wait_cycles` SM clocks instead of about a second (0 = default limit).  The kernel then
 * raises HYC_STATUS_WAIT_EXPIRED in the record's status word, waits (bounded) for the copies it
 * started, and returns without faulting; its outputs are unspecified but inside their buffers. */
int hyc_debug_wait(int64_t wait_cycles, uint32_t tx_pad_bytes);

/* Compress-only (the sites that are not norms: LoRA-A linear input, SiLU/GELU
 * input, gate*up operands, Q/K/V).  Replaces the eager chain of
 * true_divide_outlier_suboutlier_svd_compress, operators/compress_function.py:136-200,
 * as called from efficient_linear.py:46, efficient_silu.py:35, efficient_gelu.py:35,
 * efficient_hadamard.py:45-46, efficient_gemm.py:50-51,222. */
int hyc_compress(const hyc_dense* x, const hyc_packed* out, void* stream);

/* Standalone reconstruction to bf16 (for library-GEMM consumers).  Replaces
 * true_divide_outlier_suboutlier_svd_decompress, compress_function.py:203-261. */
int hyc_decompress(const hyc_packed* in, const hyc_dense* out_bf16, void* stream);

/* Fused norm forward + compression of the norm INPUT, one pass over each row.
 * Replaces _rms_norm_fwd_fused / _layer_norm_fwd_fused followed by the compress
 * chain (efficient_rmsnorm.py:179-201, efficient_rmsnorm_gemma.py:59,
 * efficient_layernorm.py:236-257).  y has x's dtype and layout (chunks == 1);
 * rstd and mean are fp32 [rows] (mean only for HYC_NORM_LAYER). */
typedef struct {
  int32_t kind;          /* hyc_norm_kind */
  float eps;
  const void* weight;    /* [cols] */
  const void* bias;      /* [cols] or NULL (required for HYC_NORM_LAYER) */
  int32_t param_dtype;   /* hyc_dtype of weight/bias */
  int32_t _pad;
  void* y;
  float* rstd;
  float* mean;
} hyc_norm_fwd;
int hyc_norm_compress(const hyc_dense* x, const hyc_norm_fwd* norm, const hyc_packed* out, void* stream);

/* The same with a second record, `out_y`, that takes the compressed norm OUTPUT y in the same pass.  In the
 * reference every LoRA-A linear behind a norm compresses the norm output again on its own
 * (efficient_linear.py:46 after efficient_rmsnorm.py:201: three times for q/k/v, twice for gate/up); here the
 * kernel that produces y compresses it once, with `out_y`'s own outlier channels.  Channel mode only, bf16
 * rows of up to 4096 channels in the plain layout; both records must share bits, group and rotation.
 * HYC_ERR_SHAPE means "this pair is not taken": make the two calls (hyc_norm_compress, then hyc_compress
 * on y) instead. */
int hyc_norm_compress2(const hyc_dense* x, const hyc_norm_fwd* norm, const hyc_packed* out_x, const hyc_packed* out_y,
                       void* stream);

/* Activation forward + compress, one pass: y = silu(x) (HYC_ACT_SILU) or the exact erf GELU (HYC_ACT_GELU_TANH:
 * the GELU site, named for its backward formula), the record of the input x and, when out_y is not NULL, the
 * record of the output y (the product site behind a SiLU saves it).  Replaces F.silu / F.gelu followed by
 * true_divide_outlier_suboutlier_svd_compress (efficient_silu.py:33-35, efficient_gelu.py:33-35) and the
 * compression of the same tensor by the next site (efficient_hadamard.py:45).  y: bf16 [rows, cols], contiguous.
 * Channel mode, bf16 rows of a multiple of 128 channels, at most 16384; both records in one format.
 * HYC_ERR_SHAPE means "not built for this call": compute y and make the separate hyc_compress calls. */
int hyc_act_compress(const hyc_dense* x, int op, void* y, const hyc_packed* out_x, const hyc_packed* out_y, void* stream);

/* Product forward + compress, one pass: y = x1 * x2, the record of x2 and, when out_y is not NULL, the record
 * of y (the LoRA-A linear behind the product saves it).  The record of x1 is not made here: in the gated MLP
 * x1 is the activation output, whose record hyc_act_compress has already made.  Replaces x1 * x2 and the
 * compress calls of efficient_hadamard.py:43-46 and efficient_linear.py:46.  Same limits and the same meaning
 * of HYC_ERR_SHAPE as hyc_act_compress. */
int hyc_product_compress(const hyc_dense* x1, const hyc_dense* x2, void* y, const hyc_packed* out_x2, const hyc_packed* out_y,
                         void* stream);

/* Decompress + norm backward.  Replaces the decompress chain followed by
 * _rms_norm_bwd_dx_fused/_dwdb or _layer_norm_bwd_dx_fused/_dwdb
 * (efficient_rmsnorm.py:214-269, efficient_layernorm.py:275-335).
 * dy: [rows, cols] bf16 or fp32 (rounded to bf16 first, efficient_rmsnorm.py:216);
 * dx: bf16 [rows, cols].  ref_compat_c2 != 0 keeps the reference's mean(w*dy)
 * term in the RMSNorm formula (efficient_rmsnorm.py:103-104).  When dweight is
 * not NULL, `partials` must hold hyc_norm_bwd_partial_rows() * cols floats
 * (twice that when dbias is not NULL); dweight/dbias are fp32 [cols]. */
typedef struct {
  int32_t kind;
  int32_t ref_compat_c2;
  const void* weight;
  int32_t param_dtype;
  int32_t dy_dtype;
  const void* dy;
  const float* rstd;
  const float* mean;     /* HYC_NORM_LAYER only */
  void* dx;
  float* dweight;        /* NULL: weight is frozen, skip */
  float* dbias;          /* NULL: skip */
  float* partials;       /* scratch, see above */
} hyc_norm_bwd_args;
int hyc_norm_bwd_partial_rows(void);
int hyc_norm_bwd(const hyc_packed* saved, const hyc_norm_bwd_args* args, void* stream);

/* Decompress + activation backward.  Replaces the decompress chain plus the
 * eager gradient formulas of efficient_silu.py:44-53, efficient_gelu.py:44-64
 * (tanh approximation) and efficient_hadamard.py:56-66 (g*x2, x1*g).
 * g and the outputs share `g_dtype` (bf16 or fp32), contiguous [rows, cols].
 * saved2/dx2 are used by HYC_ACT_PRODUCT only. */
int hyc_act_bwd(int op, const hyc_packed* saved1, const hyc_packed* saved2, const void* g,
                int g_dtype, void* dx1, void* dx2, void* stream);

/* Calibration for HYC_MODE_N: fp32 column absmax of x accumulated into
 * score[cols] (caller zeroes it first; repeated calls accumulate the max), then
 * the k best channels, ties to the lower index, written ascending.  Plays the
 * role get_statistics (compress_function.py:292-340) plays for the reference
 * mode.  `rank_scratch` holds cols int32.  Any score bits are accepted: -0 counts
 * as +0 and a NaN orders above +inf (as a descending sort places it), so exactly
 * k entries of `channels` are written. */
int hyc_channel_absmax(const hyc_dense* x, int64_t rows, int32_t cols, int32_t seq, float* score, void* stream);
int hyc_select_channels(const float* score, int32_t cols, int32_t k, int32_t* channels,
                        int32_t* rank_scratch, void* stream);

/* LoRA-A weight gradient from a packed activation, on the tcgen05 tensor cores:
 *     out[n, d] = sum_t grad[t, n] * X_hat[t, d],   fp32 [rank, cols].
 * Replaces the decompress + batched GEMM + batch sum of efficient_linear.py:61,66-67 without
 * writing X_hat to memory.  grad is bf16 [rows, rank] (contiguous, 16-byte aligned), rank a
 * multiple of 8 in [8, 64]; bits in {2,4,8}; cols*bits/8 must be a multiple of 128.  `partials` is
 * 16-byte aligned scratch of hyc_lora_wgrad_scratch_floats(saved, rank) floats (a negative return
 * is a hyc_status).  The sums over tokens are taken in a fixed order (no global atomics).
 * HYC_MODE_N: the columns of the outlier channels are out[:, channels] = grad^T * out_value,
 * computed by extra thread blocks of the same tensor-core kernel; with rotation the result already
 * includes the inverse rotation.
 * HYC_MODE_R: the static scale is folded into the gradient rows (per tensor / per position) or
 * into the result's columns (per channel); the element outliers of the pool are added as a sparse
 * side term by a second kernel.  A low-rank part is NOT included: the caller adds
 * (sum over batch elements of grad)^T * lowrank, a [rank, seq] x [seq, cols] product. */
int64_t hyc_lora_wgrad_scratch_floats(const hyc_packed* saved, int32_t rank);
int hyc_lora_wgrad(const hyc_packed* saved, const void* grad, int32_t rank, float* out, float* partials, void* stream);
/* The same with the result written in `out_dtype` (HYC_F32 or HYC_BF16; 16-byte aligned [rank, cols]): the sums
 * are taken in fp32 as above and rounded once, by the kernel that finishes them, to the dtype of the LoRA-A weight
 * -- the `.to(weight dtype)` that follows the contraction in efficient_linear.py:66-67, without a kernel of its
 * own.  accumulate != 0: the result is added to what `out` holds (in fp32, rounded once) instead of replacing it
 * -- what the autograd engine does with a second gradient for the same weight, without a kernel of its own. */
int hyc_lora_wgrad_to(const hyc_packed* saved, const void* grad, int32_t rank, void* out, int32_t out_dtype,
                      int32_t accumulate, float* partials, void* stream);

/* Thresholded ("sparse") copy of attention probabilities, rows x cols with cols <= 65535.
 * Replaces true_compress_softmax / true_decompress_softmax (compress_function.py:264-275: a
 * torch sparse COO tensor built with a host sync) and the backward of
 * EfficientMemorySoftmaxFunc (efficient_softmax.py:35-45).  Entries of a row sit contiguously in
 * `val`/`col` in ascending column order; row_meta[row] = (first entry, count).  A row that does
 * not fit the pool keeps nothing and raises HYC_STATUS_POOL_OVERFLOW. */
typedef struct {
  int64_t rows;
  int32_t cols;
  int32_t dtype;         /* hyc_dtype of the probabilities / of `val` */
  void* val;             /* [cap] */
  uint16_t* col;         /* [cap] */
  uint32_t cap;
  uint32_t _pad;
  uint32_t* used;        /* one word (compact zeroes it) */
  uint32_t* row_meta;    /* [rows, 2] */
  uint32_t* status;      /* may be NULL */
} hyc_sparse_rows;
/* keep p > *thr (compared in p's dtype) */
int hyc_softmax_compact(const void* p, const float* thr, const hyc_sparse_rows* out, void* stream);
/* dense [rows, cols] of the list's dtype, zeros where nothing was kept */
int hyc_softmax_expand(const hyc_sparse_rows* in, void* dense, void* stream);
/* dx = (g - sum(g * y_kept)) * y_kept; dx is fp32 unless both the list and g are bf16 */
int hyc_softmax_bwd(const hyc_sparse_rows* in, const void* g, int g_dtype, void* dx, void* stream);

/* Frozen base weights of the host models: blockwise 4-bit codebook storage (64 values per fp32
 * absmax, two 4-bit indices per byte, high nibble first) -> bf16.  `n` values, n % 64 == 0;
 * `codebook` is 16 floats on the device.  The reference relies on bitsandbytes for this
 * (bitsandbytes_fix/_function.py:509,540); it is not part of the compression path. */
int hyc_nf4_dequant(const void* codes, const float* absmax, const float* codebook, int64_t n, void* out_bf16,
                    void* stream);

/* Rotary position embedding of the host models, in place on the query and key projections
 * (bf16 [tokens, heads, head_dim], contiguous, head_dim a multiple of 16), half-split pairing as in
 * rotate_half / apply_rotary_pos_emb (models/modeling_llama.py:228-260).  `cos_sin` is fp32
 * [seq, head_dim/2, 2] = (cos, sin) of (position, pair index); the position of a token is
 * token % seq.  `inverse` != 0 rotates by the negative angle (the backward of the forward).
 * Host-model plumbing, not part of the compression path. */
int hyc_rope(void* q, void* k, const float* cos_sin, int64_t tokens, int32_t seq, int32_t heads_q, int32_t heads_k,
             int32_t head_dim, int32_t inverse, void* stream);

/* Channel selection for callers that cannot allocate device memory.  (No counterpart in the
 * reference; added for hosts that own no device allocator -- a foreign-language binding that
 * only sees raw pointers handed to it, or a runtime whose memory plan is frozen once its
 * buffers are reserved, so that asking for even a small rank buffer per call is not an
 * option.)  Same result as hyc_select_channels, but the cols-sized rank scratch is a fixed
 * array inside the library (hyc_select_channels_static_max_cols() entries of int32, 64 KiB,
 * resident on every GPU that loads the library until the process exits).  The entry point
 * calls no allocating routine.  Rules:
 *   - cols above the maximum is refused with HYC_ERR_CAPACITY before anything is enqueued;
 *   - the first call on a device looks the array's address up (one cudaGetSymbolAddress with
 *     that device current); make that first call outside any stream capture;
 *   - all calls on a device share the one array: two calls whose kernels can overlap on the
 *     GPU (different streams) race; keep them on one stream or order them with events;
 *   - the array keeps the previous call's ranks, which is harmless: every rank below cols is
 *     rewritten before it is read;
 *   - the looked-up address is cached per device (host threads may call concurrently); it does
 *     not survive cudaDeviceReset(), so do not call this entry point on a device after resetting it. */
int hyc_select_channels_static_max_cols(void);
int hyc_select_channels_noalloc(const float* score, int32_t cols, int32_t k, int32_t* channels, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* HYC_B200_H */
