/* C ABI of the B200 fused linear cross-entropy (FLCE) library, libflce_b200.so.
 *
 * Plain pointers and sizes only; every pointer is a CUDA device pointer unless the
 * comment says "host".  All functions return a flce_status_t, never throw, and leave a
 * human-readable message retrievable with flce_b200_last_error() (thread local) when
 * they fail.  Work is enqueued on the CUDA stream passed by the caller (a cudaStream_t
 * cast to void*); nothing synchronises the host except flce_b200_check_device_status.
 *
 * The reference has no native interface for this path: its operator is the Python
 * function pair fused_linear_cross_entropy_forward / fused_linear_cross_entropy_backward
 * (src/liger_kernel/ops/fused_linear_cross_entropy.py:21-289, :292-336) wrapped by
 * LigerFusedLinearCrossEntropyFunction (:339-487).  The entry points below are what a
 * native binding of that operator needs; each one names the slice of the reference it
 * replaces.  Status-code + last-error conventions follow the reference's only C ABI
 * (liger_cute_kernels/csrc/core/include/liger_cute/liger_cute.h:19-42).
 */
#ifndef FLCE_B200_H_
#define FLCE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum flce_status {
  FLCE_OK = 0,
  FLCE_ERR_INVALID_ARGUMENT = 1, /* null pointer, bad shape, misaligned pitch ... */
  FLCE_ERR_UNSUPPORTED = 2,      /* combination not implemented / not an sm_100 device */
  FLCE_ERR_WORKSPACE = 3,        /* workspace too small */
  FLCE_ERR_CUDA = 4,             /* a CUDA runtime / driver call failed */
  FLCE_ERR_DEVICE_TIMEOUT = 5    /* a bounded device-side wait expired (see check_device_status) */
} flce_status_t;

typedef enum flce_dtype { FLCE_BF16 = 0, FLCE_FP16 = 1, FLCE_FP32 = 2 } flce_dtype_t;
typedef enum flce_reduction { FLCE_MEAN = 0, FLCE_SUM = 1, FLCE_NONE = 2 } flce_reduction_t;

/* One FLCE problem: logits = x[n_rows, hidden] . w[vocab, hidden]^T (+ bias), then the
 * cross-entropy family of src/liger_kernel/ops/cross_entropy.py:97-336 per row.
 * Arguments mirror LigerFusedLinearCrossEntropyFunction.forward
 * (src/liger_kernel/ops/fused_linear_cross_entropy.py:342-359). */
typedef struct flce_problem {
  int64_t n_rows;       /* N: tokens held by this rank                                        */
  int64_t hidden;       /* H: must be a multiple of 8 (16-byte rows for the TMA engine)      */
  int64_t vocab;        /* V: vocabulary rows of w held by this rank                          */
  int64_t vocab_total;  /* vocabulary size used by label smoothing (== vocab when unsharded)  */
  int64_t vocab_offset; /* global id of local row 0 of w (0 when unsharded)                   */
  int64_t ld_x;         /* row pitch of x in elements (>= hidden, multiple of 8)              */
  int64_t ld_w;         /* row pitch of w in elements (>= hidden, multiple of 8)              */
  int32_t dtype;        /* flce_dtype_t of x and w: FLCE_BF16 or FLCE_FP16                    */
  int32_t reduction;    /* flce_reduction_t                                                   */
  int64_t ignore_index;
  float label_smoothing;
  float lse_square_scale;
  float softcap;             /* 0 = off                                                       */
  int32_t use_token_scaling; /* scale each row's loss and gradient by its detached p(target)  */
  int32_t flags;             /* FLCE_FLAG_* bits                                              */
  const void* x;             /* [n_rows, ld_x]                                                */
  const void* w;             /* [vocab, ld_w]                                                 */
  const int64_t* target;     /* [n_rows] global class ids or ignore_index                     */
  const float* bias;         /* [vocab] fp32 or NULL                                          */
  const float* ce_weight;    /* [vocab] fp32 class weights or NULL                            */
  const int32_t* active_rows;/* NULL, or a device word: only the first *active_rows rows matter (the others are
                              * ignored targets moved to the end by flce_b200_compact_rows); the sweeps then skip
                              * the token tiles that hold none of them                                 */
} flce_problem_t;

/* flce_problem_t.flags: track the arg-max of every row in the forward sweep (needed for token accuracy
 * and predicted tokens; rowstats planes 4 and 5 are only meaningful with it). */
#define FLCE_FLAG_ARGMAX 1

/* Number of fp32 planes in a row-statistics buffer ([FLCE_ROWSTAT_PLANES][n_rows]):
 * 0 max, 1 sum-exp relative to max, 2 target logit (0 unless this rank owns the target),
 * 3 sum of (class-weighted) soft-capped logits, 4 arg-max value, 5 arg-max index (int32 bits). */
#define FLCE_ROWSTAT_PLANES 6

/* Outputs of the forward pass.  Optional pointers may be NULL. */
typedef struct flce_forward_out {
  float* lse;               /* [n_rows] log-sum-exp of the soft-capped logits (saved for backward) */
  float* target_prob;       /* [n_rows] p(target) (needed for token scaling), optional             */
  float* loss_rows;         /* [n_rows] per-row loss incl. z-loss, 0 on ignored rows               */
  float* z_loss_rows;       /* [n_rows] optional                                                    */
  float* correct_rows;      /* [n_rows] 1.0 where arg-max == target, optional                       */
  int64_t* predicted_tokens;/* [n_rows] arg-max class id, -1 on ignored rows, optional              */
  float* scalars;           /* [4]: sum(loss_rows), sum(z_loss_rows), token accuracy, n_non_ignore  */
} flce_forward_out_t;

typedef struct flce_backward_args {
  const float* lse;          /* [n_rows] from the forward pass                                      */
  const float* target_prob;  /* [n_rows] from the forward pass; required with token scaling         */
  const float* norm;         /* [4] normalisers, see flce_b200_count                                 */
  const float* grad_output;  /* fp32 upstream gradient: 1 element, or [n_rows] when per_row != 0; NULL = 1 */
  int32_t grad_output_per_row;
  int32_t grad_dtype;        /* flce_dtype_t of grad_input / grad_weight (FLCE_FP32 allowed)        */
  void* grad_input;          /* [n_rows, hidden] dense, or NULL                                     */
  void* grad_weight;         /* [vocab, hidden] dense, or NULL                                      */
  float* grad_bias;          /* [vocab] fp32, or NULL                                               */
  int32_t slab_begin;        /* run only vocabulary slabs [slab_begin, slab_end) of the plan reported by  */
  int32_t slab_end;          /* flce_b200_backward_plan; 0,0 = all slabs                                  */
  /* Optional, for callers that fed 16-bit term splits of fp32 tensors to the logits GEMM (all zero = off):
   * grad_weight = dZ^T . proj_x ([vocab, proj_x_cols]) and grad_input = dZ . proj_w ([n_rows, proj_w_cols]) are then
   * formed against these narrower term matrices instead of x / w, in fp32; with split_logit_grad the 16-bit
   * rounding residual of dZ is kept in a second slab and its products with the first lo_cols_* columns are added. */
  const void* proj_x;        /* [n_rows, ld_proj_x] 16-bit, or NULL = x                                    */
  int64_t proj_x_cols, ld_proj_x;
  const void* proj_w;        /* [vocab, ld_proj_w] 16-bit, or NULL = w                                     */
  int64_t proj_w_cols, ld_proj_w;
  int32_t split_logit_grad;
  int64_t lo_cols_x, lo_cols_w;
} flce_backward_args_t;

typedef struct flce_fused_args {
  const flce_forward_out_t* out; /* lse, target_prob and loss_rows are required here                         */
  float* norm;                   /* [4] output, see flce_b200_count                                           */
  int32_t grad_dtype;            /* flce_dtype_t of grad_input / grad_weight (FLCE_FP32 allowed)              */
  void* grad_input;              /* [n_rows, hidden] dense, or NULL                                           */
  void* grad_weight;             /* [vocab, hidden] dense, or NULL                                            */
  float* grad_bias;              /* [vocab] fp32, or NULL                                                     */
  int32_t norm_given;            /* 1: norm is an input (already counted, e.g. all-reduced over token shards)  */
  int32_t store_mode;            /* flce_store_mode_t: what the bounded 16-bit copy of a chunk holds          */
  /* Optional hook for a caller that sums grad_weight over token shards.  When set, the last token chunk forms
   * grad_weight before grad_input; right after the launch that completes grad_weight has been enqueued the library
   * calls after_grad_weight(user) on the calling thread (the caller records an event on the stream and enqueues its
   * all-reduce on another one), and the one GEMM still to come leaves reserve_sms SMs free so that the collective's
   * kernel finds room beside it.  Takes the place of the separate all-reduce a data-parallel wrapper issues after the
   * reference's backward (the reference leaves it to DDP / FSDP). */
  void (*after_grad_weight)(void* user);
  void* after_grad_weight_user;
  int32_t reserve_sms;
  /* Optional hooks for a caller whose problem is one vocabulary shard of a larger one (vocab < vocab_total; every
   * rank holds all rows and its own columns; the pattern of the reference's
   * src/liger_kernel/ops/vocab_parallel_cross_entropy.py:235-303).  A shard alone cannot finish a row's softmax, so
   * this mode needs all three; each is called on the calling thread, between launches, with device pointers, and does
   * its cross-rank exchange on the same stream (or behind an event recorded on it):
   *   exchange_shift(user, shift, n_rows): shift[r] is the row's reference point where this shard owns the target and
   *       -inf elsewhere: replace it by the maximum over ranks (exp-store form only);
   *   exchange_rowstats(user, rowstats, rows, first_row): the chunk's [FLCE_ROWSTAT_PLANES][rows] statistics of this
   *       shard: replace them by the merge over ranks (max; sum-exp rescaled to it; target logit and logit sum added;
   *       arg-max by value, lowest class on ties);
   *   after_grad_input(user, grad_input_chunk, rows, first_row): this shard's partial grad_input rows of the chunk
   *       (dense [rows, hidden] in grad_dtype, which should be FLCE_FP32 so that the sum over ranks is rounded once)
   *       are complete once the stream reaches this point: start their sum over ranks; the chunk's grad_weight GEMM,
   *       enqueued next, leaves reserve_sms SMs free for it. */
  void (*exchange_shift)(void* user, float* shift, int64_t n_rows);
  void (*exchange_rowstats)(void* user, float* rowstats, int64_t rows, int64_t first_row);
  void (*after_grad_input)(void* user, void* grad_input_chunk, int64_t rows, int64_t first_row);
  void* exchange_user;
} flce_fused_args_t;

/* The single-sweep mode keeps a bounded 16-bit copy of each token chunk's logits.  FLCE_STORE_LOGITS keeps the
 * soft-capped logits and turns them into the logit gradient in place with one more pass once the chunk's
 * log-sum-exp is known (the reference's structure).  FLCE_STORE_EXP keeps E = exp(logit - shift) instead, with a
 * per-row reference point computed up front from the target logit: the gradient GEMMs consume E as it is (the
 * per-row factor exp(shift - lse) moves into their epilogue or other operand, the uniform label-smoothing term
 * becomes a rank-1 correction), so the extra pass disappears and every stored value is good to one 16-bit ulp
 * whatever the logit's size.  It needs bf16 operands (the stored values span e^-87 .. e^60) and does not cover label
 * smoothing combined with a soft-cap, nor grad_bias; FLCE_STORE_AUTO picks it wherever it applies. */
typedef enum { FLCE_STORE_AUTO = 0, FLCE_STORE_LOGITS = 1, FLCE_STORE_EXP = 2 } flce_store_mode_t;

enum { FLCE_PHASE_FORWARD = 0, FLCE_PHASE_BACKWARD = 1, FLCE_PHASE_FUSED = 2, FLCE_PHASE_BACKWARD_SPLIT = 3 };

/* Bytes of scratch the given phase needs for this problem (0 on invalid input).
 * `slab_budget_bytes` caps the logit-gradient slab of the backward pass (0 = default 1 GiB). */
size_t flce_b200_workspace_bytes(const flce_problem_t* p, int phase, size_t slab_budget_bytes);

/* norm is [4] fp32: norm[0] = number of rows whose target != ignore_index, norm[1] = sum of
 * ce_weight[target] over those rows (== norm[0] without class weights), norm[2] = sum of all class
 * weights (== vocab_total without class weights), norm[3] = number of targets that are neither ignore_index nor
 * inside [0, vocab_total) (such rows match no class; a caller may read it to report them).  Replaces the host-synchronising `.item()` reads at
 * src/liger_kernel/ops/fused_linear_cross_entropy.py:92-104.  A token-sharded caller all-reduces
 * norm across ranks before passing it on. */
int flce_b200_count(const flce_problem_t* p, float* norm, void* stream);

/* Sweep 1: logit tiles on the tensor cores, reduced on the fly to per-row statistics; the
 * N x V logits never reach memory.  Replaces the `X_chunk @ W.t()` GEMM plus the first pass of
 * liger_cross_entropy_kernel (src/liger_kernel/ops/fused_linear_cross_entropy.py:114,
 * src/liger_kernel/ops/cross_entropy.py:138-189).  rowstats is [FLCE_ROWSTAT_PLANES][n_rows]. */
int flce_b200_forward_stats(const flce_problem_t* p, float* rowstats, void* workspace, size_t workspace_bytes,
                            void* stream);

/* The same sweep as flce_b200_forward_stats for callers that must not allocate device memory and have no
 * workspace to lend: a host whose memory plan is fixed (for example a server that has handed the whole GPU to
 * its own arena, where a late cudaMalloc fails or fragments the plan), or a latency-critical loop that cannot
 * afford the device-wide synchronisation an allocation implies.  It has no counterpart in the reference, which
 * allocates its scratch through torch on every call.
 *   - The per-tile partial statistics go to a 32 MiB array built into the library (held by every GPU that loads
 *     the library until the process exits).  Limit: planes x ceil(vocab/256) x n_rows <= 8 Mi floats, where planes
 *     = 2, +1 with label smoothing, +2 with FLCE_FLAG_ARGMAX (e.g. 4096 rows x 128256 classes without extras);
 *     larger problems get FLCE_ERR_WORKSPACE and a message naming the limit.
 *   - Inputs and the rowstats output are still the caller's.  The call itself performs no cudaMalloc / cudaFree
 *     and calls no allocating library routine.
 *   - The first call on each device resolves the array's device address (cudaGetSymbolAddress, with that device
 *     current); make that first call before starting any stream capture.
 *   - All calls on a GPU share the one array, and it keeps the previous call's contents; nothing in it needs to
 *     start at zero.  Two calls whose kernels overlap on the same GPU (different streams or threads) race on it:
 *     serialise them.
 *   - p->active_rows is not used here: the sweep always covers all n_rows rows (results are the same, the rows a
 *     caller moved to the end are merely not skipped). */
int flce_b200_forward_stats_static(const flce_problem_t* p, float* rowstats, void* stream);

/* Per-row losses and metrics from (possibly cross-rank merged) statistics, and their sums.
 * Replaces src/liger_kernel/ops/cross_entropy.py:289-336 and
 * src/liger_kernel/ops/fused_linear_cross_entropy.py:272-283. */
int flce_b200_forward_finalize(const flce_problem_t* p, const float* rowstats, const float* norm,
                               const flce_forward_out_t* out, void* stream);

/* count + forward_stats + forward_finalize for the unsharded case.  norm ([4]) and rowstats are
 * caller-provided outputs as well. */
int flce_b200_forward(const flce_problem_t* p, float* norm, float* rowstats, const flce_forward_out_t* out,
                      void* workspace, size_t workspace_bytes, void* stream);

/* Sweep 2: recompute each logit tile, turn it into the logit gradient in the epilogue (bounded
 * [n_rows, slab] workspace), and run grad_weight = dZ^T.X and grad_input += dZ.W on the tensor
 * cores slab by slab.  Replaces the second pass of liger_cross_entropy_kernel
 * (src/liger_kernel/ops/cross_entropy.py:205-283), the projections at
 * src/liger_kernel/ops/fused_linear_cross_entropy.py:225-265 and the upstream-gradient scaling at
 * :292-336 (folded into the logit gradient). */
int flce_b200_backward(const flce_problem_t* p, const flce_backward_args_t* args, void* workspace,
                       size_t workspace_bytes, size_t slab_budget_bytes, void* stream);

/* Single-sweep mode: loss and gradients in one call, for an upstream gradient of 1, without recomputing the
 * logits: per token chunk the logit tiles are reduced to statistics AND kept as a 16-bit copy ([chunk, vocab],
 * bounded by slab_budget_bytes, default 2.5 GiB), turned into the logit gradient in place once the chunk's lse is
 * known, and projected (grad_input chunk written once, grad_weight accumulated over chunks in fp32).  This is the
 * structure of the reference's operator (src/liger_kernel/ops/fused_linear_cross_entropy.py:108-265: gradients
 * are formed inside forward, 6.N.H.V tensor FLOPs instead of 8.N.H.V) on this library's kernels.  reduction
 * 'none' is not available here.  Workspace: flce_b200_workspace_bytes(p, FLCE_PHASE_FUSED, budget). */
int flce_b200_forward_backward(const flce_problem_t* p, const flce_fused_args_t* args, void* workspace,
                               size_t workspace_bytes, size_t slab_budget_bytes, void* stream);

/* ---- The caller in front of the path: the decoder's final RMSNorm, folded into the two row moves ------------------
 * The hidden states that reach the fused operator come out of the model's final norm
 * (src/liger_kernel/transformers/model/llama.py:95-98); the reference runs that norm as its own kernel pair
 * (src/liger_kernel/ops/rms_norm.py:59-139 forward, :143-235 backward) and has no fused counterpart of what follows.
 * flce_b200_compact_rows_rmsnorm is flce_b200_compact_rows with p->x holding the *raw* hidden states: the gather writes
 * y = x * rstd * (offset + gamma) (casting_mode 0 "llama": x * rstd rounded to the input dtype first;
 * 1 "gemma": everything in fp32, one rounding at the end) into x_compact and rstd[i] = 1 / rms of compact row i.  16-bit dtypes, hidden a multiple of 8, at most 16384. */
int flce_b200_compact_rows_rmsnorm(const flce_problem_t* p, const void* gamma, float eps, float offset, int32_t casting_mode,
                                   void* x_compact, int64_t* target_compact, int32_t* perm, int32_t* active_rows, float* rstd,
                                   void* stream);

/* floats of scratch flce_b200_rmsnorm_scatter_backward needs for a hidden size */
int64_t flce_b200_rmsnorm_partial_floats(int64_t hidden);

/* flce_b200_scatter_rows with the norm's backward applied on the way: grad_normed [n_rows, ld_g] is the gradient with respect
 * to the normalised rows in compact order (what the fused operator returns as grad_input), hidden_states the raw rows in token
 * order; grad_hidden row perm[i] receives dx of compact row i (zeros for i >= *active_rows), grad_gamma [hidden] (fp32) the sum
 * over the rows of dy * (x * rstd).  perm / active_rows may be NULL (rows not moved, all of them live). */
int flce_b200_rmsnorm_scatter_backward(const void* grad_normed, int64_t ld_g, const void* hidden_states, int64_t ld_x,
                                       int32_t dtype, int64_t n_rows, int64_t hidden, const void* gamma, const float* rstd,
                                       const int32_t* perm, const int32_t* active_rows, float offset, int32_t casting_mode,
                                       void* grad_hidden, int64_t ld_gx, float* grad_gamma, float* partials, void* stream);

/* ---- Stand-alone cross-entropy on materialised logits (the operator beside the fused path) ----------------------
 * Replaces cross_entropy_forward / cross_entropy_backward and the same Triton kernel
 * (src/liger_kernel/ops/cross_entropy.py:351-502).  Forward reads the logits once and leaves them untouched;
 * backward reads them again and writes the gradient with the upstream gradient folded in (grad may be the logits
 * buffer itself, which is how the reference saves memory).  HBM-bound: 3 * n_rows * vocab * sizeof(element) bytes. */
typedef struct flce_ce_problem {
  int64_t n_rows, vocab;
  int64_t ld;               /* row pitch of logits in elements                                  */
  int32_t dtype;            /* flce_dtype_t of the logits: bf16, fp16 or fp32                   */
  int32_t reduction;        /* flce_reduction_t                                                 */
  int64_t ignore_index;
  float label_smoothing, lse_square_scale, softcap; /* softcap 0 = off                          */
  int32_t flags;            /* reserved, 0                                                      */
  const void* logits;       /* [n_rows, ld]                                                     */
  const int64_t* target;    /* [n_rows]                                                         */
  const float* ce_weight;   /* [vocab] fp32 or NULL                                             */
} flce_ce_problem_t;

/* norm: [4] output (see flce_b200_count); rowstats: [FLCE_ROWSTAT_PLANES][n_rows] output; out as in the fused path. */
int flce_b200_ce_forward(const flce_ce_problem_t* p, float* norm, float* rowstats, const flce_forward_out_t* out,
                         void* stream);

/* grad_logits: [n_rows, ld_grad] in the logits' dtype, may alias p->logits.  coef_scratch: [3 * n_rows] fp32 scratch.
 * grad_output as in flce_backward_args_t. */
int flce_b200_ce_backward(const flce_ce_problem_t* p, const float* lse, const float* norm, const float* grad_output,
                          int32_t grad_output_per_row, void* grad_logits, int64_t ld_grad, float* coef_scratch,
                          void* stream);

/* Forward and backward in one launch: the reference's own form (its forward kernel leaves the logit gradient, for an
 * upstream gradient of 1, in the logits buffer: src/liger_kernel/ops/cross_entropy.py:41-336, :428-466).  Each row is held
 * in the shared memory of a thread-block cluster between the statistics pass and the gradient pass, so HBM traffic is
 * 2 * n_rows * vocab * sizeof(element).  grad_logits ([n_rows, ld_grad], the logits' dtype) may alias p->logits.  Outputs as
 * flce_b200_ce_forward; rows with target == ignore_index are not read (lse 0, gradient 0).  Returns FLCE_ERR_UNSUPPORTED,
 * before anything is launched, when a row is longer than eight CTAs' shared memory (1.6 MB), vocab is not a multiple of the
 * 16-byte vector or rows are not 16-byte aligned: the two entry points above cover those. */
int flce_b200_ce_forward_backward(const flce_ce_problem_t* p, float* norm, float* rowstats, const flce_forward_out_t* out,
                                  void* grad_logits, int64_t ld_grad, void* stream);

/* grad_logits *= grad_output (a device scalar, or one value per row): the reference's cross_entropy_backward
 * (src/liger_kernel/ops/cross_entropy.py:484-502).  A scalar equal to 1 is recognised on the device and costs one empty
 * launch, no host synchronisation. */
int flce_b200_ce_scale_gradient(void* grad_logits, int64_t ld_grad, int64_t n_rows, int64_t vocab, int32_t dtype,
                                const float* grad_output, int32_t grad_output_per_row, void* stream);

/* fp32 inputs on 16-bit tensor cores: writes 16-bit terms of src (term 0 = round(v), term 1 = round(v - term 0),
 * term 2 = round of what is left) side by side: block b of dst, columns [b*block_cols, b*block_cols + cols), holds
 * term pattern[b] (host array of n_blocks <= 8 entries in {0,1,2}); padding columns are zero.  With X split as
 * (0,0,0,1,1,2) and W as (0,1,2,0,1,0) the product of the two wide matrices is x.w to about 2^-24.  No counterpart
 * in the reference, whose fp32 path is a cuBLAS fp32 GEMM (ops/fused_linear_cross_entropy.py:114). */
int flce_b200_split_fp32(const float* src, int64_t rows, int64_t cols, int64_t ld_src, void* dst, int64_t ld_dst,
                         int64_t block_cols, const int32_t* pattern, int32_t n_blocks, int32_t dst_dtype, void* stream);

/* Ignored tokens cost nothing once they are out of the way: stable-partition the rows of p->x / p->target so that
 * rows whose target is not ignore_index come first.  Outputs: x_compact [n_rows, hidden] dense, target_compact [n_rows],
 * perm [n_rows] (original row of each compact row) and *active_rows (how many rows matter), all on the device, no host
 * synchronisation.  Run the forward / backward entry points on a problem that points at the compact arrays and at
 * active_rows; per-row results come out in compact order.  The reference multiplies every row through all three GEMMs and
 * only skips ignored rows inside its cross-entropy kernel (src/liger_kernel/ops/cross_entropy.py:104-116). */
int flce_b200_compact_rows(const flce_problem_t* p, void* x_compact, int64_t* target_compact, int32_t* perm,
                           int32_t* active_rows, void* stream);

/* dst[perm[i]] = src[i] for i < *active_rows and zeros for the other rows (row_bytes a multiple of 16): puts a compact
 * grad_input back into token order. */
int flce_b200_scatter_rows(const void* src, int64_t row_bytes, const int32_t* perm, const int32_t* active_rows,
                           int64_t n_rows, void* dst, void* stream);

/* data[i] *= *scale for n elements of the given dtype; a no-op when the device-resident scale equals 1 (tested on
 * the device, no host synchronisation).  Replaces element_mul_kernel and the torch.equal test before it
 * (src/liger_kernel/ops/utils.py:108-141, ops/fused_linear_cross_entropy.py:292-336). */
int flce_b200_scale_gradient(void* data, int64_t n, int32_t dtype, const float* scale, void* stream);

/* The vocabulary slabs flce_b200_backward will use for this problem and slab budget: slab s covers rows
 * [s * slab_cols, min(vocab, (s+1) * slab_cols)) of w / grad_weight.  A caller that wants to overlap work with
 * the backward pass (e.g. an all-reduce of finished grad_weight rows) calls flce_b200_backward once per slab
 * range, in increasing order, with the same workspace; grad_input is complete after the last slab.
 * No counterpart in the reference (its loop is over token chunks, ops/fused_linear_cross_entropy.py:108). */
int flce_b200_backward_plan(const flce_problem_t* p, size_t slab_budget_bytes, int32_t* n_slabs, int64_t* slab_cols);

/* The token chunks flce_b200_forward_backward will use for this problem and budget: chunk c covers rows
 * [c * chunk_rows, min(n_rows, (c+1) * chunk_rows)).  The height is the tallest one within the budget's last quarter
 * that fills whole waves of grad_input tiles (few and long: K is the vocabulary).  The reference fixes its chunk
 * count from the shapes alone (src/liger_kernel/ops/fused_linear_cross_entropy.py:56-62). */
int flce_b200_forward_backward_plan(const flce_problem_t* p, size_t slab_budget_bytes, int32_t* n_chunks, int64_t* chunk_rows);

/* Plain D = A . B^T on the same main loop (fp32 or 16-bit output), for unit-testing the tensor-core
 * path in isolation.  a_mn_major / b_mn_major select which dimension is contiguous in memory:
 * 0: A is [M, K] (K contiguous), 1: A is [K, M] (M contiguous); likewise B is [N, K] or [K, N].
 * Replaces nothing in the reference (its GEMMs are cuBLAS calls, fused_linear_cross_entropy.py:114,231,257). */
int flce_b200_gemm(const void* a, const void* b, void* d, int64_t m, int64_t n, int64_t k, int64_t ld_a,
                   int64_t ld_b, int64_t ld_d, int32_t ab_dtype, int32_t d_dtype, int32_t a_mn_major,
                   int32_t b_mn_major, int32_t cta_pair, void* stream);

/* flce_b200_gemm with an fp32 accumulator: v = A . B^T (+ acc when acc != NULL); v is written to acc (fp32, in/out,
 * [m, ld_acc]) when acc != NULL and to out ([m, ld_out] in out_dtype: fp32 or the A/B dtype) when out != NULL.  n need
 * not be a multiple of 8 as long as ld_acc / ld_out, rounded to 8 elements, cover it: stores go in 16-byte groups and
 * may touch the padding of a row.  Used by the chunked losses below for grad_weight += dZ^T . X across token chunks
 * (the reference's grad_weight.add_ / torch.addmm, src/liger_kernel/ops/fused_linear_jsd.py:127-150). */
int flce_b200_gemm_accumulate(const void* a, const void* b, float* acc, void* out, int64_t m, int64_t n, int64_t k,
                              int64_t ld_a, int64_t ld_b, int64_t ld_acc, int64_t ld_out, int32_t ab_dtype,
                              int32_t out_dtype, int32_t a_mn_major, int32_t b_mn_major, int32_t cta_pair, void* stream);

/* ---- Fused linear scaled cross-entropy and fused linear JSD: row kernels over a token chunk's logits ----------------
 *
 * Both losses run as a loop over token chunks on the host (as in the reference): logits of the chunk by flce_b200_gemm
 * into a slab [rows, ld] of the operands' dtype, one of the row kernels below over the slab, then the two projections
 * (flce_b200_gemm / flce_b200_gemm_accumulate) from the slab, which by then holds the gradient with respect to the
 * logits.  dtype is the slab's flce_dtype_t; all row arrays are fp32 on the device.
 *
 * Scaled cross-entropy (src/liger_kernel/ops/fused_linear_scaled_cross_entropy.py:50-93), s = z / temperature:
 *   rows: nll[i] = lse(s_i) - s_i[target_i], entropy[i] = lse(s_i) - sum_j p_ij s_ij, both 0 when target_i ==
 *         ignore_index; lse[i] for every row.
 *   grad: logits[i][j] <- (g_nll[i] (p_ij - [j == target_i]) - g_ent[i] p_ij (log p_ij + entropy[i])) / temperature,
 *         zeros on ignored rows; grad_nll / grad_entropy may be NULL (treated as zeros). */
int flce_b200_scaled_ce_rows(const void* logits, int64_t ld, int32_t dtype, int64_t n_rows, int64_t vocab,
                             const int64_t* target, int64_t ignore_index, float temperature, float* nll, float* entropy,
                             float* lse, void* stream);
int flce_b200_scaled_ce_grad(void* logits, int64_t ld, int32_t dtype, int64_t n_rows, int64_t vocab, const int64_t* target,
                             int64_t ignore_index, float temperature, const float* lse, const float* entropy,
                             const float* grad_nll, const float* grad_entropy, void* stream);

/* Scaled cross-entropy fused into the two tensor-core sweeps (no logits slab in forward, a bounded 16-bit slab of the logit
 * gradient per vocabulary slab in backward): the same results as the rows / grad kernels above for 16-bit operands.
 * This is the form the reference's sm_90 path takes (src/liger_kernel/ops/cutedsl/ops/fused_scaled_cross_entropy_sm90.py);
 * on sm_100 the reference falls back to the chunked loop. */
typedef struct flce_sce_problem {
  int64_t n_rows;           /* tokens M                                                          */
  int64_t hidden;           /* H                                                                 */
  int64_t vocab;            /* V                                                                 */
  int64_t ld_x;             /* row pitch of x in elements (multiple of 8)                        */
  int64_t ld_w;             /* row pitch of w in elements (multiple of 8)                        */
  int32_t dtype;            /* FLCE_BF16 or FLCE_FP16                                            */
  int32_t reserved;         /* 0                                                                 */
  int64_t ignore_index;
  float temperature;        /* finite, > 0                                                       */
  float reserved2;          /* 0                                                                 */
  const void* x;            /* [n_rows, ld_x]                                                    */
  const void* w;            /* [vocab, ld_w]                                                     */
  const int64_t* target;    /* [n_rows]                                                          */
} flce_sce_problem_t;

/* phase: FLCE_PHASE_FORWARD or FLCE_PHASE_BACKWARD (slab_budget_bytes as in flce_b200_workspace_bytes; 0 = 1 GiB). */
size_t flce_b200_sce_workspace_bytes(const flce_sce_problem_t* p, int phase, size_t slab_budget_bytes);

/* nll, entropy (both 0 on ignored tokens) and lse, [n_rows] fp32 each. */
int flce_b200_sce_forward(const flce_sce_problem_t* p, float* nll, float* entropy, float* lse, void* workspace,
                          size_t workspace_bytes, void* stream);

/* lse / entropy from the forward call; grad_nll / grad_entropy [n_rows] fp32, either may be NULL (zeros).  grad_input
 * [n_rows, hidden] and grad_weight [vocab, hidden] (dense, in grad_dtype: the operands' dtype or FLCE_FP32) may each be
 * NULL.  grad_input is accumulated over vocabulary slabs in fp32 and rounded once. */
int flce_b200_sce_backward(const flce_sce_problem_t* p, const float* lse, const float* entropy, const float* grad_nll,
                           const float* grad_entropy, int32_t grad_dtype, void* grad_input, void* grad_weight,
                           void* workspace, size_t workspace_bytes, size_t slab_budget_bytes, void* stream);

/* Generalised Jensen-Shannon divergence between the student's and the teacher's distribution of every token
 * (src/liger_kernel/ops/jsd.py:12-93 and the chain rule of src/liger_kernel/ops/fused_linear_jsd.py:118-122):
 * loss_rows[i] = the token's loss / count; student[i][:] <- d loss / d (student logits), zeros when labels[i] ==
 * ignore_index (labels may be NULL: every token counts).  count: device pointer to the number of tokens that matter
 * (norm[0] of flce_b200_count), or NULL to use fixed_count; no host synchronisation either way (the reference reads the
 * count back with .item(), ops/fused_linear_jsd.py:55).  beta 0 = forward KL, 1 = reverse KL. */
int flce_b200_jsd_rows(void* student, int64_t ld_student, const void* teacher, int64_t ld_teacher, int32_t dtype,
                       int64_t n_rows, int64_t vocab, const int64_t* labels, int64_t ignore_index, float beta,
                       float temperature, const float* count, float fixed_count, float* loss_rows, void* stream);

/* Synchronises `stream`, then reports whether any kernel of this library abandoned a bounded wait
 * since the last call (FLCE_ERR_DEVICE_TIMEOUT) and clears the record.  For tests and debugging. */
int flce_b200_check_device_status(void* stream);

/* Exercises the give-up path of the library's bounded device waits without disturbing a real kernel: a one-thread
 * kernel waits on a barrier that can never complete, with a limit of limit_ns nanoseconds (1 .. 1e8).  The wait runs
 * out, the thread records the time-out in the device status word exactly as the tensor-core kernels' roles do, writes
 * 2 to *outcome (device memory; 1 would mean the wait completed) and the kernel returns.  The next
 * flce_b200_check_device_status() reports FLCE_ERR_DEVICE_TIMEOUT once and clears it.  No counterpart in the
 * reference (its Triton kernels have no device-side waits). */
int flce_b200_selftest_wait_expiry(int64_t limit_ns, int32_t* outcome, void* stream);

/* Per-kernel timing for benchmarks; no counterpart in the reference (its benchmarks time whole calls,
 * benchmark/scripts/utils.py:115-172).  While enabled, each tensor-core launch is bracketed by CUDA
 * events on the caller's stream.  profile_read waits for the recorded events and returns, per kernel
 * kind (0 forward statistics sweep, 1 logit-gradient sweep, 2 grad_weight GEMM, 3 grad_input GEMM,
 * 4 plain GEMM), the summed device time in milliseconds and the number of launches; both arrays have
 * FLCE_NUM_KERNEL_KINDS entries. */
#define FLCE_NUM_KERNEL_KINDS 5
int flce_b200_profile_enable(int on);
int flce_b200_profile_read(double* ms_by_kind, int64_t* launches_by_kind, int reset);

/* Kernels launched by this library in this process so far (host-side counter). */
int64_t flce_b200_kernel_launches(void);

/* Tunables (process-wide atomics, meant to be set once at start-up; unknown names are an error):
 *   cta_pair (1)            CTA pairs (cta_group::2) or single CTAs for the tensor-core sweeps
 *   raster_group_bytes      bytes of the re-read operand kept L2-resident per raster group of a sweep
 *   raster_n_group (-1)     gradient GEMMs: n-tiles per raster group (-1 = chosen per GEMM by estimated DRAM traffic, 0 = all)
 *   wide_tiles (1)          256 x 512 tiles for the gradient GEMMs of CTA pairs when K is long
 *   bulk_store (1)          store epilogue through TMA stores / adds from shared memory instead of vector stores
 *   stagger_pct (0)         wide fp32-accumulating GEMMs: cut each pair's first tile at its own K, spread over this % of K
 *   l2_hints (0), poll_sleep_ns (0)   L2 eviction hints on operand loads; back-off of idle epilogue warps
 *   ce_store_exp (1), ce_slice_bytes (73728), ce_warps (8)   one-launch cross-entropy: keep the exponentials of the
 *                           statistics pass; slice of a row per CTA that the cluster size is chosen for; warps per CTA */
int flce_b200_set_option(const char* name, int64_t value);

const char* flce_b200_status_string(int status);
const char* flce_b200_last_error(void);
const char* flce_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FLCE_B200_H_ */
