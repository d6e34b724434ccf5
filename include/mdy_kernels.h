/*
 * mdy_kernels.h — C ABI of libmdy_kernels.so: hand-written sm_100a CUDA kernels behind the
 * `mdy_triton.core` operator API (RMSNorm, fused add+RMSNorm, RoPE on q/k, SwiGLU, large-vocab
 * cross-entropy).  Every entry point replaces one Triton launch site of the reference package
 * (cited per function as file:line within the reference project).
 *
 * Conventions
 *   - All pointers are DEVICE pointers owned by the caller.  The operator entry points allocate nothing
 *     and keep no state apart from a per-process cached SM count, a launch counter and integer tunables
 *     (the one exception is the set-up call mdy_peer_buffer_create, which exists to allocate).
 *   - Work is enqueued asynchronously on `stream` (a cudaStream_t passed as void*; NULL = legacy
 *     default stream).  No entry point synchronises the host.
 *   - `dtype` is one of MDY_F32 / MDY_F16 / MDY_BF16 and names the element type of every tensor
 *     marked "T" below.  Statistics (rstd, lse, losses, dw partials) are always float32.
 *     All arithmetic is done in float32 regardless of T.
 *   - Strides are in ELEMENTS.  Innermost dimension is always contiguous.
 *   - Return value: 0 = OK; negative = rejected argument (MDY_ERR_*), nothing was launched;
 *     positive = cudaError_t reported by the launch.  Nothing aborts or traps.
 *   - Fast 128-bit paths are taken when base pointers are 16-byte aligned and row strides are a
 *     multiple of 16 bytes; otherwise a scalar path computes the same result.
 */
#ifndef MDY_KERNELS_H_
#define MDY_KERNELS_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MDY_F32 0
#define MDY_F16 1
#define MDY_BF16 2

#define MDY_OK 0
#define MDY_ERR_NULL (-1)      /* a required pointer is NULL                    */
#define MDY_ERR_DTYPE (-2)     /* dtype code not one of MDY_F32/F16/BF16        */
#define MDY_ERR_SIZE (-3)      /* negative size, zero hidden size, D odd, ...   */
#define MDY_ERR_UNSUPPORTED (-4) /* size above a compiled limit                 */
#define MDY_ERR_ARG (-5)       /* any other inconsistent argument               */

/* Label value that marks a row as ignored by the cross-entropy entry points
 * (reference: core/cross_entyopy_loss.py:20,56). */
#define MDY_IGNORE_INDEX (-100)

/* ---- library info ------------------------------------------------------------------------- */

/* ABI version of this header (bumped on any signature change). */
int mdy_version(void);
/* SM count of the current device, cached per device.  Replaces the per-call
 * torch.cuda.get_device_properties('cuda').multi_processor_count of core/rmsnorm.py:79 and
 * core/fused_add_norm.py:87.  Returns <= 0 if no device is usable. */
int mdy_num_sms(void);
/* Number of kernels this library has launched in this process so far. */
int64_t mdy_launch_count(void);
/* Human-readable text for a return code of this ABI (static storage). */
const char* mdy_status_string(int status);
/* Integer knobs for on-device tuning and tests (grid and CTA shapes, kernel selection).  They are not part
 * of the stable interface: the ids are listed in the library's own csrc/tunables.h and mirrored by the
 * Python loader.  Unknown id -> MDY_ERR_ARG; value <= 0 restores the built-in default. */
int mdy_set_tunable(int id, int value);
/* Kernels that wait on hardware barriers bound every wait; if one ever expires they record a non-zero
 * code in a device flag and run to completion with a wrong result instead of hanging.  This call
 * synchronises with the device, returns the flag (0 = no such event, -1 = the flag could not be
 * read) and resets it when clear != 0.  For tests and diagnostics; not needed on the hot path. */
int mdy_last_device_error(int clear);
/* The same flag per kernel family, for diagnosis: source 0 = one-pass cross-entropy (cluster kernel), 1 =
 * one-kernel vocab-parallel cross-entropy, 2 = staged RMSNorm backward; 16-19 = where the first wait of the
 * vocab-parallel kernel expired: kind (1 a row slice never arrived, 2 a peer's record, 3 / 4 a hand-off inside
 * the CTA), CTA, row index within the CTA, thread.  MDY_ERR_ARG for another source. */
int mdy_device_error_of(int source, int clear);
/* Launch geometry of the calling thread's most recent cluster-kernel cross-entropy launch: CTAs per
 * cluster, clusters launched (= co-resident clusters, or M if smaller), threads per CTA, dynamic shared
 * memory per CTA.  Any pointer may be NULL.  Returns MDY_ERR_ARG if this thread has not launched one.
 * For profiling notes and tests; the reference has no counterpart. */
int mdy_ce_last_geometry(int* cluster_ctas, int* clusters, int* threads, int* smem_bytes);
int mdy_get_tunable(int id);

/* ---- RMSNorm ------------------------------------------------------------------------------ */

/* Rows of dw partials `mdy_rmsnorm_bwd` / `mdy_add_rmsnorm_bwd` need for an [M, N] problem:
 * the caller allocates `dw_partial` as float32 [rows, N].  (The reference allocates
 * [NUM_SMS, N]: core/rmsnorm.py:80.) */
int64_t mdy_rmsnorm_bwd_partial_rows(int64_t M, int64_t N, int dtype);

/* y[r,:] = x[r,:] / sqrt(mean(x[r,:]^2) + eps) * w ;  rstd[r] = 1/sqrt(mean + eps).
 * Replaces _rmsnorm_fwd, launched at core/rmsnorm.py:63 (kernel :9-25).
 * x,y: T [M,N] with row strides; rstd: float [M]; w: [N] of element type `w_dtype`, which may
 * differ from T (float32 master weights with bf16 activations); dw of the backward entry points has
 * the weight's type. */
int mdy_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd,
                    int64_t M, int64_t N, int64_t x_row_stride, int64_t y_row_stride,
                    float eps, int dtype, int w_dtype, void* stream);

/* dx = (w*dy - xhat * mean(xhat * w*dy)) * rstd, xhat = x*rstd;  dw = sum_rows(xhat * dy).
 * Replaces _rmsnorm_bwd_dx_fused launched at core/rmsnorm.py:83 (kernel :31-50) AND the host-side
 * `dw.sum(0).to(weight.dtype)` of core/rmsnorm.py:87 (a second small kernel reduces the partials).
 * dw_partial: float scratch [mdy_rmsnorm_bwd_partial_rows(M,N,dtype), N]; dw: w_dtype [N]. */
int mdy_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                    void* dx, void* dw, float* dw_partial,
                    int64_t M, int64_t N, int64_t dy_row_stride, int64_t x_row_stride,
                    int64_t dx_row_stride, int dtype, int w_dtype, void* stream);

/* Same computation and results as mdy_rmsnorm_bwd, for callers that have no device allocator to get
 * the dw_partial scratch from: a host runtime that hands the library fixed buffers only, or code inside
 * a region where cudaMalloc (and torch's caching allocator, which may fall through to it) must not run.
 * It has no counterpart in the reference, which always allocates the partials with torch
 * (core/rmsnorm.py:80).  The partial rows live in a fixed 16 MiB array inside the library's device image
 * (held by every GPU that loads the library until the process exits: the driver sets the array's memory
 * aside when it loads the library's device image on a GPU, which with lazy loading is the first call of
 * any RMSNorm entry point there, not a later call of this one), so this entry point allocates and frees
 * nothing, here or in any routine it calls.
 *   limit      partial rows of this launch * N <= 4 * 2^20 floats, with the partial rows worked out once
 *              per call and that same number both checked and launched (at most
 *              mdy_rmsnorm_bwd_partial_rows(M, N, dtype); on a 148-SM B200: N <= 14168 with 16-bit
 *              activations); larger problems return MDY_ERR_UNSUPPORTED and launch nothing.
 *   first call on each device resolves the array's device address (cudaGetSymbolAddress) with that
 *              device current; make that first call outside any stream capture.
 *   sharing    every call on a device uses the same array.  Nothing in it has to start at zero (each
 *              call overwrites every partial it later reads), but two calls whose kernels overlap on
 *              the GPU — different streams, or different host threads on different streams — race on
 *              it: serialise them on one stream or with events. */
int mdy_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                            void* dx, void* dw,
                            int64_t M, int64_t N, int64_t dy_row_stride, int64_t x_row_stride,
                            int64_t dx_row_stride, int dtype, int w_dtype, void* stream);

/* new_res = x + res (float32 sum, stored as T); y = rmsnorm(unrounded sum) * w; rstd as above.
 * Replaces _add_rmsnorm_fwd launched at core/fused_add_norm.py:71 (kernel :6-26).
 * All of x,res,y,new_res are T [M,N] sharing `row_stride`. */
int mdy_add_rmsnorm_fwd(const void* x, const void* res, const void* w,
                        void* y, void* new_res, float* rstd,
                        int64_t M, int64_t N, int64_t row_stride,
                        float eps, int dtype, int w_dtype, void* stream);

/* d = rmsnorm_bwd(dy; new_res, w, rstd) + dnew_res, written ONCE to `dx` (it is the gradient of both
 * x and the old residual; the reference stores the same values twice, core/fused_add_norm.py:51-52).
 * dnew_res may be NULL (treated as zeros).  Replaces _add_rmsnorm_bwd_dx_fused launched at
 * core/fused_add_norm.py:92 (kernel :29-55) for every N — the reference launch passes
 * BLOCK_N=min(128, ...) (:85) and is only correct for N <= 128; this entry point follows the math. */
int mdy_add_rmsnorm_bwd(const void* dy, const void* dnew_res, const void* new_res, const void* w,
                        const float* rstd, void* dx, void* dw, float* dw_partial,
                        int64_t M, int64_t N, int64_t row_stride, int dtype, int w_dtype,
                        void* stream);

/* ---- RoPE --------------------------------------------------------------------------------- */

/* Rotate-half rotary embedding applied to q (QH heads) and k (KH heads) in ONE launch.
 *   forward : o1 = x1*cos1 - x2*sin1 ; o2 = x2*cos2 + x1*sin2
 *   backward: d1 = g1*cos1 + g2*sin2 ; d2 = g2*cos2 - g1*sin1
 * with x1 = x[..., :D/2], x2 = x[..., D/2:], cos1 = cos[..., :D/2], cos2 = cos[..., D/2:] (same for sin).
 * Replaces _fused_apply_rope_fwd (core/fused_apply_rope.py:113, kernel :8-46) when backward == 0 and
 * _fused_apply_rope_bwd (core/fused_apply_rope.py:132, kernel :50-90) when backward != 0.
 * q_in/q_out: T, logical [B, QH, L, D] addressed with strides (sb, sh, sl), inner stride 1; likewise
 * k.  q_out may equal q_in (in place, as the reference does) or be a different buffer / layout.
 * cos, sin: T [cos_b, L, D] contiguous with cos_b in {1, B} (1 = broadcast over batch,
 * reference :21-22). */
int mdy_rope(const void* q_in, void* q_out, const void* k_in, void* k_out,
             const void* cos, const void* sin,
             int64_t B, int64_t L, int64_t QH, int64_t KH, int64_t D, int64_t cos_b,
             int64_t qi_sb, int64_t qi_sh, int64_t qi_sl,
             int64_t qo_sb, int64_t qo_sh, int64_t qo_sl,
             int64_t ki_sb, int64_t ki_sh, int64_t ki_sl,
             int64_t ko_sb, int64_t ko_sh, int64_t ko_sl,
             int backward, int dtype, void* stream);

/* ---- SwiGLU ------------------------------------------------------------------------------- */

/* y = up * gate * sigmoid(gate).  up, gate, y: T [M, N] with individual row strides, so the same
 * entry point serves the split form (contiguous up and gate; _fused_silu_fwd launched at
 * core/fused_silu.py:76, kernel :8-22) and the fused-projection form where up and gate are the two
 * halves of one [M, 2N] tensor (_fused_silu_fwdv2 launched at core/fused_silu.py:203, kernel
 * :103-131; pass up = x + (order=='up-gate' ? 0 : N), gate = x + (order=='up-gate' ? N : 0),
 * strides 2N). */
int mdy_swiglu_fwd(const void* up, const void* gate, void* y,
                   int64_t M, int64_t N, int64_t up_row_stride, int64_t gate_row_stride,
                   int64_t y_row_stride, int dtype, void* stream);

/* s = sigmoid(gate); act = s*gate; dup = act*dy; dgate = (s + act*(1-s)) * up * dy.
 * Replaces _fused_silu_bwd_dupgate (core/fused_silu.py:93, kernel :25-42) and
 * _fused_silu_bwd_dupgatev2 (core/fused_silu.py:221, kernel :133-168).  dy takes a row stride
 * (the reference reads dy flat and silently mis-reads a non-contiguous dy). */
int mdy_swiglu_bwd(const void* dy, const void* up, const void* gate, void* dup, void* dgate,
                   int64_t M, int64_t N, int64_t dy_row_stride, int64_t up_row_stride,
                   int64_t gate_row_stride, int64_t dup_row_stride, int64_t dgate_row_stride,
                   int dtype, void* stream);

/* ---- cross-entropy ------------------------------------------------------------------------ */

/* Per-row online log-sum-exp over the local vocab slice [vocab_start, vocab_start + V).
 *   label == MDY_IGNORE_INDEX : losses[r] = 0, lse[r] = 0, the row is not read.
 *   split == 0 : lse[r] = logsumexp(logits[r,:]); losses[r] = lse[r] - logits[r,label]
 *                (0 when the label is outside the slice, as the reference leaves it).
 *   split != 0 : lse[r] = local logsumexp; losses[r] = -logits[r,label-vocab_start] when this slice
 *                owns the label, else 0 (vocab-parallel form; the caller combines across ranks).
 * Replaces _cross_entropy_fwd_kernel launched at core/cross_entyopy_loss.py:104 (kernel :13-42).
 * logits: T [M,V] with row stride; labels: int64 [M]; losses, lse: float [M]. */
int mdy_ce_fwd(const void* logits, const int64_t* labels, float* losses, float* lse,
               int64_t M, int64_t V, int64_t row_stride, int64_t vocab_start, int split,
               int dtype, void* stream);

/* dlogits[r,c] = (exp(logits[r,c] - lse[r]) - [c + vocab_start == label]) * dlosses[r*dloss_stride]
 * for rows with a label; rows with MDY_IGNORE_INDEX are zero-filled when fill_ignored != 0 and left
 * untouched otherwise.  dlogits may alias logits (the reference's `inplace`).
 * Replaces _cross_entropy_bwd_kernel launched at core/cross_entyopy_loss.py:135 (kernel :45-80).
 * dlosses: T_loss (dloss_dtype code) with element stride dloss_stride (0 = one broadcast value). */
int mdy_ce_bwd(const void* dlosses, int64_t dloss_stride, int dloss_dtype,
               const void* logits, void* dlogits, const int64_t* labels, const float* lse,
               int64_t M, int64_t V, int64_t row_stride, int64_t vocab_start, int fill_ignored,
               int dtype, void* stream);

/* One-pass loss + gradient: per row, sweep 1 computes lse / loss exactly as mdy_ce_fwd(split=0) and
 * sweep 2 immediately writes dlogits = (softmax - onehot) * g while the row is still on chip, with
 * g = grad_scale_host * (grad_scale_dev ? *grad_scale_dev : 1) the same for every row (the
 * d(loss.sum()/n_items)/dloss of core/cross_entyopy_loss.py:145-149).  Ignored rows are zero-filled.
 * dlogits may alias logits.  Does the work of both launches cited above in a single pass over HBM. */
int mdy_ce_fused(const void* logits, void* dlogits, const int64_t* labels, float* losses, float* lse,
                 const float* grad_scale_dev, float grad_scale_host,
                 int64_t M, int64_t V, int64_t row_stride, int dtype, void* stream);

/* buf[i] *= *scale for i < n, skipped entirely (no memory traffic) when *scale == 1.  Used when the
 * upstream gradient of the scalar loss turns out not to be 1 after mdy_ce_fused already wrote
 * dlogits.  buf: T [n] contiguous; scale: float device scalar. */
int mdy_scale_inplace(void* buf, int64_t n, const float* scale, int dtype, void* stream);

/* ---- row-wise max / min ------------------------------------------------------------------ */

/* Replaces the launches in mdy_triton/core/triton_maxmin.py:66-97 (triton_max) and :149-179
 * (triton_min).  x: T [M, N], inner-contiguous, row stride in elements; values: T [M]; indices: int64
 * [M] = smallest column holding the row's maximum (take_min = 0) or minimum (take_min != 0).  A NaN in
 * a row is returned as its extreme, as torch.max / torch.min do. */
int mdy_rowwise_extreme(const void* x, void* values, int64_t* indices, int64_t M, int64_t N,
                        int64_t row_stride, int take_min, int dtype, void* stream);

/* Vocab-parallel combine after the all-gather of per-rank (lse_local, -x_label) planes.
 * gathered: float [tp, 2, M]; labels: int64 [M]; out lse[r] = logsumexp_t(gathered[t,0,r]);
 * losses[r] = lse[r] + sum_t gathered[t,1,r], or 0 for ignored rows.  Replaces the torch sequence at
 * core/cross_entyopy_loss.py:109-117 (all_gather + all_reduce + logsumexp + masked_fill). */
int mdy_ce_vp_combine(const float* gathered, const int64_t* labels, float* losses, float* lse,
                      int64_t tp, int64_t M, void* stream);

/* ---- vocab-parallel cross-entropy in one kernel per GPU ------------------------------------- */

/* The whole tensor-parallel loss of triton_kernels/cross_entropy/test_ce.py:110-166 (local statistics,
 * the all-gather / all-reduce of core/cross_entyopy_loss.py:109-117, the gradient kernel launched at
 * :133-141) as ONE launch per GPU: each CTA stages row slices of its rank's shard in shared memory,
 * publishes (local lse, -logit[label]) for a row by storing a 16-byte record straight into every rank's
 * exchange buffer (peer memory, over NVLink), and a few rows later polls its own buffer for the records
 * of all ranks, forms the global lse and the loss, and writes (softmax - onehot) * g from the slice it
 * still holds.  The shard is read once and written once; there is no NCCL call.
 *
 *   logits / dlogits / losses / lse   host arrays of n_local_ranks DEVICE pointers: the shard T [M,
 *              shard_cols] (row_stride elements apart), its gradient (may be the same buffer), and the
 *              float [M] outputs (global lse and loss, identical on every rank) of ranks first_rank ..
 *              first_rank + n_local_ranks - 1.  In production n_local_ranks is 1 (one process per GPU);
 *              a larger value runs several ranks' shards as one launch on one GPU, which is how the
 *              exchange is exercised where there are fewer GPUs than ranks.
 *   exchange   host array of tp DEVICE pointers, indexed by rank: every rank's exchange buffer as this
 *              process can address it (its own from mdy_peer_buffer_create, the peers' from
 *              mdy_peer_buffer_open), each of mdy_ce_vp_exchange_bytes(exchange_rows, ...) bytes,
 *              zero-filled once.  The same buffers serve every call.
 *   labels     int64 [M], global vocabulary ids, identical on every rank; MDY_IGNORE_INDEX rows get zero
 *              gradient and loss and take no part in the exchange.
 *   g          grad_scale_host * (*grad_scale_dev if given): the upstream gradient of every row.
 *   epoch      a counter the caller advances by one per call, from 1, in step on all ranks (0 is not
 *              allowed): records of an older call are ignored.
 * All ranks must call it with the same M, shard_cols, tp, exchange_rows and epoch, each on its own GPU at
 * about the same time: a CTA waits, bounded to a few seconds, for the peers' records.  If a wait runs out
 * the affected rows get NaN loss and lse and mdy_last_device_error reports 2; nothing hangs.  The kernels of
 * one call on the participating GPUs must all be able to run at once: do not keep the SMs of a rank busy
 * with a kernel that itself waits for this one.
 * Returns MDY_ERR_UNSUPPORTED (launching nothing) for shards it has no geometry for (columns not a
 * multiple of the 16-byte vector, more than 32 participants per row, unaligned buffers): callers then use
 * mdy_ce_fwd -> all-gather -> mdy_ce_vp_combine -> mdy_ce_bwd. */
int mdy_ce_vp_fused(const void* const* logits, void* const* dlogits, float* const* losses, float* const* lse,
                    void* const* exchange, const int64_t* labels, const float* grad_scale_dev,
                    float grad_scale_host, int64_t M, int64_t shard_cols, int64_t row_stride, int tp,
                    int first_rank, int n_local_ranks, int64_t exchange_rows, uint32_t epoch, int dtype,
                    void* stream);
/* Bytes of one rank's exchange buffer for up to max_rows rows (negative: MDY_ERR_*). */
int64_t mdy_ce_vp_exchange_bytes(int64_t max_rows, int64_t shard_cols, int tp, int dtype);
/* The launch shape mdy_ce_vp_fused picks for shards of shard_cols columns over tp ranks (host arithmetic only, no
 * device needed; no counterpart in the reference): out8 = {column slices per shard row, 16-byte vectors per
 * slice, bytes of a shared-memory slot, slots per CTA, rows between a row's publish and its poll, compute
 * threads per CTA, vectors per thread and chunk, CTAs per SM asked for}.  MDY_ERR_UNSUPPORTED where
 * mdy_ce_vp_fused would return it for the shape. */
int mdy_ce_vp_geometry(int64_t shard_cols, int tp, int dtype, int32_t* out8);

/* Set-up of memory that peers write into (not on the hot path; the reference has no counterpart: it
 * leaves the exchange to NCCL).  create: cudaMalloc + zero fill on the current device, and the 64-byte
 * CUDA IPC handle to pass to the other processes; open: map a peer's buffer from its handle (peer
 * access is enabled as needed); close / destroy undo them. */
int mdy_peer_buffer_create(int64_t bytes, void** ptr, void* ipc_handle_64_bytes);
int mdy_peer_buffer_open(const void* ipc_handle_64_bytes, void** ptr);
int mdy_peer_buffer_close(void* ptr);
int mdy_peer_buffer_destroy(void* ptr);

#ifdef __cplusplus
}
#endif
#endif /* MDY_KERNELS_H_ */
