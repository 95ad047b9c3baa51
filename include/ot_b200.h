/* ot_b200.h - C ABI of libot_b200.so, the sm_100a transducer-loss library.
 *
 * The library replaces the native half of the reference's loss path: the
 * function bound at optimized_transducer/python/csrc/optimized_transducer.cc:12-19,
 * i.e. ot::ComputeTransducerLoss (optimized_transducer/csrc/transducer-loss.h:60-63)
 * and, below it, ot::ComputeTransducerLossCuda (optimized_transducer/csrc/cuda.cu:402-457)
 * with its kernels (optimized_transducer/csrc/kernels.cu).
 *
 * Conventions
 *  - Plain pointers and sizes only; every pointer named `d_*` is DEVICE memory
 *    of the current CUDA device, `stream` is a cudaStream_t passed as void*.
 *  - The library allocates no device memory: the caller provides outputs and
 *    one workspace whose size ot_b200_workspace_bytes() reports.  Two things
 *    live inside the library instead: the fixed scratch array of
 *    ot_b200_scores_noalloc (part of the library image, see there), and, per
 *    device, a few KB of pinned, device-mapped HOST memory for the error
 *    reports (allocated by the first call that asks for reports on a device,
 *    kept until the process exits).
 *  - Every function returns an ot_b200_status; nothing throws, traps or
 *    asserts.  ot_b200_last_error() gives the message of the calling thread's
 *    last failure.
 *  - All work is enqueued on `stream`; functions return without synchronising
 *    unless stated.  Callable from any host thread: calls share nothing but
 *    the caller's workspace, the per-device report words above (sequence
 *    numbers are atomic, every blocking call polls a slot of its own) and a
 *    few per-device caches of launch parameters (atomics).  Exception:
 *    ot_b200_scores_noalloc, whose calls share one scratch array.
 *  - Packed layout (README.md:131-204 of the reference): utterance b owns
 *    T_b*(U_b+1) consecutive rows of `logits`, row(b,t,u) = split_b + t*(U_b+1) + u,
 *    each row holding V values.  64-bit element offsets are used throughout
 *    (the reference's kernels use 32-bit offsets, kernels.cu:49).
 */
#ifndef OT_B200_H_
#define OT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OT_B200_ABI_VERSION 3

typedef enum ot_b200_status {
  OT_B200_OK = 0,
  OT_B200_ERR_ARGUMENT = 1,   /* a host-visible argument is invalid            */
  OT_B200_ERR_CUDA = 2,       /* a CUDA runtime call or a launch failed        */
  OT_B200_ERR_WORKSPACE = 3,  /* workspace missing, misaligned or too small    */
  OT_B200_ERR_INPUT = 4       /* the device-side input check found bad lengths
                                 or targets (see ot_b200_input_error)          */
} ot_b200_status;

/* What the device-side input check (the counterpart of the data-dependent
 * TORCH_CHECKs at transducer-loss.cc:49-66) can report. */
typedef enum ot_b200_input_error {
  OT_B200_INPUT_OK = 0,
  OT_B200_INPUT_BAD_LOGIT_LENGTH = 1,   /* some T_b <= 0                               */
  OT_B200_INPUT_BAD_TARGET_LENGTH = 2,  /* some U_b < 0 or U_b > max_u                 */
  OT_B200_INPUT_ROWS_MISMATCH = 3,      /* sum T_b*(U_b+1) != rows  (:49-51)           */
  OT_B200_INPUT_TARGET_RANGE = 4,       /* targets.max() >= V or a used target < 0 (:53-56) */
  OT_B200_INPUT_MAX_U_MISMATCH = 5,     /* targets.size(1) != max_b U_b  (:62-66)      */
  OT_B200_INPUT_ONE_SYM_INFEASIBLE = 6, /* one_sym_per_frame with U_b > T_b - 1: no
                                           alignment exists; the reference returns
                                           uninitialised memory here                  */
  /* Not input errors, but reported the same way (status word, error report): */
  OT_B200_TOTALS_DIFFER = 7,            /* alpha(T-1,U)+blank and beta(0,0) of an utterance
                                           are not allclose (rtol 1e-5, atol 1e-8): the
                                           check of cpu.cc:795-797; only made when a
                                           report is asked for                          */
  OT_B200_COPY_TIMEOUT = 8,             /* a bounded wait for a bulk copy of the log-prob
                                           or recursion stage ran out: results invalid  */
  OT_B200_INPUT_PACK_LENGTHS = 9        /* a packing helper: some T_b > max_t, U_b + 1 >
                                           max_u1, T_b <= 0, U_b < 0, or the lengths do
                                           not add up to rows                           */
} ot_b200_input_error;

/* Bits of `flags`. */
#define OT_B200_FROM_LOG_SOFTMAX 1u   /* input rows are log-softmax outputs         */
#define OT_B200_ONE_SYM_PER_FRAME 2u  /* modified transducer                        */
#define OT_B200_FP64 4u               /* logits/scores/grad are double, not float   */
#define OT_B200_CHECK_INPUTS 8u       /* ot_b200_forward waits until the forward half
                                         has run and returns its verdict (input check,
                                         totals check, copy timeouts: a few words the
                                         last forward kernel stores into mapped host
                                         memory), like the reference, which raises
                                         inside the call; not allowed during stream
                                         capture                                    */
#define OT_B200_REPORT_ERRORS 1024u   /* the same verdict without the wait: a failed
                                         call leaves a record in mapped host memory,
                                         and the NEXT ot_b200_forward / ot_b200_backward
                                         on the device (or ot_b200_poll_errors) that
                                         finds it returns OT_B200_ERR_INPUT without
                                         launching anything.  The host never waits
                                         for the device, so it can run ahead of it. */
#define OT_B200_FAST_MATH 16u         /* approximate exp/log in the recursions      */
#define OT_B200_LINEAR_DOMAIN 2048u    /* float recursions in a scaled linear domain
                                          (each value m * 2^e) instead of the
                                          reference's log domain: alpha/beta within
                                          one float rounding of the double recursion
                                          (the log-domain float recursion drifts by
                                          about ten), at 1.6x the recursion time.
                                          Ignored for double                        */
#define OT_B200_BF16 128u              /* logits and gradient are bfloat16; scores,  */
#define OT_B200_FP16 256u              /* loss, scale factors and the workspace stay
                                         float (at most one of FP64/BF16/FP16); no
                                         counterpart in the reference (float only)  */
#define OT_B200_TRACE 512u             /* diagnostic: every stage stores when its first
                                         block started and its last block ended
                                         (%globaltimer, ns) as uint64 pairs from byte 64
                                         of the status segment on                   */
#define OT_B200_SHARE_SMS 64u          /* where a streaming kernel runs as one resident
                                         wave of blocks (OT_B200_GRID=wave; the 16-bit
                                         gradient pass), size that wave one SM short:
                                         for callers that keep another kernel resident
                                         beside this path (a collective on a second
                                         stream)                                    */
#define OT_B200_SCALE_PER_UTTERANCE 32u /* ot_b200_backward only: d_scale holds one
                                         factor per utterance (no counterpart in the
                                         reference, which only reduces)             */

/* Byte offsets of the intermediate arrays inside the workspace, for callers
 * (and tests) that want the stage outputs.  Element type is float, or double
 * with OT_B200_FP64.  `den` is unused with OT_B200_FROM_LOG_SOFTMAX.
 *
 * den is indexed by packed row.  lp, alpha and beta are indexed by CELL:
 *   cell(b,t,u) = cell_split[b] + (t+u)*(U_b+1) + u     standard transducer
 *   cell(b,t,u) = cell_split[b] + t*(U_b+1) + u         OT_B200_ONE_SYM_PER_FRAME
 * (the standard recursion advances along anti-diagonals t+u, and storing the
 * cells in that order makes every access of the wavefront coalesced).  Entries
 * that correspond to no lattice cell, and alpha/beta outside the band of the
 * one-symbol-per-frame recursion, are undefined. */
typedef struct ot_b200_workspace_layout {
  uint64_t total_bytes;
  uint64_t status_off;      /* int32[64]: [0] ot_b200_input_error, [1] utterance index,
                               [2] 1 + utterance whose bulk-copy wait ran out (0: none),
                               [3] trace switch; from byte 64: the OT_B200_TRACE timeline */
  uint64_t split_off;       /* int64[N+1]: first packed row of each utterance        */
  uint64_t cell_split_off;  /* int64[N+1]: first cell of each utterance              */
  uint64_t den_off;         /* real[rows]: row-wise logsumexp          (cuda.cu:427)  */
  uint64_t lp_off;          /* real[cells][2]: blank / symbol log-prob (kernels.cu:30-88) */
  uint64_t alpha_off;       /* real[cells]                             (kernels.cu:200-313) */
  uint64_t beta_off;        /* real[cells]                             (kernels.cu:415-519) */
  uint64_t coef_off;        /* per-row gradient coefficients (library-private format) */
  uint64_t scores_beta_off; /* real[N]: beta(0,0), the score seen from the beta side  */
  uint64_t max_cells;       /* capacity of the per-cell arrays                        */
} ot_b200_workspace_layout;

int ot_b200_abi_version(void);

/* Message for the calling thread's most recent non-OK return ("" if none). */
const char *ot_b200_last_error(void);

/* Size and layout of the workspace for a batch of N utterances, `rows` packed
 * rows and targets of width max_u.  Replaces the temporaries the reference
 * allocates per call (row_splits/row_ids cuda.cu:411-415, denominator :427,
 * log_probs :85, alpha/beta :173,249).  The workspace must be 256-byte aligned. */
int ot_b200_workspace_layout_query(int32_t N, int64_t rows, int32_t max_u,
                                   uint32_t flags, ot_b200_workspace_layout *out);
int ot_b200_workspace_bytes(int32_t N, int64_t rows, int32_t max_u, uint32_t flags,
                            uint64_t *bytes_out);

/* Forward half: input check, row-wise logsumexp + blank/target gather, alpha
 * and beta recursions, per-row gradient coefficients, reduced loss.
 *   replaces: the checks of ot::ComputeTransducerLoss (transducer-loss.cc:49-66),
 *   RowSplitsToRowIds (cuda.cu:40-59), ComputeLogProbs[ForLogSoftmax]
 *   (cuda.cu:71-136), ComputeAlpha (cuda.cu:162-213), ComputeBeta (cuda.cu:237-287)
 *   and the reduction of the Python layer (transducer_loss.py:145-152).
 * d_logits        (rows, V) real, read only
 * d_targets       (N, max_u) int32     d_logit_lengths, d_target_lengths  (N) int32
 * d_scores        (N) real out: log P(y_b|x_b) = alpha(T-1,U) + lp_blank(T-1,U)
 * d_loss          NULL, or one real out: loss_scale * -(sum_b scores[b])
 *                 (loss_scale = 1 for reduction "sum", 1/N for "mean")
 * Whenever the verdict of the forward half is not OT_B200_INPUT_OK the streaming
 * kernels do not touch the inputs, *d_loss and (for input errors) d_scores are
 * NaN and ot_b200_backward on this workspace writes nothing.  How the caller
 * learns of it: OT_B200_CHECK_INPUTS (this call returns OT_B200_ERR_INPUT),
 * OT_B200_REPORT_ERRORS (a later call does), or ot_b200_read_input_status(). */
int ot_b200_forward(const void *d_logits, const int32_t *d_targets,
                    const int32_t *d_logit_lengths,
                    const int32_t *d_target_lengths, int32_t N, int64_t rows,
                    int32_t V, int32_t max_u, int32_t blank, uint32_t flags,
                    void *d_workspace, uint64_t workspace_bytes, void *d_scores,
                    void *d_loss, double loss_scale, void *stream);

/* Backward half: one streaming pass that writes
 *     grad = scale * d loss / d logits
 * from the coefficients ot_b200_forward left in the workspace.
 *   replaces: ComputeGradient[OneSymPerFrame] (cuda.cu:308-346) and
 *   ComputeGradientForLogSoftmax[OneSymPerFrame] (cuda.cu:364-400), plus the two
 *   elementwise passes of the Python layer (`grad /= N`, transducer_loss.py:150,
 *   and `ctx.grad.mul_(loss_grad)`, :162), which are folded into `scale`.
 * d_logits   the same rows ot_b200_forward saw
 * d_grad     (rows, V) real out; MAY EQUAL d_logits (the reference's in-place
 *            mode, cuda.cu:449).  With OT_B200_FROM_LOG_SOFTMAX d_logits is not
 *            read and d_grad must be a separate buffer (cuda.cu:444).
 * N, rows, max_u, flags  as given to ot_b200_forward (they fix the layout)
 * scale = scale_host * (d_scale ? *d_scale : 1); d_scale is a device scalar of
 *            the real type (e.g. the upstream gradient of the loss).  With
 *            OT_B200_SCALE_PER_UTTERANCE d_scale must not be NULL and holds N
 *            reals: the rows of utterance b are scaled by scale_host * d_scale[b]
 *            (the upstream gradient of a per-utterance loss vector). */
int ot_b200_backward(const void *d_logits, void *d_grad, int32_t N, int64_t rows,
                     int32_t V, int32_t max_u, int32_t blank, uint32_t flags,
                     const void *d_workspace, uint64_t workspace_bytes,
                     const void *d_scale, double scale_host, void *stream);

/* Loss and gradient in one call: what TransducerLossFunction.forward of the
 * reference does (transducer_loss.py:135-154: native call, loss = -scores,
 * mean/sum, gradient divided by N for "mean"), without its extra pass:
 *   d_scores[b] = log P(y_b|x_b);  *d_loss = loss_scale * -(sum_b d_scores[b])
 *   (d_loss may be NULL);  d_grad = grad_scale * d(-sum_b scores[b])/d logits
 *   (d_grad may be NULL: no gradient; MAY EQUAL d_logits unless
 *   OT_B200_FROM_LOG_SOFTMAX).  Arguments otherwise as for ot_b200_forward.
 * Because the whole step is one call, large batches (raw-logit input with a
 * gradient, >= 192 Mi lattice cells = rows * V) run as two groups of utterances on three
 * streams (the caller's and two the library creates per device on first use):
 * the recursion of one group overlaps the streaming kernels of the other.  The
 * caller's stream waits, by events, for everything before the function's last
 * kernel; results are bitwise those of ot_b200_forward + ot_b200_backward.
 * OT_B200_PIPELINE=0 in the environment keeps everything on the caller's stream. */
int ot_b200_loss_and_gradient(const void *d_logits, void *d_grad, const int32_t *d_targets,
                              const int32_t *d_logit_lengths,
                              const int32_t *d_target_lengths, int32_t N, int64_t rows,
                              int32_t V, int32_t max_u, int32_t blank, uint32_t flags,
                              void *d_workspace, uint64_t workspace_bytes, void *d_scores,
                              void *d_loss, double loss_scale, double grad_scale, void *stream);

/* ot_b200_loss_and_gradient with the caller's own cut of the batch into groups of
 * consecutive utterances.  Batches below the two-group size are pipelined by
 * group: stage 1 runs group after group on the caller's stream, and each group's
 * recursion, coefficient and gradient kernels follow on streams of the library's
 * own (two per group, created per device on first use) as soon as that group's
 * rows are staged, so all recursions run side by side and the gradient pass of one
 * group runs under the recursions of the others.  This is the schedule for a few
 * utterances per GPU (a batch sharded over several GPUs), where one recursion
 * takes longer than all streaming kernels together.
 *   group_rows  HOST array of n_groups + 1 packed-row positions, rising strictly
 *               from 0 to rows; 1 <= n_groups <= 4.  An utterance belongs to the
 *               group in whose range (group_rows[g], group_rows[g+1]] it ends, so
 *               any cut is valid; cuts AT utterance boundaries, shortest utterances
 *               first, overlap best.  NULL with n_groups = 0: min(N, 4) groups cut
 *               at the quantiles of the rows, which is what
 *               ot_b200_loss_and_gradient does.  n_groups = 1 forces the one-stream
 *               schedule.  Batches below 64 Mi lattice cells run on one stream
 *               whatever the cuts: there the step is the longest utterance's own
 *               chain of kernels, and the schedule's cross-stream edges (6-10 us
 *               each) and extra launches cost more than the overlap returns.
 * Results are bitwise those of the one-stream schedule.  No reference counterpart
 * (the reference launches its kernels one after the other, cuda.cu:402-457). */
int ot_b200_loss_and_gradient_groups(const void *d_logits, void *d_grad, const int32_t *d_targets,
                                     const int32_t *d_logit_lengths, const int32_t *d_target_lengths,
                                     int32_t N, int64_t rows, int32_t V, int32_t max_u, int32_t blank,
                                     uint32_t flags, void *d_workspace, uint64_t workspace_bytes,
                                     void *d_scores, void *d_loss, double loss_scale, double grad_scale,
                                     const int64_t *group_rows, int32_t n_groups, void *stream);

/* The forward half WITHOUT logits: the joiner's output projection is fused
 * into stage 1, so the (rows, V) tensor the reference materialises and reads
 * back (logits.logsumexp(1), cuda.cu:427; ComputeLogProbs, kernels.cu:30-60;
 * README.md:3-5 on its memory) never exists:
 *   logits[r,v] = sum_d x[r,d] * w[v,d] (+ bias[v])   in float accumulators
 *   d_x (rows, D) bfloat16: the packed joiner activations;  d_w (V, D) bfloat16:
 *   the projection's weight (torch.nn.Linear layout);  d_bias (V) float or NULL.
 * D a multiple of 8, d_x and d_w 16-byte aligned.  A tcgen05 (5th-generation
 * tensor core) kernel: TMA-staged operands, accumulators in tensor memory, the
 * epilogue keeps per row the running (max, sum) and the blank / target entries.
 * Then the recursions and the closing stage run as in ot_b200_forward; den, lp,
 * alpha, beta in the workspace and d_scores, d_loss are the same quantities.
 * Standard transducer only; `flags` may hold OT_B200_CHECK_INPUTS,
 * OT_B200_REPORT_ERRORS, OT_B200_FAST_MATH, OT_B200_TRACE.  Forward only: the
 * gradient pass needs logits (ot_b200_backward), so this entry serves scoring
 * and validation; size the workspace with flags = 0. */
int ot_b200_forward_linear(const void *d_x, const void *d_w, const float *d_bias,
                           const int32_t *d_targets, const int32_t *d_logit_lengths,
                           const int32_t *d_target_lengths, int32_t N, int64_t rows, int32_t D,
                           int32_t V, int32_t max_u, int32_t blank, uint32_t flags,
                           void *d_workspace, uint64_t workspace_bytes, void *d_scores, void *d_loss,
                           double loss_scale, void *stream);

/* The backward half of ot_b200_forward_linear as far as the logits go:
 *   d_grad_logits[r, v] = scale * d(-sum_b scores[b]) / d logits[r, v]     bfloat16, (rows, V)
 * with logits = x * w^T + bias RECOMPUTED tile by tile on the tensor cores (the same
 * copies and MMAs as the forward kernel) and the gradient formula of ot_b200_backward
 * (kernels.cu:522-779 of the reference) applied in the epilogue, from the per-row
 * records the forward call left in the workspace.  The (rows, V) logits exist in
 * neither half; the caller contracts the gradient tile with its operands
 * (dX = G * w, dW = G^T * x, dbias = column sums of G), e.g. with library GEMMs.
 *   d_workspace  the workspace of the ot_b200_forward_linear call, same N, rows, V, max_u
 *   scale = scale_host * (d_scale ? *d_scale : 1); d_scale a device float or NULL
 * V a multiple of 4, d_grad_logits 8-byte aligned, D a multiple of 8, x and w 16-byte
 * aligned.  When the forward call's verdict was not OK the gradient is all zeros.
 * flags may hold OT_B200_REPORT_ERRORS, OT_B200_FAST_MATH, OT_B200_TRACE.  No
 * counterpart in the reference (it needs the logits, cuda.cu:427-453). */
int ot_b200_backward_linear(const void *d_x, const void *d_w, const float *d_bias, int32_t N,
                            int64_t rows, int32_t D, int32_t V, int32_t max_u, int32_t blank,
                            uint32_t flags, const void *d_workspace, uint64_t workspace_bytes,
                            void *d_grad_logits, const float *d_scale, double scale_host, void *stream);

/* d_grad[i] *= *d_scale for i < count, unless *d_scale == 1 (then the buffer is
 * not touched: the kernel's blocks return after one load).  The counterpart of
 * `ctx.grad.mul_(loss_grad)` (transducer_loss.py:162) for a gradient that
 * ot_b200_loss_and_gradient computed ahead of the backward pass.  d_scale: one
 * device scalar of the arithmetic type (float; double with OT_B200_FP64);
 * `flags`: the storage type of d_grad (OT_B200_FP64 / BF16 / FP16, else float),
 * and optionally OT_B200_REPORT_ERRORS (a pending error record is returned
 * instead of launching, as by ot_b200_backward). */
int ot_b200_scale_gradient(void *d_grad, int64_t count, const void *d_scale, uint32_t flags,
                           void *stream);

/* One call with the reference's semantics, forward + (if d_grad != NULL)
 * backward with scale 1:  the counterpart of
 * _optimized_transducer.compute_transducer_loss
 * (python/csrc/optimized_transducer.cc:15-19), which returns (scores, grad). */
int ot_b200_compute_transducer_loss(const void *d_logits, void *d_grad,
                                    const int32_t *d_targets,
                                    const int32_t *d_logit_lengths,
                                    const int32_t *d_target_lengths, int32_t N,
                                    int64_t rows, int32_t V, int32_t max_u,
                                    int32_t blank, uint32_t flags,
                                    void *d_workspace, uint64_t workspace_bytes,
                                    void *d_scores, void *stream);

/* Error record of calls made with OT_B200_REPORT_ERRORS on the current device.
 * wait != 0: synchronises `stream` first, so every call enqueued on it has
 * delivered its verdict.  Outputs (each may be NULL): the ot_b200_input_error
 * code (0: no failed call since the last poll), the utterance it refers to,
 * and the sequence number of the failed call (calls with a report are counted
 * per device, from 1).  Clears the record.  Always returns OT_B200_OK unless a
 * CUDA call fails; the message of a found error is left in ot_b200_last_error(). */
int ot_b200_poll_errors(int32_t *code_out, int32_t *index_out, int32_t *seq_out,
                        void *stream, int32_t wait);

/* Copies the input-check status out of the workspace (synchronises `stream`).
 * code_out receives an ot_b200_input_error, index_out the offending utterance. */
int ot_b200_read_input_status(const void *d_workspace, uint64_t workspace_bytes,
                              int32_t *code_out, int32_t *index_out, void *stream);

/* ---- Callers' side of the packed layout ----------------------------------
 * Padded batch tensors <-> packed rows, row(b,t,u) = split_b + t*(U_b+1) + u.
 * max_t / max_u1 are the padded extents (max_u1 >= max_b U_b + 1); D is the
 * feature (or vocabulary) size; element type float, or as OT_B200_FP64 /
 * OT_B200_BF16 / OT_B200_FP16 say (16-bit data is added and summed in float and
 * rounded once).  The workspace holds the row splits
 * (ot_b200_pack_workspace_bytes, 8-byte aligned).  If the lengths are
 * inconsistent with rows / max_t / max_u1 the kernels do not follow them: every
 * output element becomes NaN (ot_b200_unpack_to_padded: zero), the int32 at
 * workspace offset (N+1)*8 is non-zero (1 + an offending utterance, or -1 if
 * only the sum differs from rows), and with OT_B200_REPORT_ERRORS in `flags`
 * the failure is recorded for the next call, as for ot_b200_forward. */
int ot_b200_pack_workspace_bytes(int32_t N, uint64_t *bytes_out);

/* out[row(b,t,u), :] = encoder_out[b,t,:] + decoder_out[b,u,:]
 *   replaces the list comprehension + torch.cat the reference prescribes for
 *   the joiner input (README.md:165-177).
 * d_encoder_out (N, max_t, D), d_decoder_out (N, max_u1, D), d_out (rows, D). */
int ot_b200_pack_joiner_input(const void *d_encoder_out, const void *d_decoder_out,
                              const int32_t *d_logit_lengths,
                              const int32_t *d_target_lengths, int32_t N, int64_t rows,
                              int32_t D, int32_t max_t, int32_t max_u1, uint32_t flags,
                              void *d_workspace, void *d_out, void *stream);

/* Its backward: grad_encoder[b,t,:] = sum_u g[row(b,t,u),:] (0 for t >= T_b),
 * grad_decoder[b,u,:] = sum_t g[row(b,t,u),:] (0 for u > U_b); what autograd
 * does for the reference's slicing/broadcast-add/cat. */
int ot_b200_pack_joiner_input_backward(const void *d_grad_out,
                                       const int32_t *d_logit_lengths,
                                       const int32_t *d_target_lengths, int32_t N,
                                       int64_t rows, int32_t D, int32_t max_t,
                                       int32_t max_u1, uint32_t flags, void *d_workspace,
                                       void *d_grad_encoder, void *d_grad_decoder,
                                       void *stream);

/* packed[row(b,t,u), :] = padded[b,t,u,:]   (padded: (N, max_t, max_u1, D))
 *   replaces the slicing/reshape/cat of the reference's tests
 *   (python/tests/test_compute_transducer_loss.py:36-56) for callers that hold
 *   torchaudio-style padded logits. */
int ot_b200_pack_padded(const void *d_padded, const int32_t *d_logit_lengths,
                        const int32_t *d_target_lengths, int32_t N, int64_t rows,
                        int32_t D, int32_t max_t, int32_t max_u1, uint32_t flags,
                        void *d_workspace, void *d_packed, void *stream);

/* The inverse (e.g. gradients back to the padded layout): padded[b,t,u,:] =
 * packed[row(b,t,u),:], zero outside the lattices
 * (test_compute_transducer_loss.py:95-105 slices the padded gradient the same way). */
int ot_b200_unpack_to_padded(const void *d_packed, const int32_t *d_logit_lengths,
                             const int32_t *d_target_lengths, int32_t N, int64_t rows,
                             int32_t D, int32_t max_t, int32_t max_u1, uint32_t flags,
                             void *d_workspace, void *d_padded, void *stream);

/* Scores without any allocation.  This entry point has no counterpart in the
 * reference (every path of the reference allocates its temporaries through
 * torch).  It exists for callers that cannot provide a workspace because they
 * cannot allocate device memory where the loss is evaluated: a server that has
 * given the whole GPU to its own arena, a plug-in hook that must not allocate.
 * The scratch (the alpha lattice) is a fixed array inside the library image,
 * reserved on every GPU that loads the library: 16 MiB, enough for
 * 4 Mi lattice cells (rows = sum_b T_b*(U_b+1) <= 4194304); larger batches
 * return OT_B200_ERR_ARGUMENT.  float32, standard transducer, log-softmax
 * input; computes only the per-utterance scores
 *     d_scores[b] = log P(y_b | x_b)
 * (an utterance whose lengths or targets are invalid gets NaN).  Calls no
 * cudaMalloc/cudaFree and no allocating library routine.  All calls share the
 * one array, so calls that overlap on the GPU race: serialise them.  The first
 * call on a device looks the array's address up (cudaGetSymbolAddress); make
 * that call before any stream capture. */
int ot_b200_scores_noalloc(const float *d_log_probs, const int32_t *d_targets,
                           const int32_t *d_logit_lengths,
                           const int32_t *d_target_lengths, int32_t N, int64_t rows,
                           int32_t V, int32_t max_u, int32_t blank, float *d_scores,
                           void *stream);

/* ---------------------------------------------------------------------------
 * Exchange of one scalar per rank over peer memory: the sum of the per-shard
 * losses of a batch that is sharded by utterance over the GPUs of one node.
 * No counterpart in the reference (single GPU, transducer_loss.py:145-152
 * reduces one tensor); it replaces an NCCL all-reduce of the 0-dim loss.
 *
 * Every rank owns a table of ring x world entries of 16 bytes
 * (ot_b200_exchange_bytes), zeroed before the first use, that all ranks can
 * address (peer-mapped device memory).  d_tables is a DEVICE array of `world`
 * pointers: d_tables[p] = the table owned by rank p, as addressed from this rank.
 *
 * ot_b200_exchange_publish: one warp stores {*d_value, step + 1} into entry
 *   [step % ring][rank] of every table (plain peer stores, value before a
 *   system-scope release of the sequence number).  It never waits.
 * ot_b200_exchange_gather: one warp polls the `world` entries of slot
 *   step % ring of the caller's OWN table until each carries step + 1, then
 *   *d_out = scale * (sum in rank order).  The poll gives up after max_wait_ns:
 *   *d_error (set it to 0 beforehand) becomes 1 + the rank that did not arrive
 *   (101 + rank: its entry was already overwritten by a step >= step + ring),
 *   *d_out becomes NaN and the kernel returns.
 * d_value / d_out are float, or double with OT_B200_FP64.  world <= 32.
 *
 * ot_b200_exchange_allreduce: publish + gather of one step in ONE call, on a
 *   highest-priority stream the library keeps per device (created on first use):
 *   that stream first waits (by an event) for what `stream` holds so far, i.e.
 *   for *d_value; nothing in `stream` waits for the exchange.  *d_out is defined
 *   once ot_b200_exchange_wait(reader_stream) has made the reader's stream wait
 *   for the most recent all-reduce of the device.  d_value and d_out must stay
 *   valid until then (the Python layer keeps a ring of slots for them). */
int ot_b200_exchange_bytes(int32_t world, int32_t ring, uint64_t *bytes_out);
int ot_b200_exchange_allreduce(const void *d_value, void *d_out, uint32_t flags, void *const *d_tables,
                               const void *d_table, int32_t world, int32_t rank, int32_t ring,
                               uint64_t step, double scale, int32_t *d_error, uint64_t max_wait_ns,
                               void *stream);
int ot_b200_exchange_wait(void *stream);
int ot_b200_exchange_publish(const void *d_value, uint32_t flags, void *const *d_tables,
                             int32_t world, int32_t rank, int32_t ring, uint64_t step,
                             void *stream);
int ot_b200_exchange_gather(const void *d_table, int32_t world, int32_t ring, uint64_t step,
                            void *d_out, uint32_t flags, double scale, int32_t *d_error,
                            uint64_t max_wait_ns, void *stream);

#ifdef __cplusplus
}
#endif
#endif  /* OT_B200_H_ */
