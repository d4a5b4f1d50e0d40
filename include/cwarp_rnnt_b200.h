/*
 * cwarp_rnnt_b200 - C ABI of the B200 (sm_100a) RNN-T loss engine for compact-layout inputs.
 *
 * This is the boundary a binding of the reference project (maxwellzh/CompactWarpRNNTLoss) targets instead of its own
 * CUDA host functions. Plain pointers and sizes only: no torch types, no exceptions. Unless a comment says otherwise,
 * every pointer is a DEVICE pointer valid on the device that is current at the call, every call is asynchronous on
 * `stream`, performs no allocation and no host synchronisation, and returns a cwrnnt_status (0 = launched).
 *
 * Data layout ("compact", reference test/test.py:34-48, cwarp_cuda_gather_kernel.cu:36, cwarp_cuda.cpp:72-77):
 * sequence n owns rows [offset[n], offset[n] + T_n*(U_n+1)) of the row-major [n_rows, V] matrix, rows ordered (t,u)
 * row-major; offset = exclusive prefix sum of T_n*(U_n+1). Labels are a padded row-major int32 [B, y_stride] matrix
 * of which only y[n][u], u < U_n, is read. T_n = lx[n] >= 1, U_n = ly[n] >= 0.
 */
#ifndef CWARP_RNNT_B200_H
#define CWARP_RNNT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CWRNNT_ABI_VERSION 3

#if defined(__GNUC__)
#define CWRNNT_API __attribute__((visibility("default")))
#else
#define CWRNNT_API
#endif

typedef struct CUstream_st *cwrnnt_stream_t; /* same type as cudaStream_t */

typedef enum {
    CWRNNT_F32 = 0,  /* float logits, float costs and gradients                         */
    CWRNNT_F16 = 1,  /* __half logits and gradients, float math and costs               */
    CWRNNT_BF16 = 2, /* __nv_bfloat16 logits and gradients, float math and costs        */
    CWRNNT_F64 = 3   /* double logits, costs and gradients (the reference's other type) */
} cwrnnt_dtype;

typedef enum {
    CWRNNT_OK = 0,
    CWRNNT_ERR_ARGUMENT = 1,   /* null pointer, negative size, blank outside [0,V), unknown dtype or flag */
    CWRNNT_ERR_WORKSPACE = 2,  /* workspace pointer misaligned or smaller than cwrnnt_workspace_bytes()   */
    CWRNNT_ERR_UNSUPPORTED = 3,/* max_u + 1 above CWRNNT_MAX_COLUMNS                                      */
    CWRNNT_ERR_LAUNCH = 4,     /* a CUDA launch or runtime call failed (cudaGetLastError text via cwrnnt_last_error) */
    CWRNNT_ERR_CAPACITY = 5    /* more rows or sequences than cwrnnt_costs_static holds scratch for            */
} cwrnnt_status;

/* Option bits of cwrnnt_problem.flags */
#define CWRNNT_FUSED_LOG_SOFTMAX 0x01 /* x holds raw logits: normalise each row over V inside the op and return dense
                                         gradients w.r.t. the logits. Clear: x holds log-probabilities (the reference
                                         contract) and gradients are zero except the blank and label columns. */
#define CWRNNT_COSTS_ONLY        0x02 /* backward variables only, no state for a backward pass (reference
                                         cwarp_cuda_cal_costs, cwarp_cuda_rnnt_kernel.cu:523-576) */
#define CWRNNT_REDUCE_MEAN       0x04 /* *loss = sum(costs) / mean_denominator; backward scales by the same factor */
#define CWRNNT_REDUCE_SUM        0x08 /* *loss = sum(costs) */
#define CWRNNT_AVERAGE_FRAMES    0x10 /* costs[n] (and its gradient weight) divided by T_n */

#define CWRNNT_MAX_COLUMNS 4096       /* largest supported max_u + 1 */

/* Bits of the device status word 0 (see cwrnnt_read_status) */
#define CWRNNT_ST_BAD_LENGTH   0x01 /* some lx[n] < 1, ly[n] < 0 or ly[n] > max_u: nothing was computed, costs = NaN */
#define CWRNNT_ST_ROW_MISMATCH 0x02 /* sum T_n*(U_n+1) != n_rows: nothing was computed, costs = NaN              */
#define CWRNNT_ST_BAD_LABEL    0x04 /* a label outside [0,V) was read; it was clamped into range                   */
#define CWRNNT_ST_FWD_BWD_GAP  0x08 /* alpha-end and beta-start differ by more than 1e-3 relative for some sequence;
                                       as in the reference (cwarp_cuda_rnnt_kernel.cu:356-364) their mean was used */
#define CWRNNT_ST_FATAL (CWRNNT_ST_BAD_LENGTH | CWRNNT_ST_ROW_MISMATCH)

typedef struct {
    int64_t n_rows;           /* rows of x: must equal sum_n lx[n]*(ly[n]+1) (checked on the device)      */
    int32_t V;                /* vocabulary size = columns of x                                           */
    int32_t B;                /* number of sequences                                                      */
    int32_t y_stride;         /* row stride (elements) of the padded label matrix, >= max_u               */
    int32_t max_u;            /* upper bound of ly[n]; the reference uses y.size(1) (cwarp_rnnt/__init__.py:49) */
    int32_t blank;            /* blank index, 0 <= blank < V (cwarp_rnnt/__init__.py:50)                  */
    int32_t dtype;            /* cwrnnt_dtype                                                             */
    int32_t flags;            /* CWRNNT_* option bits                                                     */
    int32_t mean_denominator; /* divisor of CWRNNT_REDUCE_MEAN; 0 means B. Sharded runs pass the global B. */
} cwrnnt_problem;

/* Library identity; replaces nothing in the reference (which exports no version from its extension). */
CWRNNT_API int cwrnnt_abi_version(void);

/* Text of a cwrnnt_status, and the CUDA error text recorded by the last CWRNNT_ERR_LAUNCH on this thread. */
CWRNNT_API const char *cwrnnt_status_string(int status);
CWRNNT_API const char *cwrnnt_last_error(void);

/*
 * Bytes of device workspace cwrnnt_forward needs for this problem (depends on n_rows and B only); < 0 on bad
 * arguments. Replaces the reference's internal allocations: alphas/betas [N,Tmax,Umax+1], grads, costs, locks
 * (cwarp_cuda_rnnt_kernel.cu:399-404), the gathered [STU,2] matrix (cwarp_cuda_gather_kernel.cu:87) and the offset
 * tensors (cwarp_cuda.cpp:98-103). The workspace must be 256-byte aligned. It carries the state that
 * cwrnnt_backward, cwrnnt_pair_grads and cwrnnt_export_alpha_beta read, so keep it until those have run.
 */
CWRNNT_API int64_t cwrnnt_workspace_bytes(const cwrnnt_problem *p);

/*
 * Forward: costs[n] = -log P(y_n | x_n), optionally the reduced loss.
 * Replaces compact_rnnt_loss_forward (cwarp_cuda.cpp:84-108 = gather_cuda_forward + cwarp_cuda_costs_with_grad)
 * and, with CWRNNT_COSTS_ONLY, compact_rnnt_loss (cwarp_cuda.cpp:58-82). With CWRNNT_FUSED_LOG_SOFTMAX it also
 * replaces the caller's log_softmax (test/test.py:19-20).
 *   x      [n_rows, V] logits or log-probs in p->dtype (row start must be 16-byte aligned for the vector path;
 *          other shapes take a scalar path)
 *   lx, ly [B] int32;  y [B, y_stride] int32
 *   costs  [B] float (double for CWRNNT_F64), written
 *   loss   1 element of the costs type or NULL; written when a CWRNNT_REDUCE_* flag is set
 */
CWRNNT_API int cwrnnt_forward(const cwrnnt_problem *p, const void *x, const int32_t *lx, const int32_t *ly, const int32_t *y,
                   void *workspace, int64_t workspace_bytes, void *costs, void *loss, cwrnnt_stream_t stream);

/*
 * Forward of one shard of a batch that is split across GPUs by whole sequences (one process per GPU). As
 * cwrnnt_forward, and in addition the kernel's epilogue fills `cost_vector` [n_global + 1] (costs type): zero
 * everywhere except cost_vector[global_ids[n]] = costs[n] for this rank's sequences and cost_vector[n_global] = this
 * rank's loss contribution (sum of its costs, divided by mean_denominator under CWRNNT_REDUCE_MEAN). One
 * all-reduce(sum) of that vector over the ranks then leaves every sequence's cost and the global loss on every rank.
 * global_ids NULL means the identity. No counterpart in the reference, which is single-GPU (no device guard, no
 * collective anywhere in its tree).
 */
CWRNNT_API int cwrnnt_forward_sharded(const cwrnnt_problem *p, const void *x, const int32_t *lx, const int32_t *ly,
                                      const int32_t *y, void *workspace, int64_t workspace_bytes, void *costs,
                                      void *loss, const int32_t *global_ids, int32_t n_global, void *cost_vector,
                                      cwrnnt_stream_t stream);

/*
 * The alpha/beta recursion and the cost step by themselves, on a workspace that cwrnnt_forward (or cwrnnt_loss_grad)
 * has already filled for the same problem and the same lx / ly: the gathered log-probabilities and the row offsets are
 * taken as they stand, alpha, beta, costs and loss are recomputed. The counterpart of cwarp_cuda_costs_with_grad and,
 * with CWRNNT_COSTS_ONLY, cwarp_cuda_cal_costs (cwarp_cuda_rnnt_kernel.cu:386-497, :523-576), which likewise start
 * from gathered log-probabilities. Its duration divided by the longest T_n + U_n of the batch is the recursion's
 * latency per lattice diagonal, the figure this stage is measured by.
 */
CWRNNT_API int cwrnnt_recursion(const cwrnnt_problem *p, const int32_t *lx, const int32_t *ly, void *workspace,
                                int64_t workspace_bytes, void *costs, void *loss, cwrnnt_stream_t stream);

/*
 * Backward: grad_x[r][k] = d (sum_n g_n * costs[n]) / d x[r][k] in one streaming pass over [n_rows, V].
 * Replaces compact_rnnt_loss_backward_ (cwarp_cuda.cpp:110-136 = cwarp_cuda_backward_ + zeros[STU,V] +
 * gather_cuda_backward_) and, with CWRNNT_FUSED_LOG_SOFTMAX, the caller's log_softmax backward as well.
 *   workspace          as left by cwrnnt_forward on the same problem (not modified)
 *   grad_costs         costs type; element n*grad_costs_stride is g_n (stride 0 broadcasts one scalar, e.g. the
 *                      gradient of the reduced loss; the CWRNNT_REDUCE_MEAN / AVERAGE_FRAMES factors are applied
 *                      inside). NULL means g_n = 1.
 *   grad_x             [n_rows, V] in p->dtype, fully written (no pre-zeroing needed)
 * Unlike the reference (cwarp_cuda_rnnt_kernel.cu:518-520) nothing saved by the forward is modified, so the call can
 * be repeated. When a label equals `blank` the two terms add (the reference scatter overwrites one of them,
 * cwarp_cuda_gather_kernel.cu:70-73).
 */
CWRNNT_API int cwrnnt_backward(const cwrnnt_problem *p, const void *x, const int32_t *lx, const int32_t *ly, const int32_t *y,
                    const void *workspace, const void *grad_costs, int32_t grad_costs_stride, void *grad_x,
                    cwrnnt_stream_t stream);

/*
 * One training step in one call: costs, loss AND the gradient, as a software pipeline over groups of sequences.
 * Replaces what the reference's autograd forward already does in one go - _cwarp_rnnt_forward computes the gradients
 * during the forward call and backward only scales them (cwarp_rnnt/__init__.py:10-29, cwarp_cuda.cpp:84-136) - and,
 * with CWRNNT_FUSED_LOG_SOFTMAX, the caller's log_softmax forward and backward.
 * The rows are cut into `groups` ranges; group g = the sequences whose last row lies in range g. On the caller's
 * stream and one more stream of the pipe, alternating: K0, then the gather of range 0..G-1. On the pipe's
 * high-priority side stream g: the alpha/beta wavefront of group g as soon as ranges 0..g are gathered. The gradient
 * of group g follows its wavefront - in group order on the two gather streams for batches of narrow lattices, on side
 * stream g itself (so in the order in which the wavefronts finish, at the lowest launch priority) when max_u + 1 > 256
 * or B <= 8, where one wavefront can outlast a pass. The wavefront (a chain of T+U dependent steps on a few SMs)
 * thereby runs underneath the two bandwidth-bound passes instead of between them. The step uses 2 + G streams, few
 * enough for the device's hardware queues. Everything is joined back into `stream` before the call returns
 * (event waits, nothing blocks the host), so results are ordered on `stream` exactly like those of cwrnnt_forward +
 * cwrnnt_backward; they are bit-identical to that pair's. Rows laid out with the longest T+U first start the longest
 * chains first (sharding.plan_shards does that for a shard).
 *   pipe        side streams and events, from cwrnnt_pipe_create on the same device; one call at a time per pipe.
 *               NULL runs the same work on `stream` alone without overlap.
 *   grad_costs / grad_costs_stride / grad_x   as cwrnnt_backward (NULL grad_costs: upstream gradient 1)
 *   global_ids / n_global / cost_vector       as cwrnnt_forward_sharded, or NULL / 0 / NULL
 *   groups      0 = chosen from the size of x (one group, i.e. no overlap, below 256 MB of logits); 1..8 to force
 * CWRNNT_COSTS_ONLY is refused (use cwrnnt_forward). The workspace ends up in the same state as after
 * cwrnnt_forward, so cwrnnt_backward / cwrnnt_pair_grads / cwrnnt_export_alpha_beta may follow.
 */
typedef struct cwrnnt_pipe cwrnnt_pipe;
CWRNNT_API int cwrnnt_pipe_create(cwrnnt_pipe **pipe);
CWRNNT_API void cwrnnt_pipe_destroy(cwrnnt_pipe *pipe);
/*
 * Tracing of a pipelined step. A pipe from cwrnnt_pipe_create_traced records its events with timestamps (a pipe from
 * cwrnnt_pipe_create does not: untimed events are cheaper). After the stream of the last cwrnnt_loss_grad has been
 * synchronised, cwrnnt_pipe_timeline writes, for every sequence group g of that step, three times in milliseconds
 * since the step's fork point (right after the row-offset kernel): ms[3g] = range g gathered, ms[3g+1] = wavefront of
 * group g done, ms[3g+2] = gradient of group g done (-1 where an event is not available). Returns the number of
 * groups (0 for an ungrouped step, which records nothing), or -1 on a bad argument, an untraced pipe or capacity
 * below 3 * groups. The reference has no tracing (its only diagnostic is a device printf,
 * cwarp_cuda_rnnt_kernel.cu:361).
 */
CWRNNT_API int cwrnnt_pipe_create_traced(cwrnnt_pipe **pipe);
CWRNNT_API int cwrnnt_pipe_timeline(cwrnnt_pipe *pipe, float *ms, int32_t capacity);
CWRNNT_API int cwrnnt_loss_grad(cwrnnt_pipe *pipe, const cwrnnt_problem *p, const void *x, const int32_t *lx,
                                const int32_t *ly, const int32_t *y, void *workspace, int64_t workspace_bytes,
                                void *costs, void *loss, const void *grad_costs, int32_t grad_costs_stride,
                                void *grad_x, const int32_t *global_ids, int32_t n_global, void *cost_vector,
                                int32_t groups, cwrnnt_stream_t stream);

/*
 * Makes `stream` wait until the costs, the loss and the cost vector of the last cwrnnt_loss_grad issued through
 * `pipe` are written - which is before its gradient kernels are done. A sharded caller puts its all-reduce of the cost
 * vector on a second stream behind this wait, so the collective runs underneath the gradient pass instead of after
 * it. No counterpart in the reference (single GPU).
 */
CWRNNT_API int cwrnnt_pipe_wait_costs(cwrnnt_pipe *pipe, cwrnnt_stream_t stream);

/* Number of sequence groups cwrnnt_loss_grad uses for this problem and `groups` argument (with a pipe); < 0 on bad
 * arguments. A step then launches 1 + 3 * groups kernels. No counterpart in the reference. */
CWRNNT_API int32_t cwrnnt_pipeline_groups(const cwrnnt_problem *p, int32_t groups);

/*
 * grad_x *= *factor in place; `factor` is one device scalar of the costs type. For a gradient that cwrnnt_loss_grad
 * computed for an upstream gradient of 1 before the real one was known (autograd's backward arrives later): replaces
 * the scaling step of the reference's backward (cwarp_cuda_rnnt_kernel.cu:512-521). When the factor is 1 - the usual
 * case for a training loss - the kernel returns before touching grad_x.
 */
CWRNNT_API int cwrnnt_scale_grad(const cwrnnt_problem *p, void *grad_x, const void *factor, cwrnnt_stream_t stream);

/*
 * The reference's intermediate results in the reference's own shapes, for callers of its extension module
 * (cwarp_cuda.cpp:140-143 returns (costs, grads[STU,2], alphas[N,Tmax,Umax+1], betas[N,Tmax,Umax+1])).
 * cwrnnt_pair_grads: grads[r] = (d cost/d lp_blank, d cost/d lp_label) = (-occupancy) as in
 * cwarp_cuda_rnnt_kernel.cu:296-307 and :325-331; costs type, [n_rows, 2], fully written.
 * cwrnnt_export_alpha_beta: zero-padded [B, t_max, u_max1] arrays of the costs type (cwarp_cuda_rnnt_kernel.cu:399-400);
 * either pointer may be NULL.
 */
CWRNNT_API int cwrnnt_pair_grads(const cwrnnt_problem *p, const void *x, const int32_t *lx, const int32_t *ly, const int32_t *y,
                      const void *workspace, void *grads, cwrnnt_stream_t stream);
CWRNNT_API int cwrnnt_export_alpha_beta(const cwrnnt_problem *p, const int32_t *lx, const int32_t *ly, const void *workspace,
                             int32_t t_max, int32_t u_max1, void *alphas, void *betas, cwrnnt_stream_t stream);

/*
 * What the reference leaves to the caller of its alpha / beta outputs (cwarp_cuda_rnnt_kernel.cu:383-384 "for
 * debugging or analysis", returned at :496), computed from the state cwrnnt_forward left in the workspace:
 * cwrnnt_export_alignment: the most probable alignment of every sequence - the alpha recursion (:105-125) with max in
 *   place of log-sum-exp, then a walk back from (T-1,U). moves [B, path_stride] int32: moves[n][k], k < T_n+U_n, is 0
 *   for a blank move (next frame) and 1 for a label move (next label), the last one being the final blank; -1 beyond
 *   (path_stride >= max_n T_n+U_n, shorter rows are truncated at the front). Equal scores go to the blank move.
 *   scores [B] (costs type): log-probability of that path. scratch: cwrnnt_alignment_scratch_bytes(p) bytes (one per
 *   lattice node). Works after a CWRNNT_COSTS_ONLY forward too (it reads the gathered log-probabilities only).
 * cwrnnt_export_posteriors: exp(alpha(t,u) + beta(t,u) - log P(y|x)), the probability that the alignment passes
 *   through node (t,u), zero-padded [B, t_max, u_max1] of the costs type like the alpha / beta export; the entries of
 *   every anti-diagonal t+u = d of a sequence add up to one.
 */
CWRNNT_API int64_t cwrnnt_alignment_scratch_bytes(const cwrnnt_problem *p);
CWRNNT_API int cwrnnt_export_alignment(const cwrnnt_problem *p, const int32_t *lx, const int32_t *ly,
                                       const void *workspace, void *scratch, int64_t scratch_bytes,
                                       int32_t path_stride, int32_t *moves, void *scores, cwrnnt_stream_t stream);
CWRNNT_API int cwrnnt_export_posteriors(const cwrnnt_problem *p, const int32_t *lx, const int32_t *ly,
                                        const void *workspace, int32_t t_max, int32_t u_max1, void *posteriors,
                                        cwrnnt_stream_t stream);

/*
 * The cost step by itself: costs[n] = -ll[n] (divided by T_n under CWRNNT_AVERAGE_FRAMES) from per-sequence
 * log-likelihoods held in DEVICE double arrays - ll_alpha[n] = alpha(T-1,U) + the final blank, ll_beta[n] = beta(0,0).
 * Replaces fill_cost_kernel (cwarp_cuda_rnnt_kernel.cu:334-367) including its consistency guard: where the two differ
 * by more than 1e-3 relative, their mean is used and CWRNNT_ST_FWD_BWD_GAP is OR-ed into the DEVICE word *status (the
 * reference prints from the device instead, :361). ll_alpha NULL: no guard, as in the costs-only path (:575). Only B,
 * dtype (type of costs) and the CWRNNT_AVERAGE_FRAMES flag of `p` are used. cwrnnt_forward runs the same step inside
 * the wavefront kernel's epilogue; this entry serves callers that hold alpha/beta from elsewhere, and the tests of
 * the guard.
 */
CWRNNT_API int cwrnnt_fill_costs(const cwrnnt_problem *p, const int32_t *lx, const double *ll_alpha,
                                 const double *ll_beta, void *costs, int32_t *status, cwrnnt_stream_t stream);

/*
 * Reference-shaped backward from saved pair gradients: dense[r][blank] = grads[r][0]*g_n, dense[r][y] =
 * grads[r][1]*g_n, zero elsewhere. Replaces cwarp_cuda_backward_ + torch::zeros + gather_cuda_backward_
 * (cwarp_cuda_rnnt_kernel.cu:512-521, cwarp_cuda.cpp:131-135, cwarp_cuda_gather_kernel.cu:52-74) without mutating
 * `grads`. `scratch` needs cwrnnt_scatter_scratch_bytes(B) bytes (offsets are recomputed as cwarp_cuda.cpp:124-129).
 * p->dtype is the type of grads, grad_costs and dense (CWRNNT_F32 or CWRNNT_F64).
 */
CWRNNT_API int64_t cwrnnt_scatter_scratch_bytes(int32_t B);
CWRNNT_API int cwrnnt_scatter_backward(const cwrnnt_problem *p, const void *grads, const void *grad_costs, const int32_t *lx,
                            const int32_t *ly, const int32_t *y, void *scratch, int64_t scratch_bytes, void *dense,
                            cwrnnt_stream_t stream);

/*
 * Padded joint output [B, t_max, u_max1, V] -> compact [n_rows, V] and its transpose for the gradient (which also
 * zero-fills the padding). Replaces the reference's 4-D convenience path, gather.cat on the flattened [T*(U+1)] axis
 * (cwarp_rnnt/__init__.py:52-59) - with the per-sequence slicing its own test defines, x[n, :T_n, :U_n+1, :]
 * (test/test.py:45-46); the reference's version is only right when every U_n equals Umax. p supplies n_rows, V, B,
 * dtype and max_u (<= u_max1 - 1); `scratch` needs cwrnnt_scatter_scratch_bytes(B) bytes. When sum T_n*(U_n+1)
 * differs from n_rows the pack leaves `compact` untouched and the unpack writes zeros only.
 */
CWRNNT_API int cwrnnt_pack_padded(const cwrnnt_problem *p, const void *padded, int32_t t_max, int32_t u_max1,
                                  const int32_t *lx, const int32_t *ly, void *scratch, int64_t scratch_bytes,
                                  void *compact, cwrnnt_stream_t stream);
CWRNNT_API int cwrnnt_unpack_padded(const cwrnnt_problem *p, const void *compact, int32_t t_max, int32_t u_max1,
                                    const int32_t *lx, const int32_t *ly, void *scratch, int64_t scratch_bytes,
                                    void *padded, cwrnnt_stream_t stream);

/*
 * Copies the 4 int32 status words of a workspace to HOST memory `out` and waits for the stream (the one call here
 * that synchronises). out[0] = CWRNNT_ST_* bits, out[1] = first offending sequence (-1 if none), out[2] = computed
 * sum of T_n*(U_n+1) (low 31 bits), out[3] = reserved. Replaces the reference's device printf warning
 * (cwarp_cuda_rnnt_kernel.cu:361) and adds the checks it lacks.
 */
CWRNNT_API int cwrnnt_read_status(const void *workspace, int32_t out[4], cwrnnt_stream_t stream);

/*
 * Input validation by itself, ahead of the heavy kernels: one small kernel over lx, ly and y, four words copied to
 * HOST memory `out`, one wait on the stream (about 20 us). out[0] = CWRNNT_ST_BAD_LENGTH / ROW_MISMATCH / BAD_LABEL
 * bits, out[1] = first sequence with an invalid length (-1 if none), out[2] = max_n lx[n], out[3] = max_n ly[n].
 * Covers the reference's host-side assertions that read device data (`y.size(1) == ly.max()`, `lx.max() == T`,
 * cwarp_rnnt/__init__.py:49,58) and the checks it lacks, without waiting for the loss itself: a caller that validates
 * first can then launch cwrnnt_forward / cwrnnt_loss_grad and never synchronise. `scratch`: 16 bytes of device
 * memory, 4-byte aligned.
 */
CWRNNT_API int cwrnnt_validate(const cwrnnt_problem *p, const int32_t *lx, const int32_t *ly, const int32_t *y,
                               void *scratch, int32_t out[4], cwrnnt_stream_t stream);

/*
 * The same validation without the wait: the kernel and the 16-byte copy into HOST memory `out` are queued on `stream`
 * and the call returns. The caller queues the loss kernels behind it (they protect themselves: invalid lengths make
 * them return without touching the inputs, labels are clamped), and only then waits - on an event recorded right
 * after this call, or on the stream - before reading `out` and raising. The GPU therefore never idles for the
 * validation round trip, and the reference's host-side assertions (cwarp_rnnt/__init__.py:49,58) still fire before a
 * loss is handed back. `out` should be pinned memory (a pageable buffer makes the copy synchronous) and, like
 * `scratch`, must stay valid until the stream has passed this point. With B == 0 `out` is written at once.
 */
CWRNNT_API int cwrnnt_validate_async(const cwrnnt_problem *p, const int32_t *lx, const int32_t *ly, const int32_t *y,
                                     void *scratch, int32_t out[4], cwrnnt_stream_t stream);

/*
 * The joint network's broadcast-add written straight into the compact layout - the producer in front of the loss:
 *     out[off_n + t*(U_n+1) + u][:] = act(enc[n][t][:] + pred[n][u][:])
 * from the padded encoder output enc [B, t_max, H] and predictor output pred [B, u_max1, H] (p->dtype; H = p->V,
 * p->n_rows = sum_n lx[n]*(ly[n]+1); blank and flags of `p` are not used). The reference has no such function: its
 * callers build the padded [N, T, U+1, H] joint tensor and compact that (test/test.py:34-48 defines the layout,
 * cwarp_rnnt/__init__.py:52-59 compacts a padded 4-D input); here the padding is never materialised. A linear layer
 * (a library GEMM) maps out [n_rows, H] to the logits [n_rows, V] that cwrnnt_forward / cwrnnt_loss_grad take.
 * cwrnnt_joint_backward: grad_enc[n][t] = sum_u g*act', grad_pred[n][u] = sum_t g*act' with g = grad_out
 * [n_rows, H]; both outputs are fully written (zero in the padding); deterministic summation order.
 * scratch: cwrnnt_scatter_scratch_bytes(B) bytes, 8-byte aligned. Lengths that disagree with n_rows leave the forward
 * output untouched and give zero gradients.
 */
#define CWRNNT_ACT_NONE 0
#define CWRNNT_ACT_RELU 1
#define CWRNNT_ACT_TANH 2
CWRNNT_API int cwrnnt_joint_forward(const cwrnnt_problem *p, int32_t activation, const void *enc, int32_t t_max,
                                    const void *pred, int32_t u_max1, const int32_t *lx, const int32_t *ly,
                                    void *scratch, int64_t scratch_bytes, void *out, cwrnnt_stream_t stream);
CWRNNT_API int cwrnnt_joint_backward(const cwrnnt_problem *p, int32_t activation, const void *enc, int32_t t_max,
                                     const void *pred, int32_t u_max1, const int32_t *lx, const int32_t *ly,
                                     const void *grad_out, void *scratch, int64_t scratch_bytes, void *grad_enc,
                                     void *grad_pred, cwrnnt_stream_t stream);

/*
 * Costs (and the reduced loss) without any caller workspace and without any allocation: for hosts that cannot call
 * cudaMalloc - a plug-in in a serving process whose framework owns all device memory, a foreign-language binding with
 * no device allocator to size a workspace with, a scoring loop that cannot afford the synchronisation an allocation
 * implies. No counterpart in the reference (which allocates five tensors per call, cwarp_cuda_rnnt_kernel.cu:535-537,
 * cwarp_cuda_gather_kernel.cu:87). Same arguments and results as cwrnnt_forward with CWRNNT_COSTS_ONLY (the flag is
 * implied); the scratch is a fixed device array inside the library (about 5.3 MB, held by every GPU that loads the
 * library until the process exits), so:
 *   - problems above CWRNNT_STATIC_MAX_ROWS rows or CWRNNT_STATIC_MAX_SEQUENCES sequences are refused with
 *     CWRNNT_ERR_CAPACITY before anything is launched;
 *   - the first call on each device resolves the array's device address (cudaGetSymbolAddress); make that first call
 *     outside any stream capture;
 *   - all calls on a device share the one array and it keeps the previous call's contents (the words that must start
 *     at zero are cleared at the start of every call): two calls that overlap on the GPU - different streams, or
 *     different host threads - race. Serialise them on one stream;
 *   - there is no backward for this entry point (nothing is kept for it).
 * It calls no cudaMalloc, cudaFree or allocating library routine.
 */
#define CWRNNT_STATIC_MAX_ROWS 131072
#define CWRNNT_STATIC_MAX_SEQUENCES 1024
CWRNNT_API int cwrnnt_costs_static(const cwrnnt_problem *p, const void *x, const int32_t *lx, const int32_t *ly,
                                   const int32_t *y, void *costs, void *loss, cwrnnt_stream_t stream);
/*
 * Status words of the last cwrnnt_costs_static on the current device, as cwrnnt_read_status returns them for a
 * caller-owned workspace (the built-in scratch cannot be handed to that function): 16 bytes copied to HOST memory
 * `out`, one wait on `stream`, nothing allocated. Without it a clamped label (CWRNNT_ST_BAD_LABEL) would go unseen
 * and invalid lengths would show only as NaN costs. No counterpart in the reference.
 */
CWRNNT_API int cwrnnt_static_status(int32_t out[4], cwrnnt_stream_t stream);

/*
 * Host-buffer pipeline: logits, lengths and labels in HOST memory (pinned for overlap), costs / loss / gradients
 * back in HOST memory. Sequences are cut into chunks; upload, kernels and download of successive chunks overlap on
 * three streams. This is the call to bind where the caller's tensors live on the host. It owns its device buffers
 * inside an opaque context (created once per device; capacity grows on demand), synchronises before returning, and
 * is not thread-safe per context. No counterpart in the reference, which accepts CUDA tensors only
 * (cwarp_cuda.cpp:46-52).
 *   grad_x_host may be NULL (costs only). grad_costs_host: HOST array as in cwrnnt_backward or NULL.
 *   chunk_rows: target rows per chunk (0 = default).
 */
typedef struct cwrnnt_host_ctx cwrnnt_host_ctx;
CWRNNT_API int cwrnnt_host_ctx_create(cwrnnt_host_ctx **ctx);
CWRNNT_API void cwrnnt_host_ctx_destroy(cwrnnt_host_ctx *ctx);
CWRNNT_API const char *cwrnnt_host_ctx_error(const cwrnnt_host_ctx *ctx); /* CUDA error text of the last failing call */
CWRNNT_API int cwrnnt_loss_grad_host(cwrnnt_host_ctx *ctx, const cwrnnt_problem *p, const void *x_host, const int32_t *lx_host,
                          const int32_t *ly_host, const int32_t *y_host, const void *grad_costs_host,
                          int32_t grad_costs_stride, void *costs_host, void *loss_host, void *grad_x_host,
                          int64_t chunk_rows, int32_t status_out[4]);

#ifdef __cplusplus
}
#endif
#endif /* CWARP_RNNT_B200_H */
