// C ABI of the engine (include/cwarp_rnnt_b200.h): argument checks, workspace carving, kernel sequencing.
// No device allocation, no synchronisation (except cwrnnt_read_status and cwrnnt_validate), no exceptions; cwrnnt_pipe_create owns the
// only resources made here (side streams and events).
#include <cstdio>
#include <cstring>
#include <new>

#include "cwrnnt_kernels.h"

using namespace cwrnnt;

// Side streams and events of a pipelined step (cwrnnt_loss_grad).
struct cwrnnt_pipe {
    int device;
    cudaStream_t alt;                  // streaming kernels of the odd groups (even ones: the caller's stream)
    cudaStream_t side[kMaxGroups];     // highest priority: the wavefront of group g, then its gradient
    cudaEvent_t gathered[kMaxGroups];  // recorded after the gather of range g
    cudaEvent_t solved[kMaxGroups];    // recorded on side[g] after the wavefront of group g
    cudaEvent_t graded[kMaxGroups];    // recorded on side[g] after the gradient of group g
    cudaEvent_t forked, joined;        // caller's stream -> alt at the start, alt -> caller's stream at the end
    cudaEvent_t costs_ready;           // every wavefront of the last step is done: costs, loss, cost vector written
    bool traced;                       // events carry timestamps (cwrnnt_pipe_create_traced): cwrnnt_pipe_timeline works
    int last_groups;                   // group count of the last step issued through this pipe
};

namespace {

int64_t elt_bytes(int dtype) { return dtype == CWRNNT_F32 ? 4 : (dtype == CWRNNT_F64 ? 8 : 2); }

thread_local char g_last_error[256] = "";

// Sequence groups of a pipelined step. Enough of them that the first wavefront starts early and the last one has
// gradient work to hide under, few enough that the streaming launches stay large (each ends in a partly filled wave).
GroupPlan plan_groups(const cwrnnt_problem &p, int groups)
{
    const int64_t bytes = p.n_rows * int64_t(p.V) * elt_bytes(p.dtype);
    // measured on B200: 4 groups for a large batch of ordinary sequences (32 x [200 x 50] x 1024 fp32: 0.592 ms against
    // 0.628 unpipelined, 0.607 with 2, 0.609 with 8); 8 when the batch is a handful of long sequences, whose
    // wavefronts are the critical path (4 x [1250 x 300] x 512: 1.48 ms against 1.85, 1.64 with 4)
    const int large = p.B <= 8 ? 8 : 4;
    // below 256 MB no grouping: the wavefront chain is then the critical path, and it runs slower next to the
    // streaming kernels than alone (230 MB of ragged rows: 0.416 ms with two groups against 0.379 ms with one)
    const int by_size = bytes >= (int64_t(256) << 20) ? large : 1;
    const int want = groups > 0 ? groups : by_size;
    const int64_t kAlign = 512;  // whole tiles of every row shape of the streaming kernels (at most 64 runs of 8 rows)
    GroupPlan plan{1, p.n_rows > 0 ? p.n_rows : 1};
    if (want > 1 && p.n_rows > kAlign) {
        plan.range_rows = align_up((p.n_rows + want - 1) / want, kAlign);
        plan.count = int((p.n_rows + plan.range_rows - 1) / plan.range_rows);
    }
    return plan;
}

int fail_launch(const char *what, cudaError_t e)
{
    std::snprintf(g_last_error, sizeof g_last_error, "%s: %s", what, cudaGetErrorString(e));
    return CWRNNT_ERR_LAUNCH;
}

int check_problem(const cwrnnt_problem *p)
{
    if (!p) return CWRNNT_ERR_ARGUMENT;
    if (p->n_rows < 0 || p->V < 1 || p->B < 0 || p->max_u < 0 || p->y_stride < p->max_u) return CWRNNT_ERR_ARGUMENT;
    if (p->blank < 0 || p->blank >= p->V) return CWRNNT_ERR_ARGUMENT;
    if (p->dtype < CWRNNT_F32 || p->dtype > CWRNNT_F64) return CWRNNT_ERR_ARGUMENT;
    if (p->mean_denominator < 0) return CWRNNT_ERR_ARGUMENT;
    const int known = CWRNNT_FUSED_LOG_SOFTMAX | CWRNNT_COSTS_ONLY | CWRNNT_REDUCE_MEAN | CWRNNT_REDUCE_SUM |
                      CWRNNT_AVERAGE_FRAMES;
    if (p->flags & ~known) return CWRNNT_ERR_ARGUMENT;
    if ((p->flags & CWRNNT_REDUCE_MEAN) && (p->flags & CWRNNT_REDUCE_SUM)) return CWRNNT_ERR_ARGUMENT;
    if (p->max_u + 1 > CWRNNT_MAX_COLUMNS) return CWRNNT_ERR_UNSUPPORTED;
    return CWRNNT_OK;
}

int check_workspace(const cwrnnt_problem *p, const void *ws, int64_t bytes, Workspace *w)
{
    if (!ws || reinterpret_cast<uintptr_t>(ws) % 256 != 0) return CWRNNT_ERR_WORKSPACE;
    const int64_t need = carve_workspace(p->n_rows, p->B, const_cast<void *>(ws), w);
    if (bytes >= 0 && bytes < need) return CWRNNT_ERR_WORKSPACE;
    return CWRNNT_OK;
}

}  // namespace

void cwrnnt::set_last_error(const char *text) { std::snprintf(g_last_error, sizeof g_last_error, "%s", text); }

extern "C" {

int cwrnnt_abi_version(void) { return CWRNNT_ABI_VERSION; }

const char *cwrnnt_status_string(int status)
{
    switch (status) {
    case CWRNNT_OK: return "ok";
    case CWRNNT_ERR_ARGUMENT: return "invalid argument";
    case CWRNNT_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case CWRNNT_ERR_UNSUPPORTED: return "label length above the supported maximum";
    case CWRNNT_ERR_LAUNCH: return "CUDA launch or runtime failure";
    case CWRNNT_ERR_CAPACITY: return "problem larger than the fixed capacity of this entry point";
    }
    return "unknown status";
}

const char *cwrnnt_last_error(void) { return g_last_error; }

int64_t cwrnnt_workspace_bytes(const cwrnnt_problem *p)
{
    if (check_problem(p) != CWRNNT_OK) return -1;
    return carve_workspace(p->n_rows, p->B, nullptr, nullptr);
}

static int forward_impl(const cwrnnt_problem *p, const void *x, const int32_t *lx, const int32_t *ly, const int32_t *y,
                        void *workspace, int64_t workspace_bytes, void *costs, void *loss, const ShardOutput *shard,
                        cwrnnt_stream_t stream)
{
    int st = check_problem(p);
    if (st) return st;
    if (p->B == 0) return CWRNNT_OK;  // an empty batch: nothing to read, nothing to write
    if (!lx || !ly || !costs || (p->n_rows > 0 && !x) || (p->max_u > 0 && !y)) return CWRNNT_ERR_ARGUMENT;
    Workspace w{};
    st = check_workspace(p, workspace, workspace_bytes, &w);
    if (st) return st;
    if (p->B == 0) return CWRNNT_OK;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    cudaError_t e;
    e = launch_prep(*p, lx, ly, w, costs, s, GroupPlan{1, 1}, loss, shard ? shard->cost_vector : nullptr,
                    shard ? shard->n_global : 0);
    if (e != cudaSuccess) return fail_launch("prep", e);
    if ((e = launch_gather(*p, x, lx, ly, y, w, s)) != cudaSuccess) return fail_launch("gather", e);
    if ((e = launch_wavefront(*p, lx, ly, w, costs, loss, shard, s)) != cudaSuccess) return fail_launch("wavefront", e);
    return CWRNNT_OK;
}

int cwrnnt_forward(const cwrnnt_problem *p, const void *x, const int32_t *lx, const int32_t *ly, const int32_t *y,
                   void *workspace, int64_t workspace_bytes, void *costs, void *loss, cwrnnt_stream_t stream)
{
    return forward_impl(p, x, lx, ly, y, workspace, workspace_bytes, costs, loss, nullptr, stream);
}

int cwrnnt_forward_sharded(const cwrnnt_problem *p, const void *x, const int32_t *lx, const int32_t *ly,
                           const int32_t *y, void *workspace, int64_t workspace_bytes, void *costs, void *loss,
                           const int32_t *global_ids, int32_t n_global, void *cost_vector, cwrnnt_stream_t stream)
{
    if (!p || !cost_vector || n_global < p->B) return CWRNNT_ERR_ARGUMENT;
    ShardOutput shard{global_ids, n_global, cost_vector};
    return forward_impl(p, x, lx, ly, y, workspace, workspace_bytes, costs, loss, &shard, stream);
}

int cwrnnt_recursion(const cwrnnt_problem *p, const int32_t *lx, const int32_t *ly, void *workspace,
                     int64_t workspace_bytes, void *costs, void *loss, cwrnnt_stream_t stream)
{
    int st = check_problem(p);
    if (st) return st;
    if (p->B == 0) return CWRNNT_OK;
    if (!lx || !ly || !costs) return CWRNNT_ERR_ARGUMENT;
    Workspace w{};
    st = check_workspace(p, workspace, workspace_bytes, &w);
    if (st) return st;
    cudaError_t e = launch_wavefront(*p, lx, ly, w, costs, loss, nullptr, reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? CWRNNT_OK : fail_launch("wavefront", e);
}

int cwrnnt_backward(const cwrnnt_problem *p, const void *x, const int32_t *lx, const int32_t *ly, const int32_t *y,
                    const void *workspace, const void *grad_costs, int32_t grad_costs_stride, void *grad_x,
                    cwrnnt_stream_t stream)
{
    int st = check_problem(p);
    if (st) return st;
    if (p->flags & CWRNNT_COSTS_ONLY) return CWRNNT_ERR_ARGUMENT;  // that forward kept no alpha
    if (p->B == 0) return CWRNNT_OK;
    if (!lx || !ly || (p->n_rows > 0 && (!x || !grad_x)) || (p->max_u > 0 && !y)) return CWRNNT_ERR_ARGUMENT;
    if (grad_costs_stride != 0 && grad_costs_stride != 1) return CWRNNT_ERR_ARGUMENT;
    Workspace w{};
    st = check_workspace(p, workspace, -1, &w);
    if (st) return st;
    if (p->B == 0) return CWRNNT_OK;
    cudaError_t e = launch_grad(*p, x, lx, ly, y, w, grad_costs, grad_costs_stride, grad_x,
                                reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? CWRNNT_OK : fail_launch("grad", e);
}

static int pipe_create(cwrnnt_pipe **out, bool traced)
{
    if (!out) return CWRNNT_ERR_ARGUMENT;
    *out = nullptr;
    cwrnnt_pipe *pipe = new (std::nothrow) cwrnnt_pipe{};
    if (!pipe) return CWRNNT_ERR_LAUNCH;
    pipe->traced = traced;
    const unsigned ev_flags = traced ? cudaEventDefault : cudaEventDisableTiming;  // timestamps only when traced
    int least = 0, greatest = 0;
    cudaError_t e = cudaGetDevice(&pipe->device);
    if (e == cudaSuccess) e = cudaDeviceGetStreamPriorityRange(&least, &greatest);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&pipe->alt, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&pipe->forked, ev_flags);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&pipe->joined, ev_flags);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&pipe->costs_ready, ev_flags);
    for (int g = 0; g < kMaxGroups && e == cudaSuccess; ++g) {
        // highest priority: a wavefront CTA must get onto an SM as soon as a CTA of the streaming kernels retires
        e = cudaStreamCreateWithPriority(&pipe->side[g], cudaStreamNonBlocking, greatest);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&pipe->gathered[g], ev_flags);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&pipe->solved[g], ev_flags);
        if (e == cudaSuccess) e = cudaEventCreateWithFlags(&pipe->graded[g], ev_flags);
    }
    if (e != cudaSuccess) {
        fail_launch("pipe_create", e);
        cwrnnt_pipe_destroy(pipe);
        return CWRNNT_ERR_LAUNCH;
    }
    *out = pipe;
    return CWRNNT_OK;
}

int cwrnnt_pipe_create(cwrnnt_pipe **out) { return pipe_create(out, false); }
int cwrnnt_pipe_create_traced(cwrnnt_pipe **out) { return pipe_create(out, true); }

int cwrnnt_pipe_timeline(cwrnnt_pipe *pipe, float *ms, int32_t capacity)
{
    if (!pipe || !ms || capacity < 0) return -1;
    if (!pipe->traced) return -1;
    const int G = pipe->last_groups;
    if (G < 2) return 0;  // an ungrouped step stays on the caller's stream and records no events
    if (capacity < 3 * G) return -1;
    for (int g = 0; g < G; ++g) {
        cudaEvent_t ev[3] = {pipe->gathered[g], pipe->solved[g], pipe->graded[g]};
        for (int k = 0; k < 3; ++k)
            if (cudaEventElapsedTime(&ms[3 * g + k], pipe->forked, ev[k]) != cudaSuccess) {
                cudaGetLastError();
                ms[3 * g + k] = -1.0f;
            }
    }
    return G;
}

void cwrnnt_pipe_destroy(cwrnnt_pipe *pipe)
{
    if (!pipe) return;
    if (pipe->alt) cudaStreamDestroy(pipe->alt);
    if (pipe->forked) cudaEventDestroy(pipe->forked);
    if (pipe->joined) cudaEventDestroy(pipe->joined);
    if (pipe->costs_ready) cudaEventDestroy(pipe->costs_ready);
    for (int g = 0; g < kMaxGroups; ++g) {
        if (pipe->side[g]) cudaStreamDestroy(pipe->side[g]);
        if (pipe->gathered[g]) cudaEventDestroy(pipe->gathered[g]);
        if (pipe->solved[g]) cudaEventDestroy(pipe->solved[g]);
        if (pipe->graded[g]) cudaEventDestroy(pipe->graded[g]);
    }
    delete pipe;
}

int cwrnnt_loss_grad(cwrnnt_pipe *pipe, const cwrnnt_problem *p, const void *x, const int32_t *lx, const int32_t *ly,
                     const int32_t *y, void *workspace, int64_t workspace_bytes, void *costs, void *loss,
                     const void *grad_costs, int32_t grad_costs_stride, void *grad_x, const int32_t *global_ids,
                     int32_t n_global, void *cost_vector, int32_t groups, cwrnnt_stream_t stream)
{
    int st = check_problem(p);
    if (st) return st;
    if (p->flags & CWRNNT_COSTS_ONLY) return CWRNNT_ERR_ARGUMENT;
    if (groups < 0 || groups > kMaxGroups) return CWRNNT_ERR_ARGUMENT;
    if (grad_costs_stride != 0 && grad_costs_stride != 1) return CWRNNT_ERR_ARGUMENT;
    if (cost_vector ? n_global < p->B : (global_ids != nullptr || n_global != 0)) return CWRNNT_ERR_ARGUMENT;
    if (p->B == 0) return CWRNNT_OK;
    if (!lx || !ly || !costs || (p->n_rows > 0 && (!x || !grad_x)) || (p->max_u > 0 && !y)) return CWRNNT_ERR_ARGUMENT;
    Workspace w{};
    st = check_workspace(p, workspace, workspace_bytes, &w);
    if (st) return st;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    cudaError_t e;
    if (pipe) {
        int device = -1;
        if ((e = cudaGetDevice(&device)) != cudaSuccess) return fail_launch("loss_grad", e);
        if (device != pipe->device) return CWRNNT_ERR_ARGUMENT;
    }

    const GroupPlan plan = plan_groups(*p, pipe ? groups : 1);
    const int G = plan.count;
    if (pipe) pipe->last_groups = G;
    ShardOutput shard{global_ids, n_global, cost_vector};

    // Streams - few of them on purpose: a device serves its streams through a small number of hardware queues (8
    // unless the process asks for more), and streams that share a queue wait for one another as if they were one. The
    // step uses 2 + G: the gathers of consecutive ranges alternate between the caller's stream and pipe->alt (two
    // launches on one stream leave the SMs idle between the last CTAs of one and the first of the next, on two
    // streams the next one's CTAs fill in as the previous one's run out); group g's wavefront runs on the
    // high-priority stream side[g]; the gradients reuse these streams (see below).
#define CWRNNT_TRY(call, what) \
    if ((e = (call)) != cudaSuccess) return fail_launch(what, e)
    auto rows_stream = [&](int g) { return (G > 1 && (g & 1)) ? pipe->alt : s; };
    CWRNNT_TRY(launch_prep(*p, lx, ly, w, costs, s, plan, loss, cost_vector, n_global), "prep");
    if (G > 1) {
        CWRNNT_TRY(cudaEventRecord(pipe->forked, s), "event");
        CWRNNT_TRY(cudaStreamWaitEvent(pipe->alt, pipe->forked, 0), "event");
    }
    for (int g = 0; g < G; ++g) {
        const int64_t row0 = g * plan.range_rows;
        const int64_t row1 = g == G - 1 ? p->n_rows : row0 + plan.range_rows;
        CWRNNT_TRY(launch_gather(*p, x, lx, ly, y, w, rows_stream(g), row0, row1), "gather");
        cudaStream_t k2 = G > 1 ? pipe->side[g] : s;
        if (G > 1) {
            // group g needs ranges 0..g: the gathers of g, g-2, .. precede this record on its stream, those of
            // g-1, g-3, .. precede the record of g-1 on the other one
            CWRNNT_TRY(cudaEventRecord(pipe->gathered[g], rows_stream(g)), "event");
            CWRNNT_TRY(cudaStreamWaitEvent(k2, pipe->gathered[g], 0), "event");
            if (g > 0) CWRNNT_TRY(cudaStreamWaitEvent(k2, pipe->gathered[g - 1], 0), "event");
        }
        CWRNNT_TRY(launch_wavefront(*p, lx, ly, w, costs, loss, cost_vector ? &shard : nullptr, k2, plan, g),
                   "wavefront");
        if (G > 1) CWRNNT_TRY(cudaEventRecord(pipe->solved[g], k2), "event");
        if (pipe && G == 1) CWRNNT_TRY(cudaEventRecord(pipe->costs_ready, s), "event");  // before the gradient
    }
    // Where the gradient of group g is launched. Two schedules:
    //  - in order, on the two gather streams alternately, each launch behind its group's wavefront (event): the
    //    launches run back to back in group order, each filling in as the one before runs out of CTAs. Best when the
    //    wavefronts are short next to the passes (narrow lattices): every wavefront but the last is long done;
    //  - adaptive: behind the group's wavefront on that wavefront's own stream, so that the gradient launches start in
    //    the order in which the wavefronts FINISH, whatever the order of the rows - a group of short lattices that was
    //    gathered last is differentiated while the long chains of an earlier group are still running. For batches
    //    whose wavefronts can outlast a pass: wide lattices, or a handful of long sequences.
    const bool adaptive = G > 1 && (p->max_u + 1 > 256 || p->B <= 8);
    for (int g = 0; g < G; ++g) {
        GradRows span{nullptr, 0, 0, 0, false};
        cudaStream_t k3 = s;
        if (G > 1) {
            k3 = adaptive ? pipe->side[g] : rows_stream(g);
            if (adaptive) {
                // not before the gather pass is over: a gradient kernel started earlier (a short group's wavefront is
                // done in no time) would take bandwidth from the gathers that the other groups' wavefronts wait for
                CWRNNT_TRY(cudaStreamWaitEvent(k3, pipe->gathered[G - 1], 0), "event");
                CWRNNT_TRY(cudaStreamWaitEvent(k3, pipe->gathered[G - 2], 0), "event");
            } else {
                CWRNNT_TRY(cudaStreamWaitEvent(k3, pipe->solved[g], 0), "event");
            }
            // A group holds the sequences that END in its range, so it is about one range long, give or take a
            // sequence: the grid is sized for one range and a longer group is finished by the same CTAs. On a
            // wavefront's (high-priority) stream the launch itself asks for the lowest priority.
            const int64_t row0 = g * plan.range_rows;
            span = GradRows{w.bounds + g, plan.range_rows, row0, g == G - 1 ? p->n_rows : row0 + plan.range_rows,
                            adaptive};
        }
        CWRNNT_TRY(launch_grad(*p, x, lx, ly, y, w, grad_costs, grad_costs_stride, grad_x, k3, span), "grad");
        if (G > 1) CWRNNT_TRY(cudaEventRecord(pipe->graded[g], k3), "event");
    }
    if (G > 1) {
        // costs, loss and the cost vector are final once every wavefront launch is done - before the gradient kernels
        // have finished. The event lets another stream (a collective on the cost vector) start from there; it is
        // recorded on a stream of the pipe that carries no gradient launch.
        cudaStream_t collect = adaptive ? pipe->alt : pipe->side[0];
        for (int g = 0; g < G; ++g) CWRNNT_TRY(cudaStreamWaitEvent(collect, pipe->solved[g], 0), "event");
        CWRNNT_TRY(cudaEventRecord(pipe->costs_ready, collect), "event");
        // join: every gradient, pipe->alt (its gathers) and the costs-ready point
        for (int g = 0; g < G; ++g) CWRNNT_TRY(cudaStreamWaitEvent(s, pipe->graded[g], 0), "event");
        CWRNNT_TRY(cudaEventRecord(pipe->joined, pipe->alt), "event");
        CWRNNT_TRY(cudaStreamWaitEvent(s, pipe->joined, 0), "event");
        CWRNNT_TRY(cudaStreamWaitEvent(s, pipe->costs_ready, 0), "event");
    }
#undef CWRNNT_TRY
    return CWRNNT_OK;
}

int cwrnnt_pipe_wait_costs(cwrnnt_pipe *pipe, cwrnnt_stream_t stream)
{
    if (!pipe) return CWRNNT_ERR_ARGUMENT;
    cudaError_t e = cudaStreamWaitEvent(reinterpret_cast<cudaStream_t>(stream), pipe->costs_ready, 0);
    return e == cudaSuccess ? CWRNNT_OK : fail_launch("pipe_wait_costs", e);
}

int32_t cwrnnt_pipeline_groups(const cwrnnt_problem *p, int32_t groups)
{
    if (check_problem(p) != CWRNNT_OK || groups < 0 || groups > kMaxGroups) return -1;
    return plan_groups(*p, groups).count;
}

int cwrnnt_scale_grad(const cwrnnt_problem *p, void *grad_x, const void *factor, cwrnnt_stream_t stream)
{
    int st = check_problem(p);
    if (st) return st;
    if (!factor || (p->n_rows > 0 && !grad_x)) return CWRNNT_ERR_ARGUMENT;
    cudaError_t e = launch_scale(*p, grad_x, factor, reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? CWRNNT_OK : fail_launch("scale_grad", e);
}

int cwrnnt_pair_grads(const cwrnnt_problem *p, const void *x, const int32_t *lx, const int32_t *ly, const int32_t *y,
                      const void *workspace, void *grads, cwrnnt_stream_t stream)
{
    (void)x;
    (void)y;
    int st = check_problem(p);
    if (st) return st;
    if ((p->flags & CWRNNT_COSTS_ONLY) || !lx || !ly || (p->n_rows > 0 && !grads)) return CWRNNT_ERR_ARGUMENT;
    Workspace w{};
    st = check_workspace(p, workspace, -1, &w);
    if (st) return st;
    if (p->B == 0) return CWRNNT_OK;
    cudaError_t e = launch_pair_grads(*p, lx, ly, w, grads, reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? CWRNNT_OK : fail_launch("pair_grads", e);
}

int cwrnnt_export_alpha_beta(const cwrnnt_problem *p, const int32_t *lx, const int32_t *ly, const void *workspace,
                             int32_t t_max, int32_t u_max1, void *alphas, void *betas, cwrnnt_stream_t stream)
{
    int st = check_problem(p);
    if (st) return st;
    if (!lx || !ly || t_max < 0 || u_max1 < 0) return CWRNNT_ERR_ARGUMENT;
    if ((p->flags & CWRNNT_COSTS_ONLY) && alphas) return CWRNNT_ERR_ARGUMENT;
    Workspace w{};
    st = check_workspace(p, workspace, -1, &w);
    if (st) return st;
    if (p->B == 0 || (!alphas && !betas)) return CWRNNT_OK;
    cudaError_t e = launch_export_ab(*p, lx, ly, w, t_max, u_max1, alphas, betas,
                                     reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? CWRNNT_OK : fail_launch("export_alpha_beta", e);
}

int64_t cwrnnt_alignment_scratch_bytes(const cwrnnt_problem *p)
{
    if (check_problem(p) != CWRNNT_OK) return -1;
    return align_up(p->n_rows > 0 ? p->n_rows : 1, 256);
}

int cwrnnt_export_alignment(const cwrnnt_problem *p, const int32_t *lx, const int32_t *ly, const void *workspace,
                            void *scratch, int64_t scratch_bytes, int32_t path_stride, int32_t *moves, void *scores,
                            cwrnnt_stream_t stream)
{
    int st = check_problem(p);
    if (st) return st;
    if (p->B == 0) return CWRNNT_OK;
    if (!lx || !ly || !moves || !scores || path_stride < 1) return CWRNNT_ERR_ARGUMENT;
    if (!scratch || scratch_bytes < cwrnnt_alignment_scratch_bytes(p)) return CWRNNT_ERR_WORKSPACE;
    Workspace w{};
    st = check_workspace(p, workspace, -1, &w);
    if (st) return st;
    cudaError_t e = launch_alignment(*p, lx, ly, w, static_cast<unsigned char *>(scratch), path_stride, moves, scores,
                                     reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? CWRNNT_OK : fail_launch("export_alignment", e);
}

int cwrnnt_export_posteriors(const cwrnnt_problem *p, const int32_t *lx, const int32_t *ly, const void *workspace,
                             int32_t t_max, int32_t u_max1, void *posteriors, cwrnnt_stream_t stream)
{
    int st = check_problem(p);
    if (st) return st;
    if ((p->flags & CWRNNT_COSTS_ONLY) || !lx || !ly || t_max < 0 || u_max1 < 0) return CWRNNT_ERR_ARGUMENT;
    Workspace w{};
    st = check_workspace(p, workspace, -1, &w);
    if (st) return st;
    if (p->B == 0 || int64_t(t_max) * u_max1 == 0) return CWRNNT_OK;
    if (!posteriors) return CWRNNT_ERR_ARGUMENT;
    cudaError_t e = launch_posteriors(*p, lx, ly, w, t_max, u_max1, posteriors, reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? CWRNNT_OK : fail_launch("export_posteriors", e);
}

int cwrnnt_fill_costs(const cwrnnt_problem *p, const int32_t *lx, const double *ll_alpha, const double *ll_beta,
                      void *costs, int32_t *status, cwrnnt_stream_t stream)
{
    int st = check_problem(p);
    if (st) return st;
    if (p->B == 0) return CWRNNT_OK;
    if (!lx || !ll_beta || !costs || !status) return CWRNNT_ERR_ARGUMENT;
    cudaError_t e = launch_fill_costs(*p, lx, ll_alpha, ll_beta, costs, status, reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? CWRNNT_OK : fail_launch("fill_costs", e);
}

int64_t cwrnnt_scatter_scratch_bytes(int32_t B) { return B < 0 ? -1 : align_up(8 * (int64_t(B) + 1), 256); }

int cwrnnt_scatter_backward(const cwrnnt_problem *p, const void *grads, const void *grad_costs, const int32_t *lx,
                            const int32_t *ly, const int32_t *y, void *scratch, int64_t scratch_bytes, void *dense,
                            cwrnnt_stream_t stream)
{
    int st = check_problem(p);
    if (st) return st;
    if (p->dtype != CWRNNT_F32 && p->dtype != CWRNNT_F64) return CWRNNT_ERR_ARGUMENT;
    if (!lx || !ly || !grad_costs || (p->n_rows > 0 && (!grads || !dense)) || (p->max_u > 0 && !y))
        return CWRNNT_ERR_ARGUMENT;
    if (!scratch || reinterpret_cast<uintptr_t>(scratch) % 8 != 0 || scratch_bytes < cwrnnt_scatter_scratch_bytes(p->B))
        return CWRNNT_ERR_WORKSPACE;
    if (p->B == 0) return CWRNNT_OK;
    cudaError_t e = launch_scatter(*p, grads, grad_costs, lx, ly, y, static_cast<int64_t *>(scratch), dense,
                                   reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? CWRNNT_OK : fail_launch("scatter_backward", e);
}

static int pack_impl(const cwrnnt_problem *p, bool to_compact, const void *src, void *dst, int32_t t_max,
                     int32_t u_max1, const int32_t *lx, const int32_t *ly, void *scratch, int64_t scratch_bytes,
                     cwrnnt_stream_t stream)
{
    int st = check_problem(p);
    if (st) return st;
    if (p->B == 0) return CWRNNT_OK;
    if (!lx || !ly || t_max < 0 || u_max1 < 1 || u_max1 < p->max_u + 1) return CWRNNT_ERR_ARGUMENT;
    const int64_t padded_rows = int64_t(p->B) * t_max * u_max1;
    if ((p->n_rows > 0 && !(to_compact ? dst : src)) || (padded_rows > 0 && !(to_compact ? src : dst)))
        return CWRNNT_ERR_ARGUMENT;
    if (!scratch || reinterpret_cast<uintptr_t>(scratch) % 8 != 0 || scratch_bytes < cwrnnt_scatter_scratch_bytes(p->B))
        return CWRNNT_ERR_WORKSPACE;
    cudaError_t e = launch_pack(*p, to_compact, src, dst, t_max, u_max1, lx, ly, static_cast<int64_t *>(scratch),
                                reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? CWRNNT_OK : fail_launch(to_compact ? "pack_padded" : "unpack_padded", e);
}

int cwrnnt_pack_padded(const cwrnnt_problem *p, const void *padded, int32_t t_max, int32_t u_max1, const int32_t *lx,
                       const int32_t *ly, void *scratch, int64_t scratch_bytes, void *compact, cwrnnt_stream_t stream)
{
    return pack_impl(p, true, padded, compact, t_max, u_max1, lx, ly, scratch, scratch_bytes, stream);
}

int cwrnnt_unpack_padded(const cwrnnt_problem *p, const void *compact, int32_t t_max, int32_t u_max1,
                         const int32_t *lx, const int32_t *ly, void *scratch, int64_t scratch_bytes, void *padded,
                         cwrnnt_stream_t stream)
{
    return pack_impl(p, false, compact, padded, t_max, u_max1, lx, ly, scratch, scratch_bytes, stream);
}

static int validate_impl(const cwrnnt_problem *p, const int32_t *lx, const int32_t *ly, const int32_t *y,
                         void *scratch, int32_t out[4], cwrnnt_stream_t stream, bool wait)
{
    int st = check_problem(p);
    if (st) return st;
    if (!out) return CWRNNT_ERR_ARGUMENT;
    if (p->B == 0) {
        out[0] = p->n_rows != 0 ? CWRNNT_ST_ROW_MISMATCH : 0, out[1] = -1, out[2] = 0, out[3] = 0;
        return CWRNNT_OK;
    }
    if (!lx || !ly || (p->max_u > 0 && !y)) return CWRNNT_ERR_ARGUMENT;
    if (!scratch || reinterpret_cast<uintptr_t>(scratch) % 4 != 0) return CWRNNT_ERR_WORKSPACE;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    cudaError_t e = launch_validate(*p, lx, ly, y, static_cast<int32_t *>(scratch), s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(out, scratch, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess && wait) e = cudaStreamSynchronize(s);
    return e == cudaSuccess ? CWRNNT_OK : fail_launch("validate", e);
}

int cwrnnt_validate(const cwrnnt_problem *p, const int32_t *lx, const int32_t *ly, const int32_t *y, void *scratch,
                    int32_t out[4], cwrnnt_stream_t stream)
{
    return validate_impl(p, lx, ly, y, scratch, out, stream, true);
}

int cwrnnt_validate_async(const cwrnnt_problem *p, const int32_t *lx, const int32_t *ly, const int32_t *y,
                          void *scratch, int32_t out[4], cwrnnt_stream_t stream)
{
    return validate_impl(p, lx, ly, y, scratch, out, stream, false);
}

static int joint_impl(const cwrnnt_problem *p, int32_t activation, bool backward, const void *enc, int32_t t_max,
                      const void *pred, int32_t u_max1, const int32_t *lx, const int32_t *ly, const void *grad_out,
                      void *scratch, int64_t scratch_bytes, void *a, void *b, cwrnnt_stream_t stream)
{
    int st = check_problem(p);
    if (st) return st;
    if (activation < CWRNNT_ACT_NONE || activation > CWRNNT_ACT_TANH) return CWRNNT_ERR_ARGUMENT;
    if (p->B == 0) return CWRNNT_OK;
    if (!lx || !ly || t_max < 1 || u_max1 < 1 || u_max1 < p->max_u + 1) return CWRNNT_ERR_ARGUMENT;
    if (!enc || !pred || (backward ? (!a || !b || (p->n_rows > 0 && !grad_out)) : (p->n_rows > 0 && !a)))
        return CWRNNT_ERR_ARGUMENT;
    if (!scratch || reinterpret_cast<uintptr_t>(scratch) % 8 != 0 || scratch_bytes < cwrnnt_scatter_scratch_bytes(p->B))
        return CWRNNT_ERR_WORKSPACE;
    cudaError_t e = launch_joint(*p, activation, backward, enc, t_max, pred, u_max1, lx, ly,
                                 static_cast<int64_t *>(scratch), grad_out, a, b,
                                 reinterpret_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? CWRNNT_OK : fail_launch(backward ? "joint_backward" : "joint_forward", e);
}

int cwrnnt_joint_forward(const cwrnnt_problem *p, int32_t activation, const void *enc, int32_t t_max, const void *pred,
                         int32_t u_max1, const int32_t *lx, const int32_t *ly, void *scratch, int64_t scratch_bytes,
                         void *out, cwrnnt_stream_t stream)
{
    return joint_impl(p, activation, false, enc, t_max, pred, u_max1, lx, ly, nullptr, scratch, scratch_bytes, out,
                      nullptr, stream);
}

int cwrnnt_joint_backward(const cwrnnt_problem *p, int32_t activation, const void *enc, int32_t t_max,
                          const void *pred, int32_t u_max1, const int32_t *lx, const int32_t *ly, const void *grad_out,
                          void *scratch, int64_t scratch_bytes, void *grad_enc, void *grad_pred,
                          cwrnnt_stream_t stream)
{
    return joint_impl(p, activation, true, enc, t_max, pred, u_max1, lx, ly, grad_out, scratch, scratch_bytes,
                      grad_enc, grad_pred, stream);
}

int cwrnnt_read_status(const void *workspace, int32_t out[4], cwrnnt_stream_t stream)
{
    if (!workspace || !out) return CWRNNT_ERR_ARGUMENT;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(out, workspace, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    return e == cudaSuccess ? CWRNNT_OK : fail_launch("read_status", e);
}

}  // extern "C"
