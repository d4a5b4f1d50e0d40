// Launchers of the device kernels (one per translation unit). Internal.
#pragma once
#include "cwrnnt_common.cuh"

namespace cwrnnt {

// Text returned by cwrnnt_last_error() on the calling thread.
void set_last_error(const char *text);

// K0: offsets, validation, longest-first order, first row of every sequence group of `plan`. 1 CTA. On invalid
// lengths it writes NaN to costs, to *loss (when a reduction flag is set) and to the n_global + 1 entries of a sharded
// run's cost vector; either pointer may be null.
cudaError_t launch_prep(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                        void *costs, cudaStream_t s, GroupPlan plan = GroupPlan{1, 1}, void *loss = nullptr,
                        void *cost_vector = nullptr, int n_global = 0);

// Lengths, row count and labels checked by one small kernel; four words into out_device (see cwrnnt_validate).
cudaError_t launch_validate(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const int32_t *y,
                            int32_t *out_device, cudaStream_t s);

cudaError_t launch_offsets_only(const int32_t *lx, const int32_t *ly, int B, int max_u, int64_t *off, cudaStream_t s);

// K1: row log-sum-exp + blank/label log-prob gather into the diagonal-major arrays, rows [row0, row1)
// (row1 < 0: up to the last row).
cudaError_t launch_gather(const cwrnnt_problem &p, const void *x, const int32_t *lx, const int32_t *ly,
                          const int32_t *y, const Workspace &w, cudaStream_t s, int64_t row0 = 0, int64_t row1 = -1);

// Sharded runs: where the costs go besides the local [B] array (see cwrnnt_forward_sharded).
struct ShardOutput {
    const int32_t *global_ids;  // [B] global slot of each local sequence, or nullptr for the identity
    int32_t n_global;           // number of sequences over all ranks
    void *cost_vector;          // [n_global + 1], costs type
};

// K2: alpha/beta anti-diagonal wavefront, costs, loss. With a plan of several groups, one launch per group: only the
// sequences of `group` run, and the CTA that takes the last completion ticket over ALL launches writes costs and loss.
cudaError_t launch_wavefront(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                             void *costs, void *loss, const ShardOutput *shard, cudaStream_t s,
                             GroupPlan plan = GroupPlan{1, 1}, int group = 0);

// K3: dense gradient in one streaming pass, over all rows or over the rows device_range[0] .. device_range[1]
// (a sequence group; the pair lives in device memory, the grid is sized for grid_rows rows). nominal_begin/end: the
// host-known row range this launch stands for, used only to fill the gradient with NaN after a fatal input error.
struct GradRows {
    const int64_t *device_range;
    int64_t grid_rows;
    int64_t nominal_begin, nominal_end;
    bool lowest_priority;  // launch at the device's lowest priority whatever the stream's (dense logits-mode kernels)
};
cudaError_t launch_grad(const cwrnnt_problem &p, const void *x, const int32_t *lx, const int32_t *ly,
                        const int32_t *y, const Workspace &w, const void *grad_costs, int32_t gc_stride, void *grad_x,
                        cudaStream_t s, const GradRows &span = GradRows{nullptr, 0, 0, 0, false});

// grad_x *= *factor (a device scalar of the costs' type); returns at once on the device when the factor is 1.
cudaError_t launch_scale(const cwrnnt_problem &p, void *grad_x, const void *factor, cudaStream_t s);

// Reference-shaped exports.
cudaError_t launch_pair_grads(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                              void *grads, cudaStream_t s);
cudaError_t launch_export_ab(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                             int32_t t_max, int32_t u_max1, void *alphas, void *betas, cudaStream_t s);
cudaError_t launch_scatter(const cwrnnt_problem &p, const void *grads, const void *grad_costs, const int32_t *lx,
                           const int32_t *ly, const int32_t *y, int64_t *off_scratch, void *dense, cudaStream_t s);

// Analysis exports: best path of every sequence (`back`: one byte per lattice node of scratch) and node posteriors in
// the padded [B, t_max, u_max1] layout.
cudaError_t launch_alignment(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                             unsigned char *back, int32_t stride, int32_t *moves, void *scores, cudaStream_t s);
cudaError_t launch_posteriors(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                              int32_t t_max, int32_t u_max1, void *post, cudaStream_t s);

// Costs from per-sequence log-likelihoods with the forward/backward guard (ll_alpha may be null: no guard).
cudaError_t launch_fill_costs(const cwrnnt_problem &p, const int32_t *lx, const double *ll_alpha,
                              const double *ll_beta, void *costs, int32_t *status, cudaStream_t s);

// Padded [B, t_max, u_max1, V] <-> compact [n_rows, V] (to_compact: src padded, dst compact; else the transpose,
// zero-filling the padding).
cudaError_t launch_pack(const cwrnnt_problem &p, bool to_compact, const void *src, void *dst, int32_t t_max,
                        int32_t u_max1, const int32_t *lx, const int32_t *ly, int64_t *off_scratch, cudaStream_t s);

// Joint broadcast-add into compact rows (forward: `out_or_grad_enc` = out [n_rows, H]) and its two reductions
// (backward: grad_enc [B, t_max, H], grad_pred [B, u_max1, H] from grad_out [n_rows, H]); H = p.V.
cudaError_t launch_joint(const cwrnnt_problem &p, int activation, bool backward, const void *enc, int32_t t_max,
                         const void *pred, int32_t u_max1, const int32_t *lx, const int32_t *ly, int64_t *off_scratch,
                         const void *grad_out, void *out_or_grad_enc, void *grad_pred, cudaStream_t s);

}  // namespace cwrnnt
