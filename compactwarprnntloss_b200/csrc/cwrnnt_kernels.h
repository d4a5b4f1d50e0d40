// Launchers of the device kernels (one per translation unit). Internal.
#pragma once
#include "cwrnnt_common.cuh"

namespace cwrnnt {

// Text returned by cwrnnt_last_error() on the calling thread.
void set_last_error(const char *text);

// K0: offsets, validation, longest-first order. 1 CTA.
cudaError_t launch_prep(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                        void *costs, cudaStream_t s);

cudaError_t launch_offsets_only(const int32_t *lx, const int32_t *ly, int B, int max_u, int64_t *off, cudaStream_t s);

// K1: row log-sum-exp + blank/label log-prob gather into the diagonal-major arrays.
cudaError_t launch_gather(const cwrnnt_problem &p, const void *x, const int32_t *lx, const int32_t *ly,
                          const int32_t *y, const Workspace &w, cudaStream_t s);

// Sharded runs: where the costs go besides the local [B] array (see cwrnnt_forward_sharded).
struct ShardOutput {
    const int32_t *global_ids;  // [B] global slot of each local sequence, or nullptr for the identity
    int32_t n_global;           // number of sequences over all ranks
    void *cost_vector;          // [n_global + 1], costs type
};

// K2: alpha/beta anti-diagonal wavefront, costs, loss.
cudaError_t launch_wavefront(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                             void *costs, void *loss, const ShardOutput *shard, cudaStream_t s);

// K3: dense gradient in one streaming pass.
cudaError_t launch_grad(const cwrnnt_problem &p, const void *x, const int32_t *lx, const int32_t *ly,
                        const int32_t *y, const Workspace &w, const void *grad_costs, int32_t gc_stride, void *grad_x,
                        cudaStream_t s);

// Reference-shaped exports.
cudaError_t launch_pair_grads(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                              void *grads, cudaStream_t s);
cudaError_t launch_export_ab(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                             int32_t t_max, int32_t u_max1, void *alphas, void *betas, cudaStream_t s);
cudaError_t launch_scatter(const cwrnnt_problem &p, const void *grads, const void *grad_costs, const int32_t *lx,
                           const int32_t *ly, const int32_t *y, int64_t *off_scratch, void *dense, cudaStream_t s);

// Padded [B, t_max, u_max1, V] <-> compact [n_rows, V] (to_compact: src padded, dst compact; else the transpose,
// zero-filling the padding).
cudaError_t launch_pack(const cwrnnt_problem &p, bool to_compact, const void *src, void *dst, int32_t t_max,
                        int32_t u_max1, const int32_t *lx, const int32_t *ly, int64_t *off_scratch, cudaStream_t s);

}  // namespace cwrnnt
