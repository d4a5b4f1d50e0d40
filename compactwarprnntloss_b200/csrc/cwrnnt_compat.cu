// Reference-shaped views of the engine's state, for callers of the reference extension module's three functions:
//   pair gradients [STU,2]              (cwarp_cuda_rnnt_kernel.cu:275-332 fill_grad_blank/label kernels)
//   zero-padded alphas/betas [N,Tm,Up]  (cwarp_cuda_rnnt_kernel.cu:399-400, returned at :496)
//   scale + scatter backward            (cwarp_cuda_rnnt_kernel.cu:512-521, cwarp_cuda.cpp:134,
//                                        cwarp_cuda_gather_kernel.cu:52-74)
// All three are small streaming kernels over [STU] (or [STU,V] for the scatter, which is write-only).
#include "cwrnnt_kernels.h"
#include "cwrnnt_rowmap.cuh"

namespace cwrnnt {

template <typename CostT>
__global__ void __launch_bounds__(kStreamThreads)
pair_grads_kernel(int64_t n_rows, int B, const int32_t *__restrict__ lx, const int32_t *__restrict__ ly, Workspace w,
                  CostT *__restrict__ grads)
{
    if (w.status[0] & CWRNNT_ST_FATAL) return;
    int cursor = 0;
    const int64_t stride = int64_t(gridDim.x) * kStreamThreads;
    for (int64_t r = int64_t(blockIdx.x) * kStreamThreads + threadIdx.x; r < n_rows; r += stride) {
        const int n = cursor = find_sequence(w.off, B, r, cursor);
        const int64_t off = w.off[n];
        const int T = lx[n], U = ly[n], m = U + 1;
        const unsigned rel = unsigned(r - off);
        const int t = int(rel / unsigned(m)), u = int(rel - unsigned(t) * unsigned(m));
        int64_t cell, next;
        diag_cell_and_next(t, u, T, m, &cell, &next);
        const int64_t at = off + cell;
        const double ll = w.ll_beta[n], a = w.alpha[at];
        double gb = 0.0, gl = 0.0;
        if (t < T - 1)
            gb = -exp(a + w.beta[off + next] + w.lp_blank[at] - ll);
        else if (u == U)
            gb = -exp(a + w.lp_blank[at] - ll);
        if (u < U) gl = -exp(a + w.beta[off + next + 1] + w.lp_label[at] - ll);
        grads[2 * r] = CostT(gb);
        grads[2 * r + 1] = CostT(gl);
    }
}

// One thread per padded cell [n, t, u]; cells outside the sequence's lattice are zero.
template <typename CostT>
__global__ void __launch_bounds__(kStreamThreads)
export_ab_kernel(int B, int t_max, int u_max1, const int32_t *__restrict__ lx, const int32_t *__restrict__ ly,
                 Workspace w, CostT *__restrict__ alphas, CostT *__restrict__ betas)
{
    if (w.status[0] & CWRNNT_ST_FATAL) return;
    const int64_t per = int64_t(t_max) * u_max1, total = per * B;
    const int64_t stride = int64_t(gridDim.x) * kStreamThreads;
    for (int64_t i = int64_t(blockIdx.x) * kStreamThreads + threadIdx.x; i < total; i += stride) {
        const int n = int(i / per);
        const int64_t rem = i - int64_t(n) * per;
        const int t = int(rem / u_max1), u = int(rem - int64_t(t) * u_max1);
        const int T = lx[n], U = ly[n];
        const bool in = t < T && u <= U;
        const int64_t r = in ? w.off[n] + diag_index(t, u, T, U + 1) : 0;
        if (alphas) alphas[i] = in ? CostT(w.alpha[r]) : CostT(0);
        if (betas) betas[i] = in ? CostT(w.beta[r]) : CostT(0);
    }
}

// dense[r][:] = 0; dense[r][blank] = grads[r][0]*g_n; dense[r][y] = grads[r][1]*g_n (terms add when y == blank).
template <typename CostT>
__global__ void __launch_bounds__(kStreamThreads)
scatter_kernel(int64_t n_rows, int V, int B, const int32_t *__restrict__ lx, const int32_t *__restrict__ ly,
               const int32_t *__restrict__ y, int y_stride, int blank, const int64_t *__restrict__ off,
               const CostT *__restrict__ grads, const CostT *__restrict__ grad_costs, CostT *__restrict__ dense)
{
    if (off[B] != n_rows) return;  // row count and lengths disagree: leave the output untouched
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * kStreamThreads + threadIdx.x) >> 5;
    const int64_t n_warps = (int64_t(gridDim.x) * kStreamThreads) >> 5;
    const int64_t per_warp = (n_rows + n_warps - 1) / n_warps;
    const int64_t r_begin = warp * per_warp;
    const int64_t r_end = r_begin + per_warp < n_rows ? r_begin + per_warp : n_rows;
    if (r_begin >= r_end) return;
    bool ignored = false;
    RowWalker rw;
    rw.start(r_begin, off, B, lx, ly);
    for (int64_t r = r_begin; r < r_end; ++r) {
        const int label = rw.label(y, y_stride, V, ignored);
        const CostT g = grad_costs[rw.n];
        const CostT vb = grads[2 * r] * g;
        const CostT vl = label >= 0 ? grads[2 * r + 1] * g : CostT(0);
        CostT *row = dense + r * int64_t(V);
        for (int k = lane; k < V; k += 32) {
            CostT v = CostT(0);
            if (k == blank) v += vb;
            if (k == label) v += vl;
            __stcs(row + k, v);
        }
        rw.advance(off, B, lx, ly);
    }
}

// costs[n] = -guarded(ll_alpha[n], ll_beta[n]) (* 1/T_n under CWRNNT_AVERAGE_FRAMES): the cost step of the wavefront's
// epilogue on its own, from caller-supplied log-likelihoods (reference fill_cost_kernel,
// cwarp_cuda_rnnt_kernel.cu:334-367). status[0] receives CWRNNT_ST_FWD_BWD_GAP when the guard fires.
template <typename CostT>
__global__ void __launch_bounds__(kStreamThreads)
fill_costs_kernel(int B, int flags, const int32_t *__restrict__ lx, const double *__restrict__ ll_alpha,
                  const double *__restrict__ ll_beta, CostT *__restrict__ costs, int32_t *__restrict__ status)
{
    const int n = blockIdx.x * kStreamThreads + threadIdx.x;
    if (n >= B) return;
    bool gap = false;
    const double ll = ll_alpha ? guarded_loglik(ll_alpha[n], ll_beta[n], gap) : ll_beta[n];
    if (gap) atomicOr(status, CWRNNT_ST_FWD_BWD_GAP);
    costs[n] = CostT(-ll * sequence_scale(flags, lx[n]));
}

cudaError_t launch_fill_costs(const cwrnnt_problem &p, const int32_t *lx, const double *ll_alpha,
                              const double *ll_beta, void *costs, int32_t *status, cudaStream_t s)
{
    if (p.B == 0) return cudaSuccess;
    const int grid = (p.B + kStreamThreads - 1) / kStreamThreads;
    if (p.dtype == CWRNNT_F64)
        fill_costs_kernel<double><<<grid, kStreamThreads, 0, s>>>(p.B, p.flags, lx, ll_alpha, ll_beta,
                                                                  static_cast<double *>(costs), status);
    else
        fill_costs_kernel<float><<<grid, kStreamThreads, 0, s>>>(p.B, p.flags, lx, ll_alpha, ll_beta,
                                                                 static_cast<float *>(costs), status);
    return cudaGetLastError();
}

static int stream_grid(int64_t items, int per_cta)
{
    int64_t t = (items + per_cta - 1) / per_cta;
    const int64_t cap = kNumSMs * 8;
    return int(t < 1 ? 1 : (t < cap ? t : cap));
}

cudaError_t launch_pair_grads(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                              void *grads, cudaStream_t s)
{
    if (p.n_rows == 0) return cudaSuccess;
    const int grid = stream_grid(p.n_rows, kStreamThreads);
    if (p.dtype == CWRNNT_F64)
        pair_grads_kernel<double><<<grid, kStreamThreads, 0, s>>>(p.n_rows, p.B, lx, ly, w, static_cast<double *>(grads));
    else
        pair_grads_kernel<float><<<grid, kStreamThreads, 0, s>>>(p.n_rows, p.B, lx, ly, w, static_cast<float *>(grads));
    return cudaGetLastError();
}

cudaError_t launch_export_ab(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                             int32_t t_max, int32_t u_max1, void *alphas, void *betas, cudaStream_t s)
{
    const int64_t total = int64_t(p.B) * t_max * u_max1;
    if (total == 0) return cudaSuccess;
    const int grid = stream_grid(total, kStreamThreads);
    if (p.dtype == CWRNNT_F64)
        export_ab_kernel<double><<<grid, kStreamThreads, 0, s>>>(p.B, t_max, u_max1, lx, ly, w,
                                                                 static_cast<double *>(alphas),
                                                                 static_cast<double *>(betas));
    else
        export_ab_kernel<float><<<grid, kStreamThreads, 0, s>>>(p.B, t_max, u_max1, lx, ly, w,
                                                                static_cast<float *>(alphas),
                                                                static_cast<float *>(betas));
    return cudaGetLastError();
}

cudaError_t launch_scatter(const cwrnnt_problem &p, const void *grads, const void *grad_costs, const int32_t *lx,
                           const int32_t *ly, const int32_t *y, int64_t *off_scratch, void *dense, cudaStream_t s)
{
    cudaError_t e = launch_offsets_only(lx, ly, p.B, p.max_u, off_scratch, s);
    if (e != cudaSuccess || p.n_rows == 0) return e;
    const int grid = stream_grid(p.n_rows, kStreamThreads / 32);
    if (p.dtype == CWRNNT_F64)
        scatter_kernel<double><<<grid, kStreamThreads, 0, s>>>(p.n_rows, p.V, p.B, lx, ly, y, p.y_stride, p.blank,
                                                               off_scratch, static_cast<const double *>(grads),
                                                               static_cast<const double *>(grad_costs),
                                                               static_cast<double *>(dense));
    else
        scatter_kernel<float><<<grid, kStreamThreads, 0, s>>>(p.n_rows, p.V, p.B, lx, ly, y, p.y_stride, p.blank,
                                                              off_scratch, static_cast<const float *>(grads),
                                                              static_cast<const float *>(grad_costs),
                                                              static_cast<float *>(dense));
    return cudaGetLastError();
}

}  // namespace cwrnnt
