// K3 - gradient of the loss w.r.t. the [n_rows, V] input in a single streaming pass.
//
// Logits mode (CWRNNT_FUSED_LOG_SOFTMAX): with occupancies
//     occ_b(t,u) = exp(alpha(t,u) + beta(t+1,u) + lp_blank(t,u) - ll)     (terminal cell: no beta term)
//     occ_l(t,u) = exp(alpha(t,u) + beta(t,u+1) + lp_label(t,u) - ll)     (u < U)
// (the negated pair gradients of cwarp_cuda_rnnt_kernel.cu:296-307 and :325-331) and p = softmax(x[r]) the chain rule
// through log-softmax collapses to
//     grad[r][k] = w_n * ( p_k * (occ_b + occ_l) - [k == blank] occ_b - [k == y_u] occ_l ).
// That one pass replaces: the in-place scaling of the saved pair gradients (cwarp_cuda_rnnt_kernel.cu:512-521), the
// zero fill of [STU,V] (cwarp_cuda.cpp:134), scatter_grad_cuda_kernel (cwarp_cuda_gather_kernel.cu:52-74) and the
// caller's log_softmax backward. Each row is read once (128-bit loads, evict-first) and written once (128-bit
// streaming stores); the per-row scalars (lse, alpha, two betas) are 32 bytes against V*sizeof(element).
//
// Log-prob mode: the reference's own result, zeros plus the two sparse terms; the input rows are not read at all.
//
// Bound: HBM bandwidth. Algorithmic bytes: 2 * V * sizeof(element) per row (V * sizeof(element) in log-prob mode).
#include "cwrnnt_kernels.h"
#include "cwrnnt_rowmap.cuh"

namespace cwrnnt {

__device__ __forceinline__ double occupancy(double e, float) { return double(expf(float(e))); }
__device__ __forceinline__ double occupancy(double e, double) { return exp(e); }

// Occupancy terms of one row from the saved forward state. lpb/lpl: log-probs of blank / label at this cell.
template <typename CostT>
__device__ __forceinline__ void row_terms(const RowInfo &ri, int64_t r, const Workspace &w, double lpb, double lpl,
                                          const CostT *__restrict__ grad_costs, int gc_stride, int flags,
                                          double mean_inv, double &wb, double &wl)
{
    const int m = ri.U + 1;
    const double ll = __ldg(w.ll_beta + ri.n);
    const double a = __ldg(w.alpha + r);
    double eb = -INFINITY, el = -INFINITY;
    if (ri.t < ri.T - 1)
        eb = a + __ldg(w.beta + r + m) + lpb - ll;
    else if (ri.u == ri.U)
        eb = a + lpb - ll;
    if (ri.u < ri.U) el = a + __ldg(w.beta + r + 1) + lpl - ll;
    double g = grad_costs ? double(__ldg(grad_costs + int64_t(ri.n) * gc_stride)) : 1.0;
    g *= sequence_scale(flags, ri.T) * mean_inv;
    wb = g * occupancy(eb, CostT(0));
    wl = g * occupancy(el, CostT(0));
}

template <typename T, int LPR, int NV>
__global__ void __launch_bounds__(kStreamThreads)
grad_rows_kernel(const T *__restrict__ x, T *__restrict__ gx, int V, int64_t n_rows, int B,
                 const int32_t *__restrict__ lx, const int32_t *__restrict__ ly, const int32_t *__restrict__ y,
                 int y_stride, int blank, int flags, double mean_inv, Workspace w,
                 const typename Elt<T>::cost *__restrict__ grad_costs, int gc_stride)
{
    using E = Elt<T>;
    using A = typename E::acc;
    using CostT = typename E::cost;
    constexpr int VE = E::VE;
    constexpr int RPC = kStreamThreads / LPR;
    if (w.status[0] & CWRNNT_ST_FATAL) return;

    const int gl = threadIdx.x % LPR;
    const int grp = threadIdx.x / LPR;
    const int nvec = V / VE;
    const int64_t n_tiles = (n_rows + RPC - 1) / RPC;
    int cursor = 0;

    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int64_t r = tile * RPC + grp;
        if (r >= n_rows) continue;  // no warp-wide collectives below: each lane works alone
        RowInfo ri = locate_row(r, cursor, w.off, B, lx, ly, y, y_stride, V);
        const T *row = x + r * int64_t(V);
        T *orow = gx + r * int64_t(V);
        const uint4 *rv = reinterpret_cast<const uint4 *>(row);
        uint4 *ov = reinterpret_cast<uint4 *>(orow);
        uint4 v[NV];
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int idx = j * LPR + gl;
            if (idx < nvec) v[j] = ld_stream(rv + idx);
        }
        const A xb = E::to_acc(__ldg(row + blank));
        const A xl = ri.label >= 0 ? E::to_acc(__ldg(row + ri.label)) : A(0);
        const double lse = __ldg(w.lse + r);
        double wb, wl;
        row_terms<CostT>(ri, r, w, double(xb) - lse, double(xl) - lse, grad_costs, gc_stride, flags, mean_inv, wb, wl);
        const A tot = A(wb + wl);
        const A lse_a = A(lse);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int idx = j * LPR + gl;
            if (idx < nvec) {
                A e[VE];
                E::unpack(v[j], e);
#pragma unroll
                for (int c = 0; c < VE; ++c) e[c] = exp_shifted(e[c], lse_a) * tot;
                st_stream(ov + idx, E::pack(e));
            }
        }
        // the two sparse corrections, by the lane that stored the enclosing vector (same-thread program order)
        if ((blank / VE) % LPR == gl) {
            A gb = exp_shifted(xb, lse_a) * tot - A(wb);
            if (ri.label == blank) gb -= A(wl);
            orow[blank] = E::from_acc(gb);
        }
        if (ri.label >= 0 && ri.label != blank && (ri.label / VE) % LPR == gl)
            orow[ri.label] = E::from_acc(exp_shifted(xl, lse_a) * tot - A(wl));
    }
}

// Any V / alignment, logits mode: one warp per row, scalar coalesced accesses.
template <typename T>
__global__ void __launch_bounds__(kStreamThreads)
grad_rows_generic_kernel(const T *__restrict__ x, T *__restrict__ gx, int V, int64_t n_rows, int B,
                         const int32_t *__restrict__ lx, const int32_t *__restrict__ ly,
                         const int32_t *__restrict__ y, int y_stride, int blank, int flags, double mean_inv,
                         Workspace w, const typename Elt<T>::cost *__restrict__ grad_costs, int gc_stride)
{
    using E = Elt<T>;
    using A = typename E::acc;
    using CostT = typename E::cost;
    if (w.status[0] & CWRNNT_ST_FATAL) return;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * kStreamThreads + threadIdx.x) >> 5;
    const int64_t n_warps = (int64_t(gridDim.x) * kStreamThreads) >> 5;
    int cursor = 0;
    for (int64_t r = warp; r < n_rows; r += n_warps) {
        RowInfo ri = locate_row(r, cursor, w.off, B, lx, ly, y, y_stride, V);
        const T *row = x + r * int64_t(V);
        T *orow = gx + r * int64_t(V);
        const A xb = E::to_acc(__ldg(row + blank));
        const A xl = ri.label >= 0 ? E::to_acc(__ldg(row + ri.label)) : A(0);
        const double lse = __ldg(w.lse + r);
        double wb, wl;
        row_terms<CostT>(ri, r, w, double(xb) - lse, double(xl) - lse, grad_costs, gc_stride, flags, mean_inv, wb, wl);
        const A tot = A(wb + wl), lse_a = A(lse);
        for (int k = lane; k < V; k += 32) {
            A g = exp_shifted(E::to_acc(__ldg(row + k)), lse_a) * tot;
            if (k == blank) g -= A(wb);
            if (k == ri.label) g -= A(wl);
            orow[k] = E::from_acc(g);
        }
    }
}

// Log-prob mode: zeros and the two sparse terms; the input is only touched at two elements per row.
template <typename T>
__global__ void __launch_bounds__(kStreamThreads)
grad_rows_sparse_kernel(const T *__restrict__ x, T *__restrict__ gx, int V, int64_t n_rows, int B,
                        const int32_t *__restrict__ lx, const int32_t *__restrict__ ly,
                        const int32_t *__restrict__ y, int y_stride, int blank, int flags, double mean_inv,
                        Workspace w, const typename Elt<T>::cost *__restrict__ grad_costs, int gc_stride, int vec_ok)
{
    using E = Elt<T>;
    using A = typename E::acc;
    using CostT = typename E::cost;
    constexpr int VE = E::VE;
    if (w.status[0] & CWRNNT_ST_FATAL) return;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * kStreamThreads + threadIdx.x) >> 5;
    const int64_t n_warps = (int64_t(gridDim.x) * kStreamThreads) >> 5;
    int cursor = 0;
    for (int64_t r = warp; r < n_rows; r += n_warps) {
        RowInfo ri = locate_row(r, cursor, w.off, B, lx, ly, y, y_stride, V);
        const T *row = x + r * int64_t(V);
        T *orow = gx + r * int64_t(V);
        const A xb = E::to_acc(__ldg(row + blank));
        const A xl = ri.label >= 0 ? E::to_acc(__ldg(row + ri.label)) : A(0);
        double wb, wl;
        row_terms<CostT>(ri, r, w, double(xb), double(xl), grad_costs, gc_stride, flags, mean_inv, wb, wl);
        if (vec_ok) {
            uint4 *ov = reinterpret_cast<uint4 *>(orow);
            const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
            for (int idx = lane; idx < V / VE; idx += 32) st_stream(ov + idx, zero);
            // the lane that zeroed the enclosing vector writes the sparse term afterwards
            if ((blank / VE) % 32 == lane) orow[blank] = E::from_acc(A(-(wb + (ri.label == blank ? wl : 0.0))));
            if (ri.label >= 0 && ri.label != blank && (ri.label / VE) % 32 == lane)
                orow[ri.label] = E::from_acc(A(-wl));
        } else {
            for (int k = lane; k < V; k += 32) {
                A g = A(0);
                if (k == blank) g -= A(wb);
                if (k == ri.label) g -= A(wl);
                orow[k] = E::from_acc(g);
            }
        }
    }
}

template <typename T>
static cudaError_t launch_grad_t(const cwrnnt_problem &p, const T *x, const int32_t *lx, const int32_t *ly,
                                 const int32_t *y, const Workspace &w, const void *grad_costs, int32_t gc_stride,
                                 T *gx, cudaStream_t s)
{
    using CostT = typename Elt<T>::cost;
    if (p.n_rows == 0) return cudaSuccess;
    constexpr int VE = Elt<T>::VE;
    const int max_ctas = kNumSMs * 8;
    const CostT *gc = static_cast<const CostT *>(grad_costs);
    const double mean_inv =
        (p.flags & CWRNNT_REDUCE_MEAN) ? 1.0 / double(p.mean_denominator > 0 ? p.mean_denominator : p.B) : 1.0;
    const bool aligned = (p.V % VE == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                         (reinterpret_cast<uintptr_t>(gx) % 16 == 0);
    int64_t tiles = (p.n_rows + 7) / 8;
    int grid = int(tiles < max_ctas ? tiles : max_ctas);
    if (!(p.flags & CWRNNT_FUSED_LOG_SOFTMAX)) {
        grad_rows_sparse_kernel<T><<<grid, kStreamThreads, 0, s>>>(x, gx, p.V, p.n_rows, p.B, lx, ly, y, p.y_stride,
                                                                   p.blank, p.flags, mean_inv, w, gc, gc_stride,
                                                                   aligned ? 1 : 0);
        return cudaGetLastError();
    }
    RowShape shape{};
    if (aligned && pick_row_shape(p.V / VE, &shape)) {
#define CALL(LPR, NV)                                                                                              \
    {                                                                                                              \
        const int rpc = kStreamThreads / LPR;                                                                      \
        tiles = (p.n_rows + rpc - 1) / rpc;                                                                        \
        grid = int(tiles < max_ctas ? tiles : max_ctas);                                                           \
        grad_rows_kernel<T, LPR, NV><<<grid, kStreamThreads, 0, s>>>(x, gx, p.V, p.n_rows, p.B, lx, ly, y,         \
                                                                     p.y_stride, p.blank, p.flags, mean_inv, w, gc, \
                                                                     gc_stride);                                   \
    }
        CWRNNT_DISPATCH_SHAPE(shape, CALL);
#undef CALL
    } else {
        grad_rows_generic_kernel<T><<<grid, kStreamThreads, 0, s>>>(x, gx, p.V, p.n_rows, p.B, lx, ly, y, p.y_stride,
                                                                    p.blank, p.flags, mean_inv, w, gc, gc_stride);
    }
    return cudaGetLastError();
}

cudaError_t launch_grad(const cwrnnt_problem &p, const void *x, const int32_t *lx, const int32_t *ly,
                        const int32_t *y, const Workspace &w, const void *grad_costs, int32_t gc_stride, void *grad_x,
                        cudaStream_t s)
{
    switch (p.dtype) {
    case CWRNNT_F32:
        return launch_grad_t(p, static_cast<const float *>(x), lx, ly, y, w, grad_costs, gc_stride,
                             static_cast<float *>(grad_x), s);
    case CWRNNT_F16:
        return launch_grad_t(p, static_cast<const __half *>(x), lx, ly, y, w, grad_costs, gc_stride,
                             static_cast<__half *>(grad_x), s);
    case CWRNNT_BF16:
        return launch_grad_t(p, static_cast<const __nv_bfloat16 *>(x), lx, ly, y, w, grad_costs, gc_stride,
                             static_cast<__nv_bfloat16 *>(grad_x), s);
    case CWRNNT_F64:
        return launch_grad_t(p, static_cast<const double *>(x), lx, ly, y, w, grad_costs, gc_stride,
                             static_cast<double *>(grad_x), s);
    }
    return cudaErrorInvalidValue;
}

}  // namespace cwrnnt
