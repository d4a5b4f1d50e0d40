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
// caller's log_softmax backward. Each row is read once and written once with plain 128-bit loads and stores (the
// evict-first variants measured 7 % slower); the per-row scalars (lse, alpha, two betas) are 32 bytes against
// V*sizeof(element).
//
// Log-prob mode: the reference's own result, zeros plus the two sparse terms; the input rows are not read at all.
//
// Bound: HBM bandwidth. Algorithmic bytes: 2 * V * sizeof(element) per row (V * sizeof(element) in log-prob mode).
#include "cwrnnt_kernels.h"
#include "cwrnnt_rowmap.cuh"

namespace cwrnnt {

// Invalid lengths (fatal status): nothing upstream ran, so the rows of this launch are filled with NaN instead of being
// left as they were - a caller that never reads the status then sees the failure in the gradient itself. `rows` holds
// the host-known range of the launch (for a sequence group: its nominal row range; the ranges tile the matrix).
template <typename T>
__device__ __noinline__ void fill_rows_nan(T *__restrict__ gx, int V, const RowRange &rows)
{
    const int64_t n = (rows.end - rows.begin) * int64_t(V);
    T *base = gx + rows.begin * int64_t(V);
    const T nan = Elt<T>::from_acc(typename Elt<T>::acc(NAN));
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
        base[i] = nan;
}

__device__ __forceinline__ double occupancy(double e, float) { return double(expf(float(e))); }
__device__ __forceinline__ double occupancy(double e, double) { return exp(e); }

// Occupancy terms of one row from the saved forward state. lpb/lpl: log-probs of blank / label at this cell.
// alpha and beta are stored diagonal-major: (t,u) at rw.at, both successors side by side on the next diagonal.
template <typename CostT>
__device__ __forceinline__ void row_terms(const RowWalker &rw, const Workspace &w, double lpb, double lpl,
                                          const CostT *__restrict__ grad_costs, int gc_stride, int flags,
                                          double mean_inv, double &wb, double &wl)
{
    const double *beta_next = w.beta + rw.off + rw.next_diag();
    const double ll = __ldg(w.ll_beta + rw.n);
    const double a = __ldg(w.alpha + rw.off + rw.at);
    double eb = -INFINITY, el = -INFINITY;
    if (rw.t < rw.T - 1)
        eb = a + __ldg(beta_next) + lpb - ll;
    else if (rw.u == rw.U)
        eb = a + lpb - ll;
    if (rw.u < rw.U) el = a + __ldg(beta_next + 1) + lpl - ll;
    double g = grad_costs ? double(__ldg(grad_costs + int64_t(rw.n) * gc_stride)) : 1.0;
    g *= sequence_scale(flags, rw.T) * mean_inv;
    wb = g * occupancy(eb, CostT(0));
    wl = g * occupancy(el, CostT(0));
}

// Same row shapes and row runs as the gather kernel. No warp-wide collective is needed here: each lane scales its own
// part of the row by the row's occupancy sum. Plain (allocating) loads and stores: with the non-persistent grid the
// evict-first variants measured 7 % slower.
template <typename T, int LPR, int NV, bool FULL>
__global__ void __launch_bounds__(kStreamThreads)
grad_rows_kernel(const T *__restrict__ x, T *__restrict__ gx, int V, RowRange rows, int B,
                 const int32_t *__restrict__ lx, const int32_t *__restrict__ ly, const int32_t *__restrict__ y,
                 int y_stride, int blank, int flags, double mean_inv, Workspace w,
                 const typename Elt<T>::cost *__restrict__ grad_costs, int gc_stride, int run_len)
{
    using E = Elt<T>;
    using A = typename E::acc;
    using CostT = typename E::cost;
    constexpr int VE = E::VE;
    constexpr int GPC = kStreamThreads / LPR;
    if (w.status[0] & CWRNNT_ST_FATAL) {
        fill_rows_nan(gx, V, rows);
        return;
    }

    const int gl = threadIdx.x % LPR;
    const int nvec = V / VE;
    // A CTA covers GPC * run_len consecutive rows, one such tile per CTA (non-persistent grid, see the gather kernel);
    // it carries on gridDim.x tiles further only when the range (known on the device alone) outgrew the grid.
    int64_t r_begin, r_end;
    rows.resolve(r_begin, r_end);
    const int64_t tile_rows = int64_t(GPC) * run_len;
    bool ignored = false;

    RowWalker rw;
    for (int64_t tile = r_begin + blockIdx.x * tile_rows; tile < r_end; tile += gridDim.x * tile_rows) {
        const int64_t first = tile + (threadIdx.x / LPR) * run_len;
        const int64_t limit = first + run_len < r_end ? first + run_len : r_end;
        for (int64_t r = first; r < limit; ++r) {
            if (r == first) rw.start(r, w.off, B, lx, ly);
            const T *row = x + r * int64_t(V);
            T *orow = gx + r * int64_t(V);
            const uint4 *rv = reinterpret_cast<const uint4 *>(row);
            uint4 *ov = reinterpret_cast<uint4 *>(orow);
            uint4 v[NV];
#pragma unroll
            for (int j = 0; j < NV; ++j)
                if (FULL || j * LPR + gl < nvec) v[j] = ld_nc(rv + j * LPR + gl);
            const int label = rw.label(y, y_stride, V, ignored);
            const A xb = E::to_acc(__ldg(row + blank));
            const A xl = label >= 0 ? E::to_acc(__ldg(row + label)) : A(0);
            const double lse = __ldg(w.lse + r);
            double wb, wl;
            row_terms<CostT>(rw, w, double(xb) - lse, double(xl) - lse, grad_costs, gc_stride, flags, mean_inv, wb,
                             wl);
            const A tot = A(wb + wl);
            const A lse_a = A(lse);
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                if (FULL || j * LPR + gl < nvec) {
                    A e[VE];
                    E::unpack(v[j], e);
#pragma unroll
                    for (int c = 0; c < VE; ++c) e[c] = exp_shifted(e[c], lse_a) * tot;
                    ov[j * LPR + gl] = E::pack(e);
                }
            }
            // the two sparse corrections, by the lane that stored the enclosing vector (same-thread program order)
            if ((blank / VE) % LPR == gl) {
                A gb = exp_shifted(xb, lse_a) * tot - A(wb);
                if (label == blank) gb -= A(wl);
                orow[blank] = E::from_acc(gb);
            }
            if (label >= 0 && label != blank && (label / VE) % LPR == gl)
                orow[label] = E::from_acc(exp_shifted(xl, lse_a) * tot - A(wl));
            rw.advance(w.off, B, lx, ly);
        }
    }
}

// Rows beyond the register-resident shapes (more than 512 vectors): one warp per row, the row in segments of 32 lanes
// x 8 vectors. The gradient is element-wise once the row's scalars are known, so nothing is carried between segments.
template <typename T>
__global__ void __launch_bounds__(kStreamThreads)
grad_rows_long_kernel(const T *__restrict__ x, T *__restrict__ gx, int V, RowRange rows, int B,
                      const int32_t *__restrict__ lx, const int32_t *__restrict__ ly, const int32_t *__restrict__ y,
                      int y_stride, int blank, int flags, double mean_inv, Workspace w,
                      const typename Elt<T>::cost *__restrict__ grad_costs, int gc_stride, int run_len)
{
    using E = Elt<T>;
    using A = typename E::acc;
    using CostT = typename E::cost;
    constexpr int VE = E::VE;
    constexpr int NV = 8;
    constexpr int kWarps = kStreamThreads / 32;
    if (w.status[0] & CWRNNT_ST_FATAL) {
        fill_rows_nan(gx, V, rows);
        return;
    }

    const int lane = threadIdx.x & 31;
    const int nvec = V / VE;
    int64_t r_begin, r_end;
    rows.resolve(r_begin, r_end);
    const int64_t tile_rows = int64_t(kWarps) * run_len;
    bool ignored = false;

    RowWalker rw;
    for (int64_t tile = r_begin + blockIdx.x * tile_rows; tile < r_end; tile += gridDim.x * tile_rows) {
        const int64_t first = tile + (threadIdx.x >> 5) * run_len;
        const int64_t limit = first + run_len < r_end ? first + run_len : r_end;
        for (int64_t r = first; r < limit; ++r) {
            if (r == first) rw.start(r, w.off, B, lx, ly);
            const T *row = x + r * int64_t(V);
            T *orow = gx + r * int64_t(V);
            const uint4 *rv = reinterpret_cast<const uint4 *>(row);
            uint4 *ov = reinterpret_cast<uint4 *>(orow);
            const int label = rw.label(y, y_stride, V, ignored);
            const A xb = E::to_acc(__ldg(row + blank));
            const A xl = label >= 0 ? E::to_acc(__ldg(row + label)) : A(0);
            const double lse = __ldg(w.lse + r);
            double wb, wl;
            row_terms<CostT>(rw, w, double(xb) - lse, double(xl) - lse, grad_costs, gc_stride, flags, mean_inv, wb,
                             wl);
            const A tot = A(wb + wl);
            const A lse_a = A(lse);
            for (int seg = 0; seg < nvec; seg += 32 * NV) {
                uint4 v[NV];
#pragma unroll
                for (int j = 0; j < NV; ++j)
                    if (seg + j * 32 + lane < nvec) v[j] = ld_nc(rv + seg + j * 32 + lane);
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    if (seg + j * 32 + lane < nvec) {
                        A e[VE];
                        E::unpack(v[j], e);
#pragma unroll
                        for (int c = 0; c < VE; ++c) e[c] = exp_shifted(e[c], lse_a) * tot;
                        ov[seg + j * 32 + lane] = E::pack(e);
                    }
                }
            }
            // the two sparse corrections, by the lane that stored the enclosing vector (same-thread program order)
            if ((blank / VE) % 32 == lane) {
                A gb = exp_shifted(xb, lse_a) * tot - A(wb);
                if (label == blank) gb -= A(wl);
                orow[blank] = E::from_acc(gb);
            }
            if (label >= 0 && label != blank && (label / VE) % 32 == lane)
                orow[label] = E::from_acc(exp_shifted(xl, lse_a) * tot - A(wl));
            rw.advance(w.off, B, lx, ly);
        }
    }
}

// Any V / alignment, logits mode: one warp per row, scalar coalesced accesses.
template <typename T>
__global__ void __launch_bounds__(kStreamThreads)
grad_rows_generic_kernel(const T *__restrict__ x, T *__restrict__ gx, int V, RowRange rows, int B,
                         const int32_t *__restrict__ lx, const int32_t *__restrict__ ly,
                         const int32_t *__restrict__ y, int y_stride, int blank, int flags, double mean_inv,
                         Workspace w, const typename Elt<T>::cost *__restrict__ grad_costs, int gc_stride)
{
    using E = Elt<T>;
    using A = typename E::acc;
    using CostT = typename E::cost;
    if (w.status[0] & CWRNNT_ST_FATAL) {
        fill_rows_nan(gx, V, rows);
        return;
    }
    const int lane = threadIdx.x & 31;
    int64_t row0, row1;
    rows.resolve(row0, row1);
    const int64_t n_warps = (int64_t(gridDim.x) * kStreamThreads) >> 5;
    const int64_t per_warp = (row1 - row0 + n_warps - 1) / n_warps;
    const int64_t r_begin = row0 + ((int64_t(blockIdx.x) * kStreamThreads + threadIdx.x) >> 5) * per_warp;
    const int64_t r_end = r_begin + per_warp < row1 ? r_begin + per_warp : row1;
    if (r_begin >= r_end) return;
    bool ignored = false;
    RowWalker rw;
    rw.start(r_begin, w.off, B, lx, ly);
    for (int64_t r = r_begin; r < r_end; ++r) {
        const T *row = x + r * int64_t(V);
        T *orow = gx + r * int64_t(V);
        const int label = rw.label(y, y_stride, V, ignored);
        const A xb = E::to_acc(__ldg(row + blank));
        const A xl = label >= 0 ? E::to_acc(__ldg(row + label)) : A(0);
        const double lse = __ldg(w.lse + r);
        double wb, wl;
        row_terms<CostT>(rw, w, double(xb) - lse, double(xl) - lse, grad_costs, gc_stride, flags, mean_inv, wb, wl);
        const A tot = A(wb + wl), lse_a = A(lse);
        for (int k = lane; k < V; k += 32) {
            A g = exp_shifted(E::to_acc(__ldg(row + k)), lse_a) * tot;
            if (k == blank) g -= A(wb);
            if (k == label) g -= A(wl);
            orow[k] = E::from_acc(g);
        }
        rw.advance(w.off, B, lx, ly);
    }
}

// Log-prob mode: zeros and the two sparse terms; the input is only touched at two elements per row.
template <typename T>
__global__ void __launch_bounds__(kStreamThreads)
grad_rows_sparse_kernel(const T *__restrict__ x, T *__restrict__ gx, int V, RowRange rows, int B,
                        const int32_t *__restrict__ lx, const int32_t *__restrict__ ly,
                        const int32_t *__restrict__ y, int y_stride, int blank, int flags, double mean_inv,
                        Workspace w, const typename Elt<T>::cost *__restrict__ grad_costs, int gc_stride, int vec_ok)
{
    using E = Elt<T>;
    using A = typename E::acc;
    using CostT = typename E::cost;
    constexpr int VE = E::VE;
    if (w.status[0] & CWRNNT_ST_FATAL) {
        fill_rows_nan(gx, V, rows);
        return;
    }
    const int lane = threadIdx.x & 31;
    int64_t row0, row1;
    rows.resolve(row0, row1);
    const int64_t n_warps = (int64_t(gridDim.x) * kStreamThreads) >> 5;
    const int64_t per_warp = (row1 - row0 + n_warps - 1) / n_warps;
    const int64_t r_begin = row0 + ((int64_t(blockIdx.x) * kStreamThreads + threadIdx.x) >> 5) * per_warp;
    const int64_t r_end = r_begin + per_warp < row1 ? r_begin + per_warp : row1;
    if (r_begin >= r_end) return;
    bool ignored = false;
    RowWalker rw;
    rw.start(r_begin, w.off, B, lx, ly);
    for (int64_t r = r_begin; r < r_end; ++r) {
        const T *row = x + r * int64_t(V);
        T *orow = gx + r * int64_t(V);
        const int label = rw.label(y, y_stride, V, ignored);
        const A xb = E::to_acc(__ldg(row + blank));
        const A xl = label >= 0 ? E::to_acc(__ldg(row + label)) : A(0);
        double wb, wl;
        row_terms<CostT>(rw, w, double(xb), double(xl), grad_costs, gc_stride, flags, mean_inv, wb, wl);
        if (vec_ok) {
            uint4 *ov = reinterpret_cast<uint4 *>(orow);
            const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
            for (int idx = lane; idx < V / VE; idx += 32) st_stream(ov + idx, zero);
            // the lane that zeroed the enclosing vector writes the sparse term afterwards
            if ((blank / VE) % 32 == lane) orow[blank] = E::from_acc(A(-(wb + (label == blank ? wl : 0.0))));
            if (label >= 0 && label != blank && (label / VE) % 32 == lane) orow[label] = E::from_acc(A(-wl));
        } else {
            for (int k = lane; k < V; k += 32) {
                A g = A(0);
                if (k == blank) g -= A(wb);
                if (k == label) g -= A(wl);
                orow[k] = E::from_acc(g);
            }
        }
        rw.advance(w.off, B, lx, ly);
    }
}

// A launch of a streaming kernel, optionally at the device's LOWEST priority whatever the stream's own (launch
// attribute): in a pipelined step the gradient of a group follows the group's wavefront on that wavefront's
// high-priority stream, and must not take SM slots from the wavefront CTAs of other groups that are still arriving.
template <typename... KArgs, typename... Args>
static void launch_rows(void (*kernel)(KArgs...), unsigned grid, cudaStream_t s, bool lowest_priority, Args... args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kStreamThreads);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    if (lowest_priority) {
        static const int lowest = [] {
            int least = 0, greatest = 0;
            return cudaDeviceGetStreamPriorityRange(&least, &greatest) == cudaSuccess ? least : 0;
        }();
        attr[0].id = cudaLaunchAttributePriority;
        attr[0].val.priority = lowest;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);  // errors are picked up by cudaGetLastError below
}

template <typename T>
static cudaError_t launch_grad_t(const cwrnnt_problem &p, const T *x, const int32_t *lx, const int32_t *ly,
                                 const int32_t *y, const Workspace &w, const void *grad_costs, int32_t gc_stride,
                                 T *gx, cudaStream_t s, const GradRows &span)
{
    using CostT = typename Elt<T>::cost;
    if (p.n_rows == 0) return cudaSuccess;
    // rows of this launch: everything, or a sequence group whose bounds only the device knows; the grid is then
    // sized for span.grid_rows rows (the kernels cope with a longer range, more slowly)
    const RowRange rows{span.device_range ? span.nominal_begin : 0, span.device_range ? span.nominal_end : p.n_rows,
                        span.device_range};
    const int64_t n_rows = span.device_range ? (span.grid_rows < p.n_rows ? span.grid_rows : p.n_rows) : p.n_rows;
    if (n_rows <= 0) return cudaSuccess;
    constexpr int VE = Elt<T>::VE;
    const CostT *gc = static_cast<const CostT *>(grad_costs);
    const double mean_inv =
        (p.flags & CWRNNT_REDUCE_MEAN) ? 1.0 / double(p.mean_denominator > 0 ? p.mean_denominator : p.B) : 1.0;
    const bool aligned = (p.V % VE == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                         (reinterpret_cast<uintptr_t>(gx) % 16 == 0);
    if (!(p.flags & CWRNNT_FUSED_LOG_SOFTMAX)) {
        const unsigned grid = tiled_grid(n_rows, 8 * 4);  // 8 warps, 4 rows each
        grad_rows_sparse_kernel<T><<<grid, kStreamThreads, 0, s>>>(x, gx, p.V, rows, p.B, lx, ly, y, p.y_stride,
                                                                   p.blank, p.flags, mean_inv, w, gc, gc_stride,
                                                                   aligned ? 1 : 0);
        return cudaGetLastError();
    }
    RowShape shape{};
    if (aligned && !pick_row_shape(p.V / VE, &shape)) {
        const int run_len = 4;  // long rows, in 4 KB segments: 32 rows per CTA
        const unsigned grid = tiled_grid(n_rows, int64_t(kStreamThreads / 32) * run_len);
        launch_rows(grad_rows_long_kernel<T>, grid, s, span.lowest_priority, x, gx, p.V, rows, p.B, lx, ly, y,
                    p.y_stride, p.blank, p.flags, mean_inv, w, gc, gc_stride, run_len);
    } else if (aligned && pick_row_shape(p.V / VE, &shape)) {
        const bool full = (p.V / VE) == shape.lpr * shape.nv;
        // rows per lane group, measured 1..32 on B200: a tile of 8 rows x 4 KB (run 1) or 16 rows x 2 KB (run 2)
        // per CTA streams best for the mixed read/write pattern; short rows are bound by per-row instructions and
        // want longer runs, and so do 8 KB rows, whose 16 vector registers per lane leave few warps per SM
        const int64_t row_bytes = int64_t(p.V) * int64_t(sizeof(T));
        const int run_len = row_bytes >= 8192 ? 8 : (row_bytes >= 4096 ? 1 : (row_bytes >= 2048 ? 2 : 8));
#define LAUNCH(LPR, NV, FULL)                                                                                    \
    {                                                                                                            \
        const unsigned grid = tiled_grid(n_rows, int64_t(kStreamThreads / LPR) * run_len);                       \
        launch_rows(grad_rows_kernel<T, LPR, NV, FULL>, grid, s, span.lowest_priority, x, gx, p.V, rows, p.B,    \
                    lx, ly, y, p.y_stride, p.blank, p.flags, mean_inv, w, gc, gc_stride, run_len);               \
    }
#define CALL(LPR, NV)                    \
    {                                    \
        if (full) LAUNCH(LPR, NV, true)  \
        else LAUNCH(LPR, NV, false)      \
    }
        CWRNNT_DISPATCH_SHAPE(shape, CALL);
#undef CALL
#undef LAUNCH
    } else {
        const unsigned grid = tiled_grid(n_rows, 8 * 4);
        grad_rows_generic_kernel<T><<<grid, kStreamThreads, 0, s>>>(x, gx, p.V, rows, p.B, lx, ly, y, p.y_stride,
                                                                    p.blank, p.flags, mean_inv, w, gc, gc_stride);
    }
    return cudaGetLastError();
}

// In-place scaling of a gradient that was computed for an upstream gradient of 1 (cwrnnt_loss_grad). The usual
// upstream gradient of a training loss IS 1: every thread reads the factor first and leaves if there is nothing to do,
// so that case costs one empty launch and no memory traffic.
template <typename T>
__global__ void __launch_bounds__(kStreamThreads)
scale_kernel(T *__restrict__ g, int64_t n, const typename Elt<T>::cost *__restrict__ factor)
{
    using E = Elt<T>;
    using A = typename E::acc;
    constexpr int VE = E::VE;
    const A f = A(__ldg(factor));
    if (f == A(1)) return;
    const int64_t stride = int64_t(gridDim.x) * kStreamThreads;
    const int64_t tid = int64_t(blockIdx.x) * kStreamThreads + threadIdx.x;
    const int64_t head = reinterpret_cast<uintptr_t>(g) % 16 ? n : 0;  // unaligned base: everything element-wise
    const int64_t nvec = (n - head) / VE;
    uint4 *gv = reinterpret_cast<uint4 *>(g + head);
    for (int64_t i = tid; i < nvec; i += stride) {
        A e[VE];
        E::unpack(gv[i], e);
#pragma unroll
        for (int c = 0; c < VE; ++c) e[c] *= f;
        gv[i] = E::pack(e);
    }
    for (int64_t i = (head ? 0 : nvec * VE) + tid; i < n; i += stride) g[i] = E::from_acc(E::to_acc(g[i]) * f);
}

template <typename T>
static cudaError_t launch_scale_t(const cwrnnt_problem &p, T *g, const void *factor, cudaStream_t s)
{
    const int64_t n = p.n_rows * int64_t(p.V);
    if (n == 0) return cudaSuccess;
    const int64_t want = (n / Elt<T>::VE + kStreamThreads - 1) / kStreamThreads;
    const int grid = int(want < 1 ? 1 : (want < kNumSMs * 16 ? want : kNumSMs * 16));
    scale_kernel<T><<<grid, kStreamThreads, 0, s>>>(g, n, static_cast<const typename Elt<T>::cost *>(factor));
    return cudaGetLastError();
}

cudaError_t launch_scale(const cwrnnt_problem &p, void *grad_x, const void *factor, cudaStream_t s)
{
    switch (p.dtype) {
    case CWRNNT_F32: return launch_scale_t(p, static_cast<float *>(grad_x), factor, s);
    case CWRNNT_F16: return launch_scale_t(p, static_cast<__half *>(grad_x), factor, s);
    case CWRNNT_BF16: return launch_scale_t(p, static_cast<__nv_bfloat16 *>(grad_x), factor, s);
    case CWRNNT_F64: return launch_scale_t(p, static_cast<double *>(grad_x), factor, s);
    }
    return cudaErrorInvalidValue;
}

cudaError_t launch_grad(const cwrnnt_problem &p, const void *x, const int32_t *lx, const int32_t *ly,
                        const int32_t *y, const Workspace &w, const void *grad_costs, int32_t gc_stride, void *grad_x,
                        cudaStream_t s, const GradRows &span)
{
    switch (p.dtype) {
    case CWRNNT_F32:
        return launch_grad_t(p, static_cast<const float *>(x), lx, ly, y, w, grad_costs, gc_stride,
                             static_cast<float *>(grad_x), s, span);
    case CWRNNT_F16:
        return launch_grad_t(p, static_cast<const __half *>(x), lx, ly, y, w, grad_costs, gc_stride,
                             static_cast<__half *>(grad_x), s, span);
    case CWRNNT_BF16:
        return launch_grad_t(p, static_cast<const __nv_bfloat16 *>(x), lx, ly, y, w, grad_costs, gc_stride,
                             static_cast<__nv_bfloat16 *>(grad_x), s, span);
    case CWRNNT_F64:
        return launch_grad_t(p, static_cast<const double *>(x), lx, ly, y, w, grad_costs, gc_stride,
                             static_cast<double *>(grad_x), s, span);
    }
    return cudaErrorInvalidValue;
}

}  // namespace cwrnnt
