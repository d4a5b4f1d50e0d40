// K1 - fused row-wise log-sum-exp over V and blank/label log-prob gather.
//
// Replaces, on the reference path, the caller's log_softmax (test/test.py:19-20) and gather_cuda_kernel
// (cwarp_cuda_gather_kernel.cu:19-43): each [V] row is read exactly once with 128-bit coalesced loads, reduced with
// warp shuffles, and 24 bytes come out (lse, log P(blank), log P(label)). The reference kernel reads two elements per
// 4 KB row, one 32-byte sector each, with neighbouring threads (U+1)*V elements apart.
//
// Bound: HBM read bandwidth. Algorithmic bytes: V * sizeof(element) per row.
#include "cwrnnt_kernels.h"
#include "cwrnnt_rowmap.cuh"

namespace cwrnnt {

// LPR lanes hold one row in registers (NV vectors of 16 bytes each); 32/LPR rows per warp. Every lane group owns a
// short contiguous run of rows, so its lattice position is found once and then advanced incrementally.
// FULL: the row fills all LPR*NV vector slots (no per-vector predicate).
template <typename T, int LPR, int NV, bool FULL>
__global__ void __launch_bounds__(kStreamThreads)
gather_rows_kernel(const T *__restrict__ x, int V, RowRange rows, int B, const int32_t *__restrict__ lx,
                   const int32_t *__restrict__ ly, const int32_t *__restrict__ y, int y_stride, int blank,
                   Workspace w, int run_len)
{
    using E = Elt<T>;
    using A = typename E::acc;
    constexpr int VE = E::VE;
    constexpr int GPC = kStreamThreads / LPR;  // lane groups per CTA
    if (w.status[0] & CWRNNT_ST_FATAL) return;

    const int gl = threadIdx.x % LPR;  // lane within the row group
    const int nvec = V / VE;
    // A CTA covers GPC * run_len consecutive rows: lane group g takes the run_len rows starting at
    // (blockIdx.x * GPC + g) * run_len. The grid is NOT persistent - one such tile per CTA, dispatched in order by
    // the hardware, so that the CTAs in flight sweep the matrix as one front (measured: 15 % more bandwidth than a
    // persistent grid-stride loop on this access pattern). Only a range whose length the host did not know can be
    // longer than the grid; its CTAs then carry on with the tile gridDim.x further.
    int64_t r_begin, r_end;
    rows.resolve(r_begin, r_end);
    const int64_t tile_rows = int64_t(GPC) * run_len;
    bool any_bad = false;

    RowWalker rw;
    for (int64_t tile = r_begin + blockIdx.x * tile_rows; tile < r_end; tile += gridDim.x * tile_rows) {
        const int64_t first = tile + (threadIdx.x / LPR) * run_len;
        const int64_t limit = first + run_len < r_end ? first + run_len : r_end;
        for (int i = 0; i < run_len; ++i) {  // same trip count for every group of the warp (shuffles below)
            const int64_t r = first + i;
            const bool live = r < limit;
            uint4 v[NV];
            A xb = A(0), xl = A(0);
            int label = -1;
            if (live) {
                if (i == 0) rw.start(r, w.off, B, lx, ly);
                const T *row = x + r * int64_t(V);
                const uint4 *rv = reinterpret_cast<const uint4 *>(row);
#pragma unroll
                for (int j = 0; j < NV; ++j)
                    if (FULL || j * LPR + gl < nvec) v[j] = ld_nc(rv + j * LPR + gl);
                label = rw.label(y, y_stride, V, any_bad);
                xb = E::to_acc(__ldg(row + blank));
                if (label >= 0) xl = E::to_acc(__ldg(row + label));
            }
            A mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                if (live && (FULL || j * LPR + gl < nvec)) {
                    const A m = E::vec_max(v[j]);
                    mx = m > mx ? m : mx;
                }
            }
            mx = group_max<LPR>(mx);
            const RowShift<A> shift(mx);
            A sum = A(0);
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                if (live && (FULL || j * LPR + gl < nvec)) {
                    A e[VE];
                    E::unpack(v[j], e);
#pragma unroll
                    for (int c = 0; c < VE; ++c) sum += shift.term(e[c]);
                }
            }
            sum = group_sum<LPR>(sum);
            if (live) {
                if (gl == 0) {
                    const double lse = shift.lse(sum);
                    const int64_t at = rw.off + rw.at;
                    w.lse[r] = lse;
                    w.lp_blank[at] = double(xb) - lse;
                    if (label >= 0) w.lp_label[at] = double(xl) - lse;
                }
                rw.advance(w.off, B, lx, ly);
            }
        }
    }
    if (any_bad) atomicOr(w.status, CWRNNT_ST_BAD_LABEL);
}

// Rows beyond the register-resident shapes (more than 512 vectors: V > 2048 floats, > 4096 halves): one warp per row,
// the row passing through the registers in segments of 32 lanes x 8 vectors (4 KB). Every segment gets its own shifted
// sum and its own log-sum-exp in double; segments combine as log(exp(a) + exp(b)) in double. Any vector-aligned V,
// however long. (For 8 KB rows the one-piece shape {32,16} is faster: 1.46 against 1.98 ms on 5.1 GB of bfloat16 -
// the segments' reductions run one after the other - so this kernel starts where that shape ends.)
template <typename T>
__global__ void __launch_bounds__(kStreamThreads)
gather_rows_long_kernel(const T *__restrict__ x, int V, RowRange rows, int B, const int32_t *__restrict__ lx,
                        const int32_t *__restrict__ ly, const int32_t *__restrict__ y, int y_stride, int blank,
                        Workspace w, int run_len)
{
    using E = Elt<T>;
    using A = typename E::acc;
    constexpr int VE = E::VE;
    constexpr int NV = 8;
    constexpr int kWarps = kStreamThreads / 32;
    if (w.status[0] & CWRNNT_ST_FATAL) return;

    const int lane = threadIdx.x & 31;
    const int nvec = V / VE;
    int64_t r_begin, r_end;
    rows.resolve(r_begin, r_end);
    const int64_t tile_rows = int64_t(kWarps) * run_len;
    bool any_bad = false;

    RowWalker rw;
    for (int64_t tile = r_begin + blockIdx.x * tile_rows; tile < r_end; tile += gridDim.x * tile_rows) {
        const int64_t first = tile + (threadIdx.x >> 5) * run_len;
        const int64_t limit = first + run_len < r_end ? first + run_len : r_end;
        for (int64_t r = first; r < limit; ++r) {  // a warp owns its rows: no shuffle crosses a row boundary
            if (r == first) rw.start(r, w.off, B, lx, ly);
            const T *row = x + r * int64_t(V);
            const uint4 *rv = reinterpret_cast<const uint4 *>(row);
            const int label = rw.label(y, y_stride, V, any_bad);
            const A xb = E::to_acc(__ldg(row + blank));
            const A xl = label >= 0 ? E::to_acc(__ldg(row + label)) : A(0);
            double lse = -INFINITY;
            for (int seg = 0; seg < nvec; seg += 32 * NV) {
                uint4 v[NV];
#pragma unroll
                for (int j = 0; j < NV; ++j)
                    if (seg + j * 32 + lane < nvec) v[j] = ld_nc(rv + seg + j * 32 + lane);
                A mx = -INFINITY;
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    if (seg + j * 32 + lane < nvec) {
                        const A m = E::vec_max(v[j]);
                        mx = m > mx ? m : mx;
                    }
                }
                mx = group_max<32>(mx);
                const RowShift<A> shift(mx);
                A sum = A(0);
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    if (seg + j * 32 + lane < nvec) {
                        A e[VE];
                        E::unpack(v[j], e);
#pragma unroll
                        for (int c = 0; c < VE; ++c) sum += shift.term(e[c]);
                    }
                }
                sum = group_sum<32>(sum);
                const double seg_lse = shift.lse(sum);  // every segment holds at least one element: sum >= 1
                const double hi = fmax(lse, seg_lse), lo = fmin(lse, seg_lse);
                lse = lo == -INFINITY ? hi : hi + log1p(exp(lo - hi));
            }
            if (lane == 0) {
                const int64_t at = rw.off + rw.at;
                w.lse[r] = lse;
                w.lp_blank[at] = double(xb) - lse;
                if (label >= 0) w.lp_label[at] = double(xl) - lse;
            }
            rw.advance(w.off, B, lx, ly);
        }
    }
    if (any_bad) atomicOr(w.status, CWRNNT_ST_BAD_LABEL);
}

// Any V, any alignment: one warp per row, two coalesced scalar passes (the second hits L1/L2).
template <typename T>
__global__ void __launch_bounds__(kStreamThreads)
gather_rows_generic_kernel(const T *__restrict__ x, int V, RowRange rows, int B, const int32_t *__restrict__ lx,
                           const int32_t *__restrict__ ly, const int32_t *__restrict__ y, int y_stride, int blank,
                           Workspace w)
{
    using E = Elt<T>;
    using A = typename E::acc;
    if (w.status[0] & CWRNNT_ST_FATAL) return;
    const int lane = threadIdx.x & 31;
    int64_t row0, row1;
    rows.resolve(row0, row1);
    const int64_t n_warps = (int64_t(gridDim.x) * kStreamThreads) >> 5;
    const int64_t per_warp = (row1 - row0 + n_warps - 1) / n_warps;
    const int64_t r_begin = row0 + ((int64_t(blockIdx.x) * kStreamThreads + threadIdx.x) >> 5) * per_warp;
    const int64_t r_end = r_begin + per_warp < row1 ? r_begin + per_warp : row1;
    bool any_bad = false;
    RowWalker rw;
    if (r_begin < r_end) rw.start(r_begin, w.off, B, lx, ly);
    for (int64_t r = r_begin; r < r_end; ++r) {
        const int label = rw.label(y, y_stride, V, any_bad);
        const T *row = x + r * int64_t(V);
        A mx = -INFINITY;
        for (int k = lane; k < V; k += 32) {
            A e = E::to_acc(__ldg(row + k));
            mx = e > mx ? e : mx;
        }
        mx = group_max<32>(mx);
        const RowShift<A> shift(mx);
        A sum = A(0);
        for (int k = lane; k < V; k += 32) sum += shift.term(E::to_acc(__ldg(row + k)));
        sum = group_sum<32>(sum);
        if (lane == 0) {
            const double lse = shift.lse(sum);
            const int64_t at = rw.off + rw.at;
            w.lse[r] = lse;
            w.lp_blank[at] = double(E::to_acc(__ldg(row + blank))) - lse;
            if (label >= 0) w.lp_label[at] = double(E::to_acc(__ldg(row + label))) - lse;
        }
        rw.advance(w.off, B, lx, ly);
    }
    if (any_bad) atomicOr(w.status, CWRNNT_ST_BAD_LABEL);
}

// Log-probability input (the reference contract): no normalisation, two elements per row, one thread per row run.
template <typename T>
__global__ void __launch_bounds__(kStreamThreads)
gather_pair_kernel(const T *__restrict__ x, int V, RowRange rows, int B, const int32_t *__restrict__ lx,
                   const int32_t *__restrict__ ly, const int32_t *__restrict__ y, int y_stride, int blank,
                   Workspace w)
{
    using E = Elt<T>;
    if (w.status[0] & CWRNNT_ST_FATAL) return;
    bool any_bad = false;
    // consecutive threads take consecutive rows (the two 8-byte results per row then coalesce per warp); each thread
    // strides by the grid size, so its position is re-located per row
    int64_t row0, row1;
    rows.resolve(row0, row1);
    const int64_t stride = int64_t(gridDim.x) * kStreamThreads;
    for (int64_t r = row0 + int64_t(blockIdx.x) * kStreamThreads + threadIdx.x; r < row1; r += stride) {
        RowWalker rw;
        rw.start(r, w.off, B, lx, ly);
        const int label = rw.label(y, y_stride, V, any_bad);
        const T *row = x + r * int64_t(V);
        const int64_t at = rw.off + rw.at;
        w.lse[r] = 0.0;
        w.lp_blank[at] = double(E::to_acc(__ldg(row + blank)));
        if (label >= 0) w.lp_label[at] = double(E::to_acc(__ldg(row + label)));
    }
    if (any_bad) atomicOr(w.status, CWRNNT_ST_BAD_LABEL);
}

template <typename T>
static cudaError_t launch_gather_t(const cwrnnt_problem &p, const T *x, const int32_t *lx, const int32_t *ly,
                                   const int32_t *y, const Workspace &w, cudaStream_t s, int64_t row0, int64_t row1)
{
    if (row1 <= row0) return cudaSuccess;
    const int64_t n_rows = row1 - row0;
    const RowRange rows{row0, row1, nullptr};
    constexpr int VE = Elt<T>::VE;
    if (!(p.flags & CWRNNT_FUSED_LOG_SOFTMAX)) {
        const int64_t tiles = (n_rows + kStreamThreads - 1) / kStreamThreads;
        const int grid = int(tiles < kNumSMs * 8 ? tiles : kNumSMs * 8);
        gather_pair_kernel<T><<<grid, kStreamThreads, 0, s>>>(x, p.V, rows, p.B, lx, ly, y, p.y_stride, p.blank, w);
        return cudaGetLastError();
    }
    RowShape shape{};
    const bool aligned = (p.V % VE == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0);
    const bool vec_ok = aligned && pick_row_shape(p.V / VE, &shape);
    if (aligned && !vec_ok) {
        // long rows, in 4 KB segments; 8 rows per warp keep a CTA's tile at 64 rows
        const int run_len = 8;
        const unsigned grid = tiled_grid(n_rows, int64_t(kStreamThreads / 32) * run_len);
        gather_rows_long_kernel<T><<<grid, kStreamThreads, 0, s>>>(x, p.V, rows, p.B, lx, ly, y, p.y_stride, p.blank,
                                                                   w, run_len);
    } else if (vec_ok) {
        const bool full = (p.V / VE) == shape.lpr * shape.nv;
        // rows per lane group: long enough to amortise locating the run's first row (bisection, one division),
        // short enough that the CTAs in flight stay one compact front in memory (measured 1..32: 8 is best from
        // 256-byte to 4 KB rows, 16 for 8 KB rows)
        const int run_len = int64_t(p.V) * int64_t(sizeof(T)) >= 8192 ? 16 : 8;
#define LAUNCH(LPR, NV, FULL)                                                                                      \
    {                                                                                                              \
        const unsigned grid = tiled_grid(n_rows, int64_t(kStreamThreads / LPR) * run_len);                         \
        gather_rows_kernel<T, LPR, NV, FULL><<<grid, kStreamThreads, 0, s>>>(                                      \
            x, p.V, rows, p.B, lx, ly, y, p.y_stride, p.blank, w, run_len);                                        \
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
        const unsigned grid = tiled_grid(n_rows, 8 * 4);  // 8 warps, 4 rows each
        gather_rows_generic_kernel<T><<<grid, kStreamThreads, 0, s>>>(x, p.V, rows, p.B, lx, ly, y, p.y_stride,
                                                                      p.blank, w);
    }
    return cudaGetLastError();
}

cudaError_t launch_gather(const cwrnnt_problem &p, const void *x, const int32_t *lx, const int32_t *ly,
                          const int32_t *y, const Workspace &w, cudaStream_t s, int64_t row0, int64_t row1)
{
    if (row1 < 0) row1 = p.n_rows;
    switch (p.dtype) {
    case CWRNNT_F32: return launch_gather_t(p, static_cast<const float *>(x), lx, ly, y, w, s, row0, row1);
    case CWRNNT_F16: return launch_gather_t(p, static_cast<const __half *>(x), lx, ly, y, w, s, row0, row1);
    case CWRNNT_BF16: return launch_gather_t(p, static_cast<const __nv_bfloat16 *>(x), lx, ly, y, w, s, row0, row1);
    case CWRNNT_F64: return launch_gather_t(p, static_cast<const double *>(x), lx, ly, y, w, s, row0, row1);
    }
    return cudaErrorInvalidValue;
}

}  // namespace cwrnnt
