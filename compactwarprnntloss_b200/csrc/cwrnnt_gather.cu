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

// LPR lanes hold one row in registers (NV vectors of 16 bytes each); 32/LPR rows per warp.
template <typename T, int LPR, int NV>
__global__ void __launch_bounds__(kStreamThreads)
gather_rows_kernel(const T *__restrict__ x, int V, int64_t n_rows, int B, const int32_t *__restrict__ lx,
                   const int32_t *__restrict__ ly, const int32_t *__restrict__ y, int y_stride, int blank,
                   Workspace w)
{
    using E = Elt<T>;
    using A = typename E::acc;
    constexpr int VE = E::VE;
    constexpr int RPC = kStreamThreads / LPR;  // rows per CTA tile
    if (w.status[0] & CWRNNT_ST_FATAL) return;

    const int gl = threadIdx.x % LPR;     // lane within the row group
    const int grp = threadIdx.x / LPR;    // row slot within the CTA tile
    const int nvec = V / VE;
    const int64_t n_tiles = (n_rows + RPC - 1) / RPC;
    int cursor = 0;
    bool any_bad = false;

    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int64_t r = tile * RPC + grp;
        const bool live = r < n_rows;
        RowInfo ri{};
        uint4 v[NV];
        A xb = A(0), xl = A(0);
        if (live) {
            ri = locate_row(r, cursor, w.off, B, lx, ly, y, y_stride, V);
            const T *row = x + r * int64_t(V);
            const uint4 *rv = reinterpret_cast<const uint4 *>(row);
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const int idx = j * LPR + gl;
                if (idx < nvec) v[j] = ld_nc(rv + idx);
            }
            xb = E::to_acc(__ldg(row + blank));
            if (ri.label >= 0) xl = E::to_acc(__ldg(row + ri.label));
            any_bad |= ri.bad_label;
        }
        A mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            if (live && j * LPR + gl < nvec) {
                A e[VE];
                E::unpack(v[j], e);
#pragma unroll
                for (int c = 0; c < VE; ++c) mx = e[c] > mx ? e[c] : mx;
            }
        }
        mx = group_max<LPR>(mx);
        const RowShift<A> shift(mx);
        A sum = A(0);
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            if (live && j * LPR + gl < nvec) {
                A e[VE];
                E::unpack(v[j], e);
#pragma unroll
                for (int c = 0; c < VE; ++c) sum += shift.term(e[c]);
            }
        }
        sum = group_sum<LPR>(sum);
        if (live && gl == 0) {
            const double lse = shift.lse(sum);
            const int64_t at = ri.off + diag_index(ri.t, ri.u, ri.T, ri.U + 1);
            w.lse[r] = lse;
            w.lp_blank[at] = double(xb) - lse;
            if (ri.label >= 0) w.lp_label[at] = double(xl) - lse;
        }
    }
    if (any_bad) atomicOr(w.status, CWRNNT_ST_BAD_LABEL);
}

// Any V, any alignment: one warp per row, two coalesced scalar passes (the second hits L1/L2).
template <typename T>
__global__ void __launch_bounds__(kStreamThreads)
gather_rows_generic_kernel(const T *__restrict__ x, int V, int64_t n_rows, int B, const int32_t *__restrict__ lx,
                           const int32_t *__restrict__ ly, const int32_t *__restrict__ y, int y_stride, int blank,
                           Workspace w)
{
    using E = Elt<T>;
    using A = typename E::acc;
    if (w.status[0] & CWRNNT_ST_FATAL) return;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t(blockIdx.x) * kStreamThreads + threadIdx.x) >> 5;
    const int64_t n_warps = (int64_t(gridDim.x) * kStreamThreads) >> 5;
    int cursor = 0;
    bool any_bad = false;
    for (int64_t r = warp; r < n_rows; r += n_warps) {
        RowInfo ri = locate_row(r, cursor, w.off, B, lx, ly, y, y_stride, V);
        any_bad |= ri.bad_label;
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
            const int64_t at = ri.off + diag_index(ri.t, ri.u, ri.T, ri.U + 1);
            w.lse[r] = lse;
            w.lp_blank[at] = double(E::to_acc(__ldg(row + blank))) - lse;
            if (ri.label >= 0) w.lp_label[at] = double(E::to_acc(__ldg(row + ri.label))) - lse;
        }
    }
    if (any_bad) atomicOr(w.status, CWRNNT_ST_BAD_LABEL);
}

// Log-probability input (the reference contract): no normalisation, two elements per row, one thread per row.
template <typename T>
__global__ void __launch_bounds__(kStreamThreads)
gather_pair_kernel(const T *__restrict__ x, int V, int64_t n_rows, int B, const int32_t *__restrict__ lx,
                   const int32_t *__restrict__ ly, const int32_t *__restrict__ y, int y_stride, int blank,
                   Workspace w)
{
    using E = Elt<T>;
    if (w.status[0] & CWRNNT_ST_FATAL) return;
    int cursor = 0;
    bool any_bad = false;
    const int64_t stride = int64_t(gridDim.x) * kStreamThreads;
    for (int64_t r = int64_t(blockIdx.x) * kStreamThreads + threadIdx.x; r < n_rows; r += stride) {
        RowInfo ri = locate_row(r, cursor, w.off, B, lx, ly, y, y_stride, V);
        any_bad |= ri.bad_label;
        const T *row = x + r * int64_t(V);
        const int64_t at = ri.off + diag_index(ri.t, ri.u, ri.T, ri.U + 1);
        w.lse[r] = 0.0;
        w.lp_blank[at] = double(E::to_acc(__ldg(row + blank)));
        if (ri.label >= 0) w.lp_label[at] = double(E::to_acc(__ldg(row + ri.label)));
    }
    if (any_bad) atomicOr(w.status, CWRNNT_ST_BAD_LABEL);
}

template <typename T>
static cudaError_t launch_gather_t(const cwrnnt_problem &p, const T *x, const int32_t *lx, const int32_t *ly,
                                   const int32_t *y, const Workspace &w, cudaStream_t s)
{
    if (p.n_rows == 0) return cudaSuccess;
    constexpr int VE = Elt<T>::VE;
    const int max_ctas = kNumSMs * 8;
    if (!(p.flags & CWRNNT_FUSED_LOG_SOFTMAX)) {
        int64_t tiles = (p.n_rows + kStreamThreads - 1) / kStreamThreads;
        int grid = int(tiles < max_ctas ? tiles : max_ctas);
        gather_pair_kernel<T><<<grid, kStreamThreads, 0, s>>>(x, p.V, p.n_rows, p.B, lx, ly, y, p.y_stride, p.blank, w);
        return cudaGetLastError();
    }
    RowShape shape{};
    const bool vec_ok = (p.V % VE == 0) && (reinterpret_cast<uintptr_t>(x) % 16 == 0) &&
                        pick_row_shape(p.V / VE, &shape);
    if (vec_ok) {
#define CALL(LPR, NV)                                                                                             \
    {                                                                                                             \
        const int rpc = kStreamThreads / LPR;                                                                     \
        int64_t tiles = (p.n_rows + rpc - 1) / rpc;                                                               \
        int grid = int(tiles < max_ctas ? tiles : max_ctas);                                                      \
        gather_rows_kernel<T, LPR, NV><<<grid, kStreamThreads, 0, s>>>(x, p.V, p.n_rows, p.B, lx, ly, y,          \
                                                                       p.y_stride, p.blank, w);                   \
    }
        CWRNNT_DISPATCH_SHAPE(shape, CALL);
#undef CALL
    } else {
        int64_t tiles = (p.n_rows + 7) / 8;
        int grid = int(tiles < max_ctas ? tiles : max_ctas);
        gather_rows_generic_kernel<T><<<grid, kStreamThreads, 0, s>>>(x, p.V, p.n_rows, p.B, lx, ly, y, p.y_stride,
                                                                      p.blank, w);
    }
    return cudaGetLastError();
}

cudaError_t launch_gather(const cwrnnt_problem &p, const void *x, const int32_t *lx, const int32_t *ly,
                          const int32_t *y, const Workspace &w, cudaStream_t s)
{
    switch (p.dtype) {
    case CWRNNT_F32: return launch_gather_t(p, static_cast<const float *>(x), lx, ly, y, w, s);
    case CWRNNT_F16: return launch_gather_t(p, static_cast<const __half *>(x), lx, ly, y, w, s);
    case CWRNNT_BF16: return launch_gather_t(p, static_cast<const __nv_bfloat16 *>(x), lx, ly, y, w, s);
    case CWRNNT_F64: return launch_gather_t(p, static_cast<const double *>(x), lx, ly, y, w, s);
    }
    return cudaErrorInvalidValue;
}

}  // namespace cwrnnt
