// Analysis exports on the state a forward pass leaves in the workspace: the best (Viterbi) alignment of every
// sequence and the posterior probability of every lattice node.
//
// The reference hands its alpha and beta arrays back to the caller "for analysis"
// (cwarp_cuda_rnnt_kernel.cu:383-384, returned at :496) and stops there; these two kernels are what such an analysis
// computes from them. Neither is on the training path, so they are written for clarity, not for the last microsecond:
// one CTA per sequence walks the anti-diagonals with a block barrier per step (the same schedule as the alpha
// recursion, cwarp_cuda_rnnt_kernel.cu:105-125, with max in place of log-sum-exp), one thread per padded cell
// exponentiates alpha + beta - log P.
#include <map>
#include <mutex>

#include "cwrnnt_kernels.h"

namespace cwrnnt {

constexpr int kAlignThreads = 512;

// v(t,u) = max(v(t-1,u) + blank(t-1,u), v(t,u-1) + label(t,u-1)), v(0,0) = 0; one byte per cell remembers whether the
// label move won (ties go to the blank move). Thread 0 then walks back from (T-1,U). moves[k] = 0: blank move (next
// frame), 1: label move (next label), k < T+U, the last entry being the final blank; -1 beyond.
template <typename CostT>
__global__ void __launch_bounds__(kAlignThreads)
viterbi_kernel(int B, const int32_t *__restrict__ lx, const int32_t *__restrict__ ly, Workspace w,
               unsigned char *__restrict__ back, int stride, int32_t *__restrict__ moves, CostT *__restrict__ scores)
{
    extern __shared__ __align__(16) double vbuf[];  // two rows of m doubles: the previous and the current diagonal
    if (w.status[0] & CWRNNT_ST_FATAL) return;
    const int n = blockIdx.x;
    if (n >= B) return;
    const int T = lx[n], U = ly[n], m = U + 1, nd = T + U;
    const int64_t off = w.off[n];
    const double *__restrict__ lpb = w.lp_blank + off;
    const double *__restrict__ lpl = w.lp_label + off;
    unsigned char *__restrict__ bk = back + off;
    double *prev = vbuf, *cur = vbuf + m;
    int32_t *row = moves + int64_t(n) * stride;
    for (int k = nd + threadIdx.x; k < stride; k += kAlignThreads) row[k] = -1;
    if (threadIdx.x == 0) {
        prev[0] = 0.0;
        bk[0] = 0;
    }
    __syncthreads();
    for (int d = 1; d < nd; ++d) {
        const int lo = max(0, d - (T - 1)), hi = min(d, U);
        const int lo1 = max(0, d - 1 - (T - 1));                  // first column of diagonal d-1
        const int64_t before1 = cells_before(d - 1, T, m);          // start of diagonal d-1 in the diagonal-major arrays
        const int64_t before = before1 + (min(d - 1, U) - lo1 + 1);  // start of diagonal d
        for (int u = lo + threadIdx.x; u <= hi; u += kAlignThreads) {
            const int t = d - u;
            double skip = -INFINITY, emit = -INFINITY;
            if (t > 0) skip = prev[u] + lpb[before1 + (u - lo1)];           // from (t-1,u), on diagonal d-1
            if (u > 0) emit = prev[u - 1] + lpl[before1 + (u - 1 - lo1)];   // from (t,u-1), on diagonal d-1
            const bool label = emit > skip;
            cur[u] = label ? emit : skip;
            bk[before + (u - lo)] = label ? 1 : 0;
        }
        __syncthreads();
        double *tmp = prev;
        prev = cur;
        cur = tmp;
    }
    if (threadIdx.x != 0) return;
    // prev holds the last diagonal: the single cell (T-1,U)
    scores[n] = CostT(prev[U] + lpb[int64_t(T) * m - 1]);
    int t = T - 1, u = U, k = nd - 1;
    if (k < stride) row[k] = 0;
    --k;
    while ((t > 0 || u > 0) && k >= 0) {
        const bool label = bk[diag_index(t, u, T, m)] != 0;
        if (k < stride) row[k] = label ? 1 : 0;
        --k;
        if (label) --u; else --t;
    }
}

// One thread per padded cell [n, t, u]: exp(alpha + beta - log P(y|x)); zero outside the sequence's lattice.
template <typename CostT>
__global__ void __launch_bounds__(256)
posterior_kernel(int B, int t_max, int u_max1, const int32_t *__restrict__ lx, const int32_t *__restrict__ ly,
                 Workspace w, CostT *__restrict__ post)
{
    if (w.status[0] & CWRNNT_ST_FATAL) return;
    const int64_t per = int64_t(t_max) * u_max1, total = per * B;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int n = int(i / per);
        const int64_t rem = i - int64_t(n) * per;
        const int t = int(rem / u_max1), u = int(rem - int64_t(t) * u_max1);
        const int T = lx[n], U = ly[n];
        double v = 0.0;
        if (t < T && u <= U) {
            const int64_t r = w.off[n] + diag_index(t, u, T, U + 1);
            v = exp(w.alpha[r] + w.beta[r] - w.ll_beta[n]);
        }
        post[i] = CostT(v);
    }
}

cudaError_t launch_alignment(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                             unsigned char *back, int32_t stride, int32_t *moves, void *scores, cudaStream_t s)
{
    if (p.B == 0) return cudaSuccess;
    const size_t smem = size_t(2) * (size_t(p.max_u) + 1) * sizeof(double);
    const bool f64 = p.dtype == CWRNNT_F64;
    const void *kernel = f64 ? reinterpret_cast<const void *>(viterbi_kernel<double>)
                             : reinterpret_cast<const void *>(viterbi_kernel<float>);
    if (smem > 48 * 1024) {
        // once per (device, kernel): launches under stream capture after a first plain call make no attribute call
        static std::mutex lock;
        static std::map<std::pair<int, const void *>, size_t> granted;
        int device = 0;
        cudaError_t e = cudaGetDevice(&device);
        if (e != cudaSuccess) return e;
        std::lock_guard<std::mutex> hold(lock);
        size_t &have = granted[std::make_pair(device, kernel)];
        if (have < smem) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
            if (e != cudaSuccess) return e;
            have = smem;
        }
    }
    if (f64)
        viterbi_kernel<double><<<p.B, kAlignThreads, smem, s>>>(p.B, lx, ly, w, back, stride, moves,
                                                                static_cast<double *>(scores));
    else
        viterbi_kernel<float><<<p.B, kAlignThreads, smem, s>>>(p.B, lx, ly, w, back, stride, moves,
                                                               static_cast<float *>(scores));
    return cudaGetLastError();
}

cudaError_t launch_posteriors(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                              int32_t t_max, int32_t u_max1, void *post, cudaStream_t s)
{
    const int64_t total = int64_t(p.B) * t_max * u_max1;
    if (total == 0) return cudaSuccess;
    const int64_t want = (total + 255) / 256;
    const int grid = int(want < kNumSMs * 8 ? want : kNumSMs * 8);
    if (p.dtype == CWRNNT_F64)
        posterior_kernel<double><<<grid, 256, 0, s>>>(p.B, t_max, u_max1, lx, ly, w, static_cast<double *>(post));
    else
        posterior_kernel<float><<<grid, 256, 0, s>>>(p.B, t_max, u_max1, lx, ly, w, static_cast<float *>(post));
    return cudaGetLastError();
}

}  // namespace cwrnnt
