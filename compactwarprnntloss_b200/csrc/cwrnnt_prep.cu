// K0 - per-call preparation in one CTA: row offsets (exclusive prefix sum of T_n*(U_n+1), 64-bit), input
// validation into the status words, and the longest-critical-path-first order used by the wavefront kernel.
// Replaces the five ATen launches that build `offset` in the reference (cwarp_cuda.cpp:98-103) and the host-side
// max().item() synchronisations (cwarp_cuda_rnnt_kernel.cu:395-396, cwarp_cuda_gather_kernel.cu:85-86).
#include <climits>

#include "cwrnnt_kernels.h"

namespace cwrnnt {

constexpr int kPrepThreads = 1024;
constexpr int kSortLimit = 4096;  // rank sort is O(B^2 / threads); beyond this the order is the identity

template <typename CostT>
__global__ void __launch_bounds__(kPrepThreads)
prep_kernel(const int32_t *__restrict__ lx, const int32_t *__restrict__ ly, int B, int64_t n_rows, int max_u,
            Workspace w, CostT *__restrict__ costs, CostT *__restrict__ loss, CostT *__restrict__ cost_vec,
            int n_global, int64_t *off_only, GroupPlan plan)
{
    __shared__ int64_t part[kPrepThreads];
    __shared__ int bad_first;
    __shared__ int keys[kSortLimit];
    const int tid = threadIdx.x;
    int64_t *off = off_only ? off_only : w.off;
    if (tid == 0) bad_first = 0x7fffffff;
    __syncthreads();

    // contiguous slice per thread -> local sums -> block scan -> offsets
    const int per = (B + kPrepThreads - 1) / kPrepThreads;
    const int beg = min(tid * per, B), end = min(beg + per, B);
    int64_t local = 0;
    for (int n = beg; n < end; ++n) {
        int T = lx[n], U = ly[n];
        if (T < 1 || U < 0 || U > max_u) {
            atomicMin(&bad_first, n);
            T = T < 1 ? 1 : T;
            U = U < 0 ? 0 : (U > max_u ? max_u : U);
        }
        local += int64_t(T) * (int64_t(U) + 1);
    }
    part[tid] = local;
    __syncthreads();
    for (int step = 1; step < kPrepThreads; step <<= 1) {
        int64_t add = tid >= step ? part[tid - step] : 0;
        __syncthreads();
        part[tid] += add;
        __syncthreads();
    }
    int64_t run = part[tid] - local;  // exclusive prefix of this thread's slice
    for (int n = beg; n < end; ++n) {
        int T = lx[n], U = ly[n];
        T = T < 1 ? 1 : T;
        U = U < 0 ? 0 : (U > max_u ? max_u : U);
        off[n] = run;
        run += int64_t(T) * (int64_t(U) + 1);
    }
    const int64_t total = part[kPrepThreads - 1];
    // offsets alone (the copy kernels around the loss): a clamped length must not pass for a consistent batch, so the
    // total is replaced by -1, which no row count equals, and every consumer of these offsets leaves
    if (tid == 0) off[B] = (off_only && bad_first != 0x7fffffff) ? -1 : total;
    if (off_only) return;

    int st = 0;
    if (bad_first != 0x7fffffff) st |= CWRNNT_ST_BAD_LENGTH;
    if (total != n_rows) st |= CWRNNT_ST_ROW_MISMATCH;
    if (tid == 0) {
        w.status[0] = st;
        w.status[1] = bad_first != 0x7fffffff ? bad_first : -1;
        w.status[2] = int(total & 0x7fffffff);
        w.status[3] = 0;
        *w.ticket = 0u;
    }
    if (st & CWRNNT_ST_FATAL) {
        // nothing downstream runs; make that visible in every result the caller may read without asking for the
        // status: costs, the reduced loss and - for a sharded run - the whole cost vector, so that the all-reduce
        // carries the failure to every rank (the gradient kernels fill their rows with NaN themselves)
        for (int n = tid; n < B; n += kPrepThreads) costs[n] = CostT(NAN);
        if (tid == 0 && loss) *loss = CostT(NAN);
        if (cost_vec)
            for (int i = tid; i <= n_global; i += kPrepThreads) cost_vec[i] = CostT(NAN);
        return;
    }

    // first row of every sequence group (group = nominal row range that holds a sequence's last row; groups are
    // runs of consecutive sequences, possibly empty): bounds[g] = off[first sequence whose group is >= g]
    __syncthreads();  // off[] complete
    for (int n = tid; n < B; n += kPrepThreads) {
        const int g_here = group_of_row(off[n + 1] - 1, plan);
        const int g_prev = n > 0 ? group_of_row(off[n] - 1, plan) : -1;
        for (int g = g_prev + 1; g <= g_here; ++g) w.bounds[g] = off[n];
    }
    if (tid == 0)
        for (int g = (B > 0 ? group_of_row(total - 1, plan) : -1) + 1; g <= kMaxGroups; ++g) w.bounds[g] = total;

    // longest wavefront first: key = T+U, ties by index (stable, deterministic)
    if (B <= kSortLimit) {
        for (int n = tid; n < B; n += kPrepThreads) keys[n] = lx[n] + ly[n];
        __syncthreads();
        for (int n = tid; n < B; n += kPrepThreads) {
            const int k = keys[n];
            int rank = 0;
            for (int j = 0; j < B; ++j) rank += (keys[j] > k) || (keys[j] == k && j < n);
            w.order[rank] = n;
        }
    } else {
        for (int n = tid; n < B; n += kPrepThreads) w.order[n] = n;
    }
}

cudaError_t launch_prep(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                        void *costs, cudaStream_t s, GroupPlan plan, void *loss, void *cost_vector,
                        int n_global)
{
    if (plan.count < 1 || plan.count > kMaxGroups || plan.range_rows < 1) return cudaErrorInvalidValue;
    if (!(p.flags & (CWRNNT_REDUCE_MEAN | CWRNNT_REDUCE_SUM))) loss = nullptr;  // written only under a reduction
    if (p.dtype == CWRNNT_F64)
        prep_kernel<double><<<1, kPrepThreads, 0, s>>>(lx, ly, p.B, p.n_rows, p.max_u, w,
                                                       static_cast<double *>(costs), static_cast<double *>(loss),
                                                       static_cast<double *>(cost_vector), n_global, nullptr, plan);
    else
        prep_kernel<float><<<1, kPrepThreads, 0, s>>>(lx, ly, p.B, p.n_rows, p.max_u, w,
                                                      static_cast<float *>(costs), static_cast<float *>(loss),
                                                      static_cast<float *>(cost_vector), n_global, nullptr, plan);
    return cudaGetLastError();
}

// Validation alone: the checks of K0 plus the label range, and the two maxima the reference asserts on the host.
__global__ void __launch_bounds__(kPrepThreads)
validate_kernel(const int32_t *__restrict__ lx, const int32_t *__restrict__ ly, const int32_t *__restrict__ y,
                int y_stride, int B, int64_t n_rows, int max_u, int V, int32_t *__restrict__ out)
{
    __shared__ unsigned long long total;
    __shared__ int bad_first, max_t, max_l, bad_label;
    const int tid = threadIdx.x;
    if (tid == 0) {
        total = 0ull;
        bad_first = 0x7fffffff;
        max_t = INT_MIN;
        max_l = INT_MIN;
        bad_label = 0;
    }
    __syncthreads();
    unsigned long long local = 0ull;
    int lt = INT_MIN, ll = INT_MIN;
    bool label_out = false;
    for (int n = tid; n < B; n += kPrepThreads) {
        int T = lx[n], U = ly[n];
        lt = max(lt, T);
        ll = max(ll, U);
        if (T < 1 || U < 0 || U > max_u) {
            atomicMin(&bad_first, n);
            T = T < 1 ? 1 : T;
            U = U < 0 ? 0 : (U > max_u ? max_u : U);
        }
        local += (unsigned long long)(T) * (unsigned long long)(U + 1);
        for (int u = 0; u < U; ++u) {
            const int k = y[int64_t(n) * y_stride + u];
            label_out |= (k < 0 || k >= V);
        }
    }
    atomicAdd(&total, local);
    atomicMax(&max_t, lt);
    atomicMax(&max_l, ll);
    if (label_out) bad_label = 1;
    __syncthreads();
    if (tid == 0) {
        int st = 0;
        if (bad_first != 0x7fffffff) st |= CWRNNT_ST_BAD_LENGTH;
        if (int64_t(total) != n_rows) st |= CWRNNT_ST_ROW_MISMATCH;
        if (bad_label) st |= CWRNNT_ST_BAD_LABEL;
        out[0] = st;
        out[1] = bad_first != 0x7fffffff ? bad_first : -1;
        out[2] = max_t;
        out[3] = max_l;
    }
}

cudaError_t launch_validate(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const int32_t *y,
                            int32_t *out_device, cudaStream_t s)
{
    validate_kernel<<<1, kPrepThreads, 0, s>>>(lx, ly, y, p.y_stride, p.B, p.n_rows, p.max_u, p.V, out_device);
    return cudaGetLastError();
}

// Offsets only (reference-shaped scatter backward recomputes them, cwarp_cuda.cpp:124-129).
cudaError_t launch_offsets_only(const int32_t *lx, const int32_t *ly, int B, int max_u, int64_t *off, cudaStream_t s)
{
    Workspace none{};
    prep_kernel<float><<<1, kPrepThreads, 0, s>>>(lx, ly, B, 0, max_u, none, nullptr, nullptr, nullptr, 0, off,
                                                  GroupPlan{1, 1});
    return cudaGetLastError();
}

}  // namespace cwrnnt
