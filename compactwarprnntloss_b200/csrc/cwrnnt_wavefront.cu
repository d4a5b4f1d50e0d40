// K2 - alpha/beta lattice recursion as an anti-diagonal wavefront, one CTA per (sequence, direction).
//
// Replaces cal_alpha_beta_kernel / cal_beta_ / fill_cost_kernel of the reference
// (cwarp_cuda_rnnt_kernel.cu:31-273, :334-367). The reference tiles the lattice into 32-frame warps that hand over
// through global-memory spin locks; here one CTA owns a whole sequence-direction, thread u owns column u and walks
// cell (d-u, u) at step d, so no CTA ever waits on another:
//   alpha(t,u) = LSE(alpha(t-1,u) + blank(t-1,u), alpha(t,u-1) + label(t,u-1)),  alpha(0,0) = 0     (:59-125)
//   beta(t,u)  = LSE(beta(t+1,u) + blank(t,u),    beta(t,u+1) + label(t,u)),     beta(T-1,U) = blank(T-1,U)  (:165-231)
// The own-column operand stays in a register, the neighbour column arrives by warp shuffle (shared memory only at warp
// seams, one named barrier per diagonal), and the log-probs stream in from the diagonal-major arrays K1 wrote, fully
// coalesced and prefetched a few diagonals ahead of the dependent chain. alpha and beta CTAs of all sequences run
// concurrently in one launch, longest critical path first.
//
// Arithmetic: the running sums are kept in double (|alpha| reaches 10^3..10^4, where a float ulp is ~1e-4 and would
// show up directly in exp(alpha+beta-ll)); the bounded correction log1p(exp(-|a-b|)) is evaluated in float as in the
// reference (:10,:22-29), or in double for double input.
//
// Bound: latency of the dependent chain, T+U steps per sequence; reported as microseconds per diagonal.
// The last CTA to finish turns the per-sequence log-likelihoods into costs, the status bits and the reduced loss.
#include <type_traits>

#include "cwrnnt_kernels.h"

namespace cwrnnt {

__device__ __forceinline__ void cta_sync(int n_active)
{
    if (n_active > 32)
        asm volatile("bar.sync 1, %0;" ::"r"(n_active) : "memory");
    else
        __syncwarp();
}

template <bool F64>
__device__ __forceinline__ double lse2(double a, double b)
{
    const double hi = fmax(a, b), lo = fmin(a, b);
    if (hi == -INFINITY) return hi;
    if (F64) return hi + log1p(exp(lo - hi));
    return hi + double(log1pf(expf(float(lo - hi))));
}

// Walks the diagonals of a T x (U+1) lattice in either direction, tracking where each starts in diagonal-major order.
struct DiagCursor {
    int e;        // diagonal index t+u
    int64_t cum;  // cells on diagonals < e
    int T, U;
    __device__ __forceinline__ int lo() const { return max(0, e - (T - 1)); }
    __device__ __forceinline__ int hi() const { return min(e, U); }
    __device__ __forceinline__ int len() const { return hi() - lo() + 1; }
    __device__ __forceinline__ void step_up()
    {
        cum += len();
        ++e;
    }
    __device__ __forceinline__ void step_down()
    {
        --e;
        cum -= len();
    }
};

template <int C, bool F64, bool BETA>
__device__ __forceinline__ void run_direction(int T, int U, const double *__restrict__ lpb,
                                              const double *__restrict__ lpl, double *__restrict__ out,
                                              double *__restrict__ ll_out, int n_active, double (*edge)[32])
{
    constexpr int PD = (8 / C) > 2 ? (8 / C) : 2;  // diagonals prefetched ahead
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_warps = n_active >> 5;
    const int m = U + 1;
    const int nd = T + U;  // number of diagonals
    const int u0 = tid * C;

    // fetch the operands of data diagonal cur.e for this thread's columns
    auto fetch = [&](const DiagCursor &cur, double (&fb)[C], double (&fl)[C]) {
#pragma unroll
        for (int j = 0; j < C; ++j) {
            const int u = u0 + j;
            fb[j] = 0.0;
            fl[j] = 0.0;
            if (cur.e < 0 || cur.e > nd - 1 || u > U) continue;
            if (!BETA) {
                // step d = e+1 at column u: blank(t-1,u) with t-1 = e-u, label(t,u-1) with t = e-u+1
                const int tb = cur.e - u;
                if (tb >= 0 && tb <= T - 2) fb[j] = __ldg(lpb + cur.cum + (u - cur.lo()));
                if (u >= 1 && tb + 1 >= 0 && tb + 1 <= T - 1) fl[j] = __ldg(lpl + cur.cum + (u - 1 - cur.lo()));
            } else {
                // step d = e at column u: blank(t,u), label(t,u) with t = e-u
                const int t = cur.e - u;
                if (t >= 0 && t <= T - 1) {
                    fb[j] = __ldg(lpb + cur.cum + (u - cur.lo()));
                    if (u < U) fl[j] = __ldg(lpl + cur.cum + (u - cur.lo()));
                }
            }
        }
    };

    DiagCursor pf;
    pf.T = T;
    pf.U = U;
    if (!BETA) {
        pf.e = -1;  // step 0 consumes the (empty) data diagonal -1
        pf.cum = 0;
    } else {
        pf.e = nd - 1;
        pf.cum = int64_t(T) * m - 1;
    }
    auto advance = [&]() {
        if (!BETA) {
            if (pf.e >= 0) pf.step_up(); else pf.e = 0;
        } else {
            if (pf.e > 0) pf.step_down(); else pf.e = -1;
        }
    };

    double qb[PD][C], ql[PD][C];
#pragma unroll
    for (int k = 0; k < PD; ++k) {
        fetch(pf, qb[k], ql[k]);
        advance();
    }

    double prev[C];
#pragma unroll
    for (int j = 0; j < C; ++j) prev[j] = 0.0;

    // cell index (row-major, relative to the sequence) of column u0 at the current step; +-m per step
    int64_t cell0 = BETA ? int64_t(nd - 1 - u0) * m + u0 : int64_t(0 - u0) * m + u0;

    for (int s0 = 0; s0 < nd; s0 += PD) {
#pragma unroll
        for (int k = 0; k < PD; ++k) {
            const int s = s0 + k;
            if (s >= nd) break;
            const int d = BETA ? nd - 1 - s : s;

            // neighbour column's value from the previous step
            double nb = BETA ? __shfl_down_sync(0xffffffffu, prev[0], 1) : __shfl_up_sync(0xffffffffu, prev[C - 1], 1);
            if (!BETA && lane == 0 && warp > 0) nb = edge[(s + 1) & 1][warp - 1];
            if (BETA && lane == 31 && warp + 1 < n_warps) nb = edge[(s + 1) & 1][warp + 1];

            double nw[C];
#pragma unroll
            for (int j = 0; j < C; ++j) {
                const int u = u0 + j;
                const int t = d - u;
                const bool active = (u <= U) && (t >= 0) && (t <= T - 1);
                double other;  // neighbour column operand
                if (!BETA)
                    other = (j == 0) ? nb : prev[j - 1];
                else
                    other = (j == C - 1) ? nb : prev[j + 1];
                const bool has_skip = active && (BETA ? t < T - 1 : t >= 1);
                const bool has_emit = active && (BETA ? u < U : u >= 1);
                const double skip = prev[j] + qb[k][j];
                const double emit = other + ql[k][j];
                double v;
                if (has_skip && has_emit)
                    v = lse2<F64>(skip, emit);
                else if (has_skip)
                    v = skip;
                else if (has_emit)
                    v = emit;
                else
                    v = BETA ? qb[k][j] : 0.0;  // beta(T-1,U) = blank(T-1,U); alpha(0,0) = 0
                nw[j] = v;
                if (active) out[cell0 + int64_t(j) * (1 - m)] = v;
            }
#pragma unroll
            for (int j = 0; j < C; ++j) prev[j] = nw[j];
            cell0 += BETA ? -m : m;

            // refill this ring slot with the data diagonal PD steps ahead
            fetch(pf, qb[k], ql[k]);
            advance();

            if (n_warps > 1) {
                if (!BETA && lane == 31) edge[s & 1][warp] = prev[C - 1];
                if (BETA && lane == 0) edge[s & 1][warp] = prev[0];
                cta_sync(n_active);
            }
        }
    }

    // prev now holds the last diagonal: alpha(T-1,U) at column U, or beta(0,0) at column 0
    if (!BETA) {
        if (U >= u0 && U < u0 + C) {
            double last = 0.0;
#pragma unroll
            for (int j = 0; j < C; ++j)
                if (u0 + j == U) last = prev[j];
            *ll_out = last + __ldg(lpb + int64_t(T) * m - 1);
        }
    } else {
        if (tid == 0) *ll_out = prev[0];
    }
}

template <int C, bool F64>
__global__ void __launch_bounds__(1024)
wavefront_kernel(const int32_t *__restrict__ lx, const int32_t *__restrict__ ly, int B, int flags, int mean_den,
                 int n_dirs, Workspace w, typename std::conditional<F64, double, float>::type *__restrict__ costs,
                 typename std::conditional<F64, double, float>::type *__restrict__ loss)
{
    using CostT = typename std::conditional<F64, double, float>::type;
    __shared__ double edge[2][32];
    __shared__ int last_flag;
    if (w.status[0] & CWRNNT_ST_FATAL) return;

    const int n = w.order[blockIdx.x / n_dirs];
    const bool beta_dir = (n_dirs == 1) || (blockIdx.x & 1);
    const int T = lx[n], U = ly[n];
    const int64_t off = w.off[n];
    const int cols = (U + 1 + C - 1) / C;
    const int n_active = min(int(blockDim.x), (cols + 31) & ~31);
    if (int(threadIdx.x) >= n_active) return;  // whole warps leave; the rest synchronise on a named barrier

    if (beta_dir)
        run_direction<C, F64, true>(T, U, w.lp_blank + off, w.lp_label + off, w.beta + off, w.ll_beta + n, n_active,
                                    edge);
    else
        run_direction<C, F64, false>(T, U, w.lp_blank + off, w.lp_label + off, w.alpha + off, w.ll_alpha + n,
                                     n_active, edge);

    // ---- completion ticket: the last CTA of the grid finalises costs, status and loss
    __threadfence();
    cta_sync(n_active);
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(w.ticket, 1u);
        last_flag = (t == gridDim.x - 1);
    }
    cta_sync(n_active);
    if (!last_flag) return;
    __threadfence();

    double partial = 0.0;
    for (int i = threadIdx.x; i < B; i += n_active) {
        double b = __ldcg(w.ll_beta + i);
        if (n_dirs == 2) {
            // forward/backward consistency guard of the reference (cwarp_cuda_rnnt_kernel.cu:350-366)
            const double a = __ldcg(w.ll_alpha + i);
            const double big = fmax(a, b);
            if (fabs(a - b) / fabs(big) > 1e-3) {
                b = 0.5 * (a + b);
                atomicOr(w.status, CWRNNT_ST_FWD_BWD_GAP);
            }
        }
        const double c = -b * sequence_scale(flags, lx[i]);
        costs[i] = CostT(c);
        partial += c;
    }
    if (flags & (CWRNNT_REDUCE_MEAN | CWRNNT_REDUCE_SUM)) {
        // fixed-order block sum: lanes, then warps
#pragma unroll
        for (int sft = 16; sft > 0; sft >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, sft);
        cta_sync(n_active);
        if ((threadIdx.x & 31) == 0) edge[0][threadIdx.x >> 5] = partial;
        cta_sync(n_active);
        if (threadIdx.x == 0) {
            double tot = 0.0;
            for (int k = 0; k < (n_active >> 5); ++k) tot += edge[0][k];
            if (flags & CWRNNT_REDUCE_MEAN) tot /= double(mean_den > 0 ? mean_den : B);
            if (loss) *loss = CostT(tot);
        }
    }
    if (threadIdx.x == 0) *w.ticket = 0u;
}

template <bool F64>
static cudaError_t launch_wavefront_t(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                                      void *costs, void *loss, cudaStream_t s)
{
    using CostT = typename std::conditional<F64, double, float>::type;
    if (p.B == 0) return cudaSuccess;
    const int n_dirs = (p.flags & CWRNNT_COSTS_ONLY) ? 1 : 2;
    const int cols = p.max_u + 1;
    const int C = cols <= 1024 ? 1 : (cols <= 2048 ? 2 : 4);
    const int per_thread_cols = (cols + C - 1) / C;
    const int threads = (per_thread_cols + 31) & ~31;
    const int grid = p.B * n_dirs;
    CostT *c = static_cast<CostT *>(costs);
    CostT *l = static_cast<CostT *>(loss);
    if (C == 1)
        wavefront_kernel<1, F64><<<grid, threads, 0, s>>>(lx, ly, p.B, p.flags, p.mean_denominator, n_dirs, w, c, l);
    else if (C == 2)
        wavefront_kernel<2, F64><<<grid, threads, 0, s>>>(lx, ly, p.B, p.flags, p.mean_denominator, n_dirs, w, c, l);
    else
        wavefront_kernel<4, F64><<<grid, threads, 0, s>>>(lx, ly, p.B, p.flags, p.mean_denominator, n_dirs, w, c, l);
    return cudaGetLastError();
}

cudaError_t launch_wavefront(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                             void *costs, void *loss, cudaStream_t s)
{
    return p.dtype == CWRNNT_F64 ? launch_wavefront_t<true>(p, lx, ly, w, costs, loss, s)
                                 : launch_wavefront_t<false>(p, lx, ly, w, costs, loss, s);
}

}  // namespace cwrnnt
