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
#include <cstdio>
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

// log(exp(a) + exp(b)) for the recursion. The float flavour keeps the running value in double and evaluates only the
// bounded correction log1p(exp(-|a-b|)) in float, with the accurate expf/log1pf (about 1 ulp each: measured gradient
// error stays below 1e-6 on lattices of 3000 diagonals, where the MUFU-approximate ex2/lg2 pair drifted past 1e-5);
// the select of the larger operand runs beside it, off the dependent chain. -inf operands (absent move, masked
// vocabulary entry) are handled: |a-b| = inf gives a zero correction, and the NaN of (-inf) - (-inf) is clamped away.
template <bool F64>
__device__ __forceinline__ double lse2(double a, double b)
{
    if (F64) {
        const double hi = fmax(a, b), lo = fmin(a, b);
        if (hi == -INFINITY) return hi;
        return hi + log1p(exp(lo - hi));
    }
    const double diff = a - b;
    const float gap = fminf(fabsf(__double2float_rn(diff)), 3.0e38f);  // fminf drops a NaN operand
    const double hi = diff > 0.0 ? a : b;
    return hi + double(log1pf(expf(-gap)));
}

__device__ __forceinline__ void cp_async8(void *smem_dst, const void *gmem_src)
{
    const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Start of each diagonal in the diagonal-major stream, tracked incrementally in either direction.
// base = (cells on diagonals < e) - lo(e), so that cell (e-u, u) sits at element base + u.
struct DiagCursor {
    int e, base, T, U;
    __device__ __forceinline__ int lo(int d) const { return max(0, d - (T - 1)); }
    __device__ __forceinline__ int len(int d) const { return min(d, U) - lo(d) + 1; }
    __device__ __forceinline__ void up()
    {
        if (e >= 0) base += len(e) - (lo(e + 1) - lo(e));
        ++e;
    }
    __device__ __forceinline__ void down()
    {
        --e;
        if (e >= 0) base -= len(e) - (lo(e + 1) - lo(e));
    }
};

// diagonals staged ahead of the dependent chain (power of two); fewer when a thread owns several columns, so that
// the ring of a 1024-thread CTA stays at 128 KB
template <int C>
struct Ring {
    static constexpr int depth = C == 1 ? 8 : (C == 2 ? 4 : 2);
};

// One direction of one sequence. `stage` is dynamic shared memory: 2 * Ring<C>::depth * C * blockDim.x doubles; each thread
// stages the operands of its own columns with 8-byte cp.async copies (no register scoreboard is held while they are
// in flight, unlike plain loads) and reads them back one step ahead of use.
template <int C, bool F64, bool BETA>
__device__ __forceinline__ void run_direction(int T, int U, const double *__restrict__ lpb,
                                              const double *__restrict__ lpl, double *__restrict__ out,
                                              double *__restrict__ ll_out, int n_active, double (*edge)[32],
                                              double *stage)
{
    constexpr int kRing = Ring<C>::depth;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_warps = n_active >> 5;
    const int m = U + 1;
    const int nd = T + U;  // number of diagonals
    const int u0 = tid * C;
    const int nt = blockDim.x;
    double *st_b = stage + tid;                       // slot k, column j at st_b[(k*C + j) * nt]
    double *st_l = stage + size_t(kRing) * C * nt + tid;

    DiagCursor pf;
    pf.T = T;
    pf.U = U;
    if (!BETA) {
        pf.e = -1;  // step 0 consumes the (empty) data diagonal -1
        pf.base = 0;
    } else {
        pf.e = nd - 1;
        pf.base = T * m - 1 - U;  // the last diagonal holds the single cell (T-1, U)
    }

    // stage the operands of data diagonal pf.e into ring slot k
    auto issue = [&](int k) {
#pragma unroll
        for (int j = 0; j < C; ++j) {
            const int u = u0 + j;
            const int tb = pf.e - u;
            if (!BETA) {
                // step e+1 at column u needs blank(e-u, u) and label(e-u+1, u-1)
                if (u <= U && tb >= 0 && tb <= T - 2) cp_async8(st_b + (k * C + j) * nt, lpb + pf.base + u);
                if (u <= U && u >= 1 && tb >= -1 && tb <= T - 2) cp_async8(st_l + (k * C + j) * nt, lpl + pf.base + u - 1);
            } else {
                // step with d = e at column u needs blank(e-u, u) and label(e-u, u)
                if (u <= U && tb >= 0 && tb <= T - 1) {
                    cp_async8(st_b + (k * C + j) * nt, lpb + pf.base + u);
                    if (u < U) cp_async8(st_l + (k * C + j) * nt, lpl + pf.base + u);
                }
            }
        }
        cp_async_commit();
        if (!BETA) pf.up(); else pf.down();
    };

#pragma unroll
    for (int k = 0; k < kRing; ++k) issue(k);

    double cur_b[C], cur_l[C], nxt_b[C], nxt_l[C], prev[C];
    cp_async_wait<kRing - 1>();
#pragma unroll
    for (int j = 0; j < C; ++j) {
        cur_b[j] = st_b[j * nt];
        cur_l[j] = st_l[j * nt];
        prev[j] = 0.0;
    }

    // row-major cell index (relative to the sequence) of column u0 at the current step; +-m per step
    int64_t cell0 = BETA ? int64_t(nd - 1 - u0) * m + u0 : int64_t(0 - u0) * m + u0;

    for (int s0 = 0; s0 < nd; s0 += kRing) {
#pragma unroll
        for (int k = 0; k < kRing; ++k) {
            const int s = s0 + k;
            if (s >= nd) break;
            const int d = BETA ? nd - 1 - s : s;

            // operands of the next step out of the ring, then refill the slot this step's operands came from
            cp_async_wait<kRing - 2>();
#pragma unroll
            for (int j = 0; j < C; ++j) {
                nxt_b[j] = st_b[(((k + 1) % kRing) * C + j) * nt];
                nxt_l[j] = st_l[(((k + 1) % kRing) * C + j) * nt];
            }
            issue(k);

            // neighbour column's value from the previous step
            double nb = BETA ? __shfl_down_sync(0xffffffffu, prev[0], 1) : __shfl_up_sync(0xffffffffu, prev[C - 1], 1);
            if (n_warps > 1) {
                if (!BETA && lane == 0 && warp > 0) nb = edge[(s + 1) & 1][warp - 1];
                if (BETA && lane == 31 && warp + 1 < n_warps) nb = edge[(s + 1) & 1][warp + 1];
            }

            double nw[C];
#pragma unroll
            for (int j = 0; j < C; ++j) {
                const int u = u0 + j;
                const int t = d - u;
                const bool active = (u <= U) && (t >= 0) && (t <= T - 1);
                const bool has_skip = active && (BETA ? t < T - 1 : t >= 1);
                const bool has_emit = active && (BETA ? u < U : u >= 1);
                double other;  // neighbour column operand
                if (!BETA)
                    other = (j == 0) ? nb : prev[j - 1];
                else
                    other = (j == C - 1) ? nb : prev[j + 1];
                const double skip = has_skip ? prev[j] + cur_b[j] : -INFINITY;
                const double emit = has_emit ? other + cur_l[j] : -INFINITY;
                double v = lse2<F64>(skip, emit);
                if (!has_skip && !has_emit) v = BETA ? cur_b[j] : 0.0;  // beta(T-1,U) = blank(T-1,U); alpha(0,0) = 0
                nw[j] = v;
                if (active) out[cell0 + int64_t(j) * (1 - m)] = v;
            }
#pragma unroll
            for (int j = 0; j < C; ++j) {
                prev[j] = nw[j];
                cur_b[j] = nxt_b[j];
                cur_l[j] = nxt_l[j];
            }
            cell0 += BETA ? -m : m;

            if (n_warps > 1) {
                if (!BETA && lane == 31) edge[s & 1][warp] = prev[C - 1];
                if (BETA && lane == 0) edge[s & 1][warp] = prev[0];
                cta_sync(n_active);
            }
        }
    }
    cp_async_wait<0>();

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
    extern __shared__ double stage[];
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
                                    edge, stage);
    else
        run_direction<C, F64, false>(T, U, w.lp_blank + off, w.lp_label + off, w.alpha + off, w.ll_alpha + n,
                                     n_active, edge, stage);

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
    cudaError_t e = cudaSuccess;
#define CWRNNT_LAUNCH_WAVEFRONT(CC)                                                                               \
    {                                                                                                             \
        const size_t smem = size_t(2) * Ring<CC>::depth * CC * threads * sizeof(double);                          \
        if (smem > 40 * 1024) { /* default cap is 48 KB including the static part: opt in above 40 KB */       \
            e = cudaFuncSetAttribute(wavefront_kernel<CC, F64>, cudaFuncAttributeMaxDynamicSharedMemorySize,      \
                                     int(smem));                                                                  \
            if (e != cudaSuccess) {                                                                               \
                std::fprintf(stderr, "cwrnnt: cannot opt in to %zu bytes of shared memory (%d threads): %s\n",    \
                             smem, threads, cudaGetErrorString(e));                                               \
                return e;                                                                                         \
            }                                                                                                     \
        }                                                                                                         \
        wavefront_kernel<CC, F64><<<grid, threads, smem, s>>>(lx, ly, p.B, p.flags, p.mean_denominator, n_dirs,   \
                                                              w, c, l);                                           \
        e = cudaGetLastError();                                                                                   \
        if (e != cudaSuccess) {                                                                                   \
            cudaFuncAttributes fa{};                                                                              \
            cudaFuncGetAttributes(&fa, wavefront_kernel<CC, F64>);                                                \
            std::fprintf(stderr,                                                                                  \
                         "cwrnnt: wavefront launch failed (%s): grid %d, block %d, dynamic smem %zu; kernel: "     \
                         "%d regs, %zu static smem, max dynamic %d, max threads %d\n",                            \
                         cudaGetErrorString(e), grid, threads, smem, fa.numRegs, fa.sharedSizeBytes,              \
                         fa.maxDynamicSharedSizeBytes, fa.maxThreadsPerBlock);                                    \
            return e;                                                                                             \
        }                                                                                                         \
    }
    if (C == 1) CWRNNT_LAUNCH_WAVEFRONT(1)
    else if (C == 2) CWRNNT_LAUNCH_WAVEFRONT(2)
    else CWRNNT_LAUNCH_WAVEFRONT(4)
#undef CWRNNT_LAUNCH_WAVEFRONT
    return cudaGetLastError();
}

cudaError_t launch_wavefront(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                             void *costs, void *loss, cudaStream_t s)
{
    return p.dtype == CWRNNT_F64 ? launch_wavefront_t<true>(p, lx, ly, w, costs, loss, s)
                                 : launch_wavefront_t<false>(p, lx, ly, w, costs, loss, s);
}

}  // namespace cwrnnt
