// K2 - alpha/beta lattice recursion as an anti-diagonal wavefront, one CTA per (sequence, direction).
//
// Replaces cal_alpha_beta_kernel / cal_beta_ / fill_cost_kernel of the reference
// (cwarp_cuda_rnnt_kernel.cu:31-273, :334-367). The reference tiles the lattice into 32-frame warps that hand over
// through global-memory spin locks; here one CTA owns a whole sequence-direction, thread u owns column u and walks
// cell (d-u, u) at step d, so no CTA ever waits on another:
//   alpha(t,u) = LSE(alpha(t-1,u) + blank(t-1,u), alpha(t,u-1) + label(t,u-1)),  alpha(0,0) = 0     (:59-125)
//   beta(t,u)  = LSE(beta(t+1,u) + blank(t,u),    beta(t,u+1) + label(t,u)),     beta(T-1,U) = blank(T-1,U)  (:165-231)
// Two kernels share the recursion. Lattices of up to 512 columns take the split-role kernel (further down): a compute
// warp and a helper warp per 32 columns, meeting on one barrier per diagonal or, for wide float lattices, once per
// round of four diagonals. Wider ones take the single-role kernel: the own-column operand stays in a
// register, the neighbour column arrives by warp shuffle (shared memory only at warp seams), one named barrier per
// diagonal, 1, 4 or 8 columns per thread. In both, the log-probs K1 wrote diagonal-major form one contiguous stream
// per (sequence, direction); each thread stages its own operands, several diagonals ahead of the dependent chain,
// with 8-byte cp.async copies into a shared-memory ring (fully coalesced across the warp, and no register scoreboard
// is held while they fly). alpha and beta are written diagonal-major too, so a warp's store is one contiguous
// 256-byte segment. alpha and beta CTAs of all sequences run concurrently in one launch, longest critical path first.
// (A producer/consumer variant - one elected thread feeding the ring with cp.async.bulk + mbarrier - was built and
// measured: 125 us against 79 us on the 81-column workload, because its per-step chunk bookkeeping costs more
// instructions on the dependent chain than the per-thread copies it replaces; it was dropped.)
//
// Arithmetic: the running sums are kept in double (|alpha| reaches 10^3..10^4, where a float ulp is ~1e-4 and would
// show up directly in exp(alpha+beta-ll)); the bounded correction log1p(exp(-|a-b|)) is evaluated in float (the
// reference evaluates its whole log-sum-exp in float, :10,:22-29), or in double for double input.
//
// Bound: latency of the dependent chain, T+U steps per sequence; reported as microseconds per diagonal.
// The last CTA to finish turns the per-sequence log-likelihoods into costs, the status bits and the reduced loss.
#include <climits>
#include <cstdio>
#include <map>
#include <mutex>
#include <type_traits>
#include <utility>

#include "cwrnnt_kernels.h"

namespace cwrnnt {

__device__ __forceinline__ void cta_sync(int n_active)
{
    if (n_active > 32)
        asm volatile("bar.sync 1, %0;" ::"r"(n_active) : "memory");
    else
        __syncwarp();
}

// log(exp(a) + exp(b)) for the recursion: the larger operand plus the bounded correction
//     f(g) = log1p(exp(-g)),  g = |a - b| >= 0,  f in (0, ln 2].
// The running values stay in double. For float-type inputs f is read from a per-CTA shared-memory table instead of
// calling expf/log1pf: nodes every 1/16 up to g = 32, four Taylor coefficients per node (f and its first three
// derivatives over 1, 1, 2, 6, computed in double when the CTA starts), evaluated by a 3-FMA Horner step on
// |h| <= 1/32. Truncation error is below 5e-9, total error below 6e-8 absolute with no measurable bias (the libm pair
// log1pf(expf()) is at 1.1e-7), and it costs 10 instructions on the dependent chain instead of about 40 - the chain's
// length is what bounds this kernel. -inf operands (absent move, masked vocabulary entry) need no branch: g clamps to
// 32 (f = 1.3e-14), the NaN of (-inf) - (-inf) is dropped by fminf, and -inf plus a finite correction stays -inf.
constexpr int kLseNodes = 513;            // g = 0, 1/16, ..., 32
constexpr float kLseMagic = 12582912.0f;  // 1.5 * 2^23: adding it rounds to the nearest integer in the low mantissa bits

__device__ __forceinline__ void build_lse_table(float4 *tab, int tid, int n_threads)
{
    for (int i = tid; i < kLseNodes; i += n_threads) {
        const double g = double(i) * 0.0625;
        const double s = 1.0 / (1.0 + exp(g));  // minus the first derivative
        tab[i] = make_float4(float(log1p(exp(-g))), float(-s), float(0.5 * s * (1.0 - s)),
                             float(-s * (1.0 - s) * (1.0 - 2.0 * s) / 6.0));
    }
}

// The step of the split-role kernels: a = own column's term (known early), nb = the neighbour's value (arrives last),
// l = the label operand. a - (nb + l) is taken as (a - l) - nb, so that only ONE double addition stands between the
// arrival of nb and the float correction; nb + l is needed for the result only and runs beside it.
template <bool F64>
__device__ __forceinline__ double lse2_late(double a, double l, double nb, const float4 *__restrict__ tab)
{
    const double b = nb + l;
    if (F64) {
        const double hi = fmax(a, b), lo = fmin(a, b);
        if (hi == -INFINITY) return hi;
        return hi + log1p(exp(lo - hi));
    }
    const double diff = (a - l) - nb;
    const float g = fminf(fabsf(__double2float_rn(diff)), 32.0f);  // fminf drops a NaN operand
    const float q = fmaf(g, 16.0f, kLseMagic);
    const float4 t = tab[__float_as_int(q) & 0x3ff];
    const float h = fmaf(q - kLseMagic, -0.0625f, g);
    const float c = fmaf(fmaf(fmaf(t.w, h, t.z), h, t.y), h, t.x);
    const double hi = diff > 0.0 ? a : b;
    return hi + double(c);
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

// R = diagonals staged ahead of the dependent chain (power of two: 8, 4 or 2, the deepest whose ring fits in shared
// memory for the CTA's thread count). C = columns per thread: 1 up to 1024 columns, 4 up to 2048, 8 up to 4096.
// One column per thread is the fast shape: a warp issues roughly one instruction every four cycles on this chain, so
// the time of a step follows the instruction count of one warp, and spreading columns over more warps (which run on
// the SM's four schedulers side by side) beats giving a thread several columns (measured: 3 columns per thread in a
// single warp took 148 us where 3 warps take 80 us on the same 81-column lattices).

// One direction of one sequence. `stage` is dynamic shared memory: 2 * R * C * blockDim.x doubles; each thread
// stages the operands of its own columns with 8-byte cp.async copies (no register scoreboard is held while they are
// in flight, unlike plain loads) and reads them back one step ahead of use.
template <int C, int R, bool F64, bool BETA>
__device__ __forceinline__ void run_direction(int T, int U, const double *__restrict__ lpb,
                                              const double *__restrict__ lpl, double *__restrict__ out,
                                              double *__restrict__ ll_out, int n_active, double (*edge)[32],
                                              double *stage, const float4 *__restrict__ lse_tab)
{
    constexpr int kRing = R;
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

    // Stage the operands of data diagonal pf.e into ring slot k. An operand that does not exist (cell outside the
    // lattice, no label move out of the last column, ...) is staged as 0.0: the recursion below is branch-free and
    // relies on absent moves meeting a -inf running value, so their operand only has to be finite.
    // sbase[k] = base of the data diagonal staged in slot k. The results go out diagonal-major as well, and the
    // diagonal a step writes is one whose base is already here: beta writes the diagonal it reads (slot k), alpha
    // writes the diagonal the next step reads (slot k+1).
    int sbase[kRing];
    auto issue = [&](int k) {
        sbase[k] = pf.base;
#pragma unroll
        for (int j = 0; j < C; ++j) {
            const int u = u0 + j;
            const int tb = pf.e - u;
            double *sb = st_b + (k * C + j) * nt, *sl = st_l + (k * C + j) * nt;
            if (!BETA) {
                // step e+1 at column u needs blank(e-u, u) and label(e-u+1, u-1)
                if (u <= U && tb >= 0 && tb <= T - 2) cp_async8(sb, lpb + pf.base + u); else *sb = 0.0;
                if (u <= U && u >= 1 && tb >= -1 && tb <= T - 2) cp_async8(sl, lpl + pf.base + u - 1); else *sl = 0.0;
            } else {
                // step with d = e at column u needs blank(e-u, u) and label(e-u, u)
                const bool cell = u <= U && tb >= 0 && tb <= T - 1;
                if (cell) cp_async8(sb, lpb + pf.base + u); else *sb = 0.0;
                if (cell && u < U) cp_async8(sl, lpl + pf.base + u); else *sl = 0.0;
            }
        }
        cp_async_commit();
        if (!BETA) pf.up(); else pf.down();
    };

#pragma unroll
    for (int k = 0; k < kRing; ++k) issue(k);

    // Running values. Cells outside the lattice count as -inf, which makes every boundary case fall out of the one
    // interior formula v = LSE(own + blank, neighbour + label):
    //   alpha: column u starts at -inf (virtual row t = -1), column 0 starts at 0 with a zero operand so that
    //          alpha(0,0) = LSE(0 + 0, -inf) = 0; the left neighbour of column 0 is -inf.
    //   beta : column u starts at -inf (virtual row t = T), column U starts at 0 so that
    //          beta(T-1,U) = LSE(0 + blank(T-1,U), -inf); columns beyond U stay -inf for ever.
    double cur_b[C], cur_l[C], nxt_b[C], nxt_l[C], prev[C];
    int tcur[C];  // frame index of column j at the current step; parked far outside [0,T) for columns beyond U
    cp_async_wait<kRing - 1>();
#pragma unroll
    for (int j = 0; j < C; ++j) {
        const int u = u0 + j;
        cur_b[j] = st_b[j * nt];
        cur_l[j] = st_l[j * nt];
        prev[j] = (u == (BETA ? U : 0)) ? 0.0 : -INFINITY;
        tcur[j] = u <= U ? (BETA ? nd - 1 - u : -u) : INT_MIN / 2;
    }
    const bool no_neighbour = BETA ? (u0 + C - 1 >= U) : (tid == 0);


    for (int s0 = 0; s0 < nd; s0 += kRing) {
#pragma unroll
        for (int k = 0; k < kRing; ++k) {
            const int s = s0 + k;
            if (s >= nd) break;

            const int out_base = sbase[BETA ? k : (k + 1) % kRing];  // before issue(k) recycles the slot

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
            if (no_neighbour) nb = -INFINITY;
            // step 0 starts from the virtual row: its 0 at the start column must not reach the neighbouring column
            const bool first = (k == 0) && (s0 == 0);

            double nw[C];
#pragma unroll
            for (int j = 0; j < C; ++j) {
                double other;  // neighbour column operand
                if (!BETA)
                    other = (j == 0) ? nb : prev[j - 1];
                else
                    other = (j == C - 1) ? nb : prev[j + 1];
                if (first) other = -INFINITY;
                const double v = lse2_late<F64>(prev[j] + cur_b[j], cur_l[j], other, lse_tab);
                nw[j] = v;
                if (unsigned(tcur[j]) < unsigned(T)) out[out_base + u0 + j] = v;
            }
#pragma unroll
            for (int j = 0; j < C; ++j) {
                prev[j] = nw[j];
                cur_b[j] = nxt_b[j];
                cur_l[j] = nxt_l[j];
                tcur[j] += BETA ? -1 : 1;
            }

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

// Thread budget per CTA: one column per thread up to 1024 columns; C = 4 and 8 cover up to 2048 and 4096 columns with
// at most 512 threads, which leaves 128 registers per thread for the C recursions of a thread.
template <int C>
struct MaxThreads {
    static constexpr int value = C == 1 ? 1024 : 512;
};

// Everything a wavefront CTA needs besides its shared memory.
template <typename CostT>
struct WaveArgs {
    const int32_t *lx, *ly;
    int B, flags, mean_den, n_dirs;
    Workspace w;
    CostT *costs, *loss;
    // sharded runs: costs are also written into their global slots of a [n_global + 1] vector (the partial loss goes
    // into the last slot, every other slot is zeroed), ready for one all-reduce(sum) across ranks
    const int32_t *global_ids;
    int n_global;
    CostT *cost_vec;
    // pipelined step: this launch runs the sequences of one group only; one completion ticket per sequence-direction
    // over all launches of the step
    GroupPlan plan;
    int group;
    unsigned int ticket_total;
};

// True when sequence n is left to another launch of a pipelined step.
template <typename CostT>
__device__ __forceinline__ bool other_group(const WaveArgs<CostT> &g, int n)
{
    return g.plan.count > 1 && group_of_row(g.w.off[n + 1] - 1, g.plan) != g.group;
}

// Completion ticket: the last CTA of the grid turns the per-sequence log-likelihoods into costs, status and loss.
template <typename CostT>
__device__ __forceinline__ void finalize_if_last(const WaveArgs<CostT> &g, int n_active, double (*edge)[32],
                                                 int *last_flag)
{
    const Workspace &w = g.w;
    __threadfence();
    cta_sync(n_active);
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(w.ticket, 1u);
        *last_flag = (t == g.ticket_total - 1);
    }
    cta_sync(n_active);
    if (!*last_flag) return;
    __threadfence();

    if (g.cost_vec)
        for (int i = threadIdx.x; i <= g.n_global; i += n_active) g.cost_vec[i] = CostT(0);
    cta_sync(n_active);

    double partial = 0.0;
    for (int i = threadIdx.x; i < g.B; i += n_active) {
        double b = __ldcg(w.ll_beta + i);
        if (g.n_dirs == 2) {
            bool gap = false;
            b = guarded_loglik(__ldcg(w.ll_alpha + i), b, gap);
            if (gap) atomicOr(w.status, CWRNNT_ST_FWD_BWD_GAP);
        }
        const double c = -b * sequence_scale(g.flags, g.lx[i]);
        g.costs[i] = CostT(c);
        if (g.cost_vec) g.cost_vec[g.global_ids ? g.global_ids[i] : i] = CostT(c);
        partial += c;
    }
    if ((g.flags & (CWRNNT_REDUCE_MEAN | CWRNNT_REDUCE_SUM)) || g.cost_vec) {
        // fixed-order block sum: lanes, then warps
#pragma unroll
        for (int sft = 16; sft > 0; sft >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, sft);
        cta_sync(n_active);
        if ((threadIdx.x & 31) == 0) edge[0][threadIdx.x >> 5] = partial;
        cta_sync(n_active);
        if (threadIdx.x == 0) {
            double tot = 0.0;
            for (int k = 0; k < (n_active >> 5); ++k) tot += edge[0][k];
            if (g.flags & CWRNNT_REDUCE_MEAN) tot /= double(g.mean_den > 0 ? g.mean_den : g.B);
            if (g.loss) *g.loss = CostT(tot);
            if (g.cost_vec) g.cost_vec[g.n_global] = CostT(tot);
        }
    }
    if (threadIdx.x == 0) *w.ticket = 0u;
}

// Generic path: C columns per thread, per-thread cp.async ring of depth R.
template <int C, int R, bool F64>
__global__ void __launch_bounds__(MaxThreads<C>::value)
wavefront_kernel(WaveArgs<typename std::conditional<F64, double, float>::type> g)
{
    extern __shared__ __align__(16) double stage[];
    __shared__ double edge[2][32];
    __shared__ float4 lse_tab[F64 ? 1 : kLseNodes];
    __shared__ int last_flag;
    const Workspace &w = g.w;
    if (w.status[0] & CWRNNT_ST_FATAL) return;

    const int n = w.order[blockIdx.x / g.n_dirs];
    // Another launch's sequence: leave at once. Only CTAs that run a sequence-direction take a completion ticket (each
    // sequence-direction runs in exactly one launch of the step), so leaving costs no atomic and no fence.
    if (other_group(g, n)) return;
    const bool beta_dir = (g.n_dirs == 1) || (blockIdx.x & 1);
    const int T = g.lx[n], U = g.ly[n];
    const int64_t off = w.off[n];
    const int cols = (U + 1 + C - 1) / C;
    const int n_active = min(int(blockDim.x), (cols + 31) & ~31);
    if (int(threadIdx.x) >= n_active) return;  // whole warps leave; the rest synchronise on a named barrier
    if (!F64) {
        build_lse_table(lse_tab, threadIdx.x, n_active);
        cta_sync(n_active);
    }
    if (beta_dir)
        run_direction<C, R, F64, true>(T, U, w.lp_blank + off, w.lp_label + off, w.beta + off, w.ll_beta + n, n_active,
                                       edge, stage, lse_tab);
    else
        run_direction<C, R, F64, false>(T, U, w.lp_blank + off, w.lp_label + off, w.alpha + off, w.ll_alpha + n,
                                        n_active, edge, stage, lse_tab);
    finalize_if_last(g, n_active, edge, &last_flag);
}

// ------------------------------------------------------------------------------------------------ split-role path
// Up to 512 columns. The time of a step follows the number of instructions one warp has to issue on it (a warp on this
// chain issues about one instruction every four to five cycles and no other warp of the sequence can take its place),
// so the work of a 32-column group is split over two warps that run side by side on the SM's schedulers:
//   compute warp: operands out of the shared-memory ring, neighbour value, the log-sum-exp, result into shared memory
//                 and, one step later, to global memory;
//   helper warp : stages the operands `R` steps ahead (8-byte cp.async, all the index arithmetic and predicates) and
//                 publishes, per ring slot, the stream offset of the diagonal it holds (`diag_base`).
// Results pass through a double-buffered row `vbuf[2][columns]` for the neighbour exchange (no shuffles, no warp-seam
// special case). One named barrier per step joins all warps of the CTA. The global store of a result is issued at
// the START of the following step: the barrier waits for the warp's outstanding stores, so a store issued right
// before it costs its whole round trip on every step (0.163 us per diagonal at 32 columns), one issued a step's
// length ahead costs nothing (0.127-0.130; with the helper loading and storing the results instead, 0.134 - there
// the helper's own instruction stream, about 200 cycles a step, was what the compute warp waited for). Timing-only
// builds give the parts of a step at 32 columns: skeleton 0.016 us, log-sum-exp chain 0.065 us, barrier 0.013 us.
// Hand-over of ring slot x % R (operands of step x): the helper's copy group for step s+2 is complete before the
// barrier that ends step s; the compute warp reads the operands of step s+1 during step s (one step ahead, into
// registers); the helper refills slot s % R during step s, after its last read during step s-1. Step 0's operands
// are read before the loop, between two start barriers, so that the refill of slot 0 during step 0 cannot overtake
// that read.
constexpr int kRoundsMinCols = 160;  // padded column count above which a launch uses rounds
constexpr int kRoundsRing = 16;      // operand slots of the rounds variant
constexpr int kRoundsRows = 8;       // result rows of the rounds variant

template <int R, bool F64, bool BETA>
__device__ __forceinline__ void run_direction_split(int T, int U, const double *__restrict__ lpb,
                                                    const double *__restrict__ lpl, double *__restrict__ out,
                                                    double *__restrict__ ll_out, int n_cols, int n_sync,
                                                    double *stage, double *vbuf, int *diag_base,
                                                    const float4 *__restrict__ lse_tab, bool helper, int u)
{
    const int m = U + 1;
    const int nd = T + U;
    double *st_b = stage + u;                    // slot k at st_b[k * n_cols]
    double *st_l = stage + R * n_cols + u;
    // results of even / odd steps; element n_cols of each row is a permanent -inf (the neighbour of an edge column)
    double *v0 = vbuf, *v1 = vbuf + n_cols + 1;

    if (helper) {
        // Diagonal e starts at stream element base(e) + lo(e) and column u sits at base(e) + u; moving to the next
        // diagonal adds step(e) = min(e+1, c2, U+T-1-e), c2 = (U <= T-1) ? U+1 : T-1 (growing, plateau, shrinking
        // part of the lattice). e = diagonal whose operands are staged next, tb = e - u.
        const int c2 = (U <= T - 1) ? U + 1 : T - 1;
        int e = BETA ? nd - 1 : -1;
        int base = BETA ? T * m - 1 - U : 0;
        int tb = u <= U ? e - u : INT_MIN / 2;  // parked far outside every range for columns beyond U
        auto issue = [&](int k) {
            if (u == 0) diag_base[k] = base;
            double *sb = st_b + k * n_cols, *sl = st_l + k * n_cols;
            if (!BETA) {
                // step e+1 at column u needs blank(e-u, u) and label(e-u+1, u-1)
                if (unsigned(tb) < unsigned(T - 1)) cp_async8(sb, lpb + base + u); else *sb = 0.0;
                if (u >= 1 && unsigned(tb + 1) < unsigned(T)) cp_async8(sl, lpl + base + u - 1); else *sl = 0.0;
                if (e >= 0) base += min(min(e + 1, c2), U + T - 1 - e);
                ++e;
                ++tb;
            } else {
                // step with d = e at column u needs blank(e-u, u) and label(e-u, u)
                const bool cell = unsigned(tb) < unsigned(T);
                if (cell) cp_async8(sb, lpb + base + u); else *sb = 0.0;
                if (cell && u < U) cp_async8(sl, lpl + base + u); else *sl = 0.0;
                --e;
                --tb;
                if (e >= 0) base -= min(min(e + 1, c2), U + T - 1 - e);
            }
            cp_async_commit();
        };
#pragma unroll
        for (int k = 0; k < R; ++k) issue(k);
        cp_async_wait<R - 2>();  // operands of steps 0 and 1 are in place
        asm volatile("bar.sync 1, %0;" ::"r"(n_sync) : "memory");      // start barrier: steps 0 and 1 are staged
        // second barrier: the compute warps have taken the operands of step 0 out of slot 0, which the first
        // iteration below refills
        asm volatile("bar.sync 1, %0;" ::"r"(n_sync) : "memory");

        // step s: refill slot s % R with the operands of step s+R
        for (int s0 = 0; s0 < nd; s0 += R) {
#pragma unroll
            for (int k = 0; k < R; ++k) {
                if (s0 + k >= nd) break;
                issue(k);
                cp_async_wait<R - 2>();
                asm volatile("bar.sync 1, %0;" ::"r"(n_sync) : "memory");
            }
        }
        cp_async_wait<0>();
        return;
    }

    // ---- compute warp. Cells outside the lattice count as -inf: both result rows start at -inf (the "previous
    // step" of step 0 and every column's virtual predecessor row), and edge columns read the permanent -inf element.
    v0[u] = -INFINITY;
    v1[u] = -INFINITY;
    if (u == 0) {
        v0[n_cols] = -INFINITY;
        v1[n_cols] = -INFINITY;
    }
    double prev = (u == (BETA ? U : 0)) ? 0.0 : -INFINITY;
    const int nb_col = BETA ? (u >= U ? n_cols : u + 1) : (u == 0 ? n_cols : u - 1);
    // frame index of this column's cell one step before step 0 (parked far outside for columns beyond U)
    int t_prev = u <= U ? (BETA ? nd - u : -u - 1) : INT_MIN / 2;
    asm volatile("bar.sync 1, %0;" ::"r"(n_sync) : "memory");  // start barrier: operands of steps 0 and 1 are staged
    double cur_b = st_b[0], cur_l = st_l[0];
    int cur_base = diag_base[0], prev_base = 0;
    asm volatile("bar.sync 1, %0;" ::"r"(n_sync) : "memory");  // slot 0 is read: the helper may refill it
    for (int s0 = 0; s0 < nd; s0 += R) {
#pragma unroll
        for (int k = 0; k < R; ++k) {
            if (s0 + k >= nd) break;
            // The result of the previous step goes out first, so that the store has the whole step to complete
            // before this warp arrives at the barrier. It lies on the diagonal whose operands this step reads
            // (alpha) / the previous step read (beta).
            if (unsigned(t_prev) < unsigned(T)) out[(BETA ? prev_base : cur_base) + u] = prev;
            t_prev += BETA ? -1 : 1;
            const double nxt_b = st_b[((k + 1) % R) * n_cols];
            const double nxt_l = st_l[((k + 1) % R) * n_cols];
            const int nxt_base = diag_base[(k + 1) % R];
            const double nb = (k & 1) ? v0[nb_col] : v1[nb_col];  // the neighbour's result of the previous step
            const double v = lse2_late<F64>(prev + cur_b, cur_l, nb, lse_tab);
            if (k & 1) v1[u] = v; else v0[u] = v;
            prev = v;
            cur_b = nxt_b;
            cur_l = nxt_l;
            prev_base = cur_base;
            cur_base = nxt_base;
            asm volatile("bar.sync 1, %0;" ::"r"(n_sync) : "memory");
        }
    }
    if (unsigned(t_prev) < unsigned(T)) out[(BETA ? prev_base : cur_base) + u] = prev;  // the last step's result
    if (!BETA) {
        if (u == U) *ll_out = prev + __ldg(lpb + int64_t(T) * m - 1);
    } else {
        if (u == 0) *ll_out = prev;
    }
}

// ------------------------------------------------------------------------------------------------ split-role, rounds
// Wide lattices (more than kRoundsMinCols columns). With many warps in the CTA the step's barrier is the costly part,
// and the helpers do not need to meet the compute warps on every step. Here the compute warps close a step on a
// barrier of their own (half the threads), and helpers and compute warps meet once per round of Q steps:
//   ring of R = 16 operand slots (step x in slot x % R), V = 8 result rows (step x in row x % V);
//   round r, compute warps: steps Qr .. Qr+Q-1, operands read one step ahead as above;
//   round r, helper warps : for x = Qr-Q+1 .. Qr, store the result of step x-1 (written during round r-1) and refill
//                           the slot of step x (read during round r-1 at the latest) with the operands of step x+R.
// At the barrier that ends round r the operands of steps up to Qr+2Q are needed; they were issued in round r-2 at the
// latest, so one copy group per round and `wait_group 2` leave every copy between two and three rounds to land. The
// prologue stages steps 0 .. R-Q and the first round continues from there. Rows of results live for two rounds: the
// compute warps write row x % V again Q*2 = V steps later, after the barrier that ends the round in which the helpers
// read it. Measured against the per-step barrier above: 0.194 vs 0.204 us per diagonal at 256 columns, 0.248 vs
// 0.265 at 384, 0.306 vs 0.332 at 512; slower below about 160 columns (0.170 vs 0.164 at 151; more shared memory,
// longer prologue). Here the helpers keep the stores: the compute warps of a wide lattice have no issue slots to
// spare (with the stores moved to them as above: 0.202 at 256 columns, 0.321 at 512). The
// double-precision recursion (libm exp/log1p on the chain) measured slower this way up to 384 columns (0.84 vs 0.73 us
// per diagonal at 256) and stays on the per-step barrier.
template <bool F64, bool BETA>
__device__ __forceinline__ void run_direction_rounds(int T, int U, const double *__restrict__ lpb,
                                                     const double *__restrict__ lpl, double *__restrict__ out,
                                                     double *__restrict__ ll_out, int n_cols, int n_sync,
                                                     double *stage, double *vbuf,
                                                     const float4 *__restrict__ lse_tab, bool helper, int u)
{
    constexpr int R = kRoundsRing, Q = 4, V = kRoundsRows;
    const int m = U + 1;
    const int nd = T + U;
    const int n_rounds = (nd + Q - 1) / Q;
    double *st_b = stage + u;
    double *st_l = stage + R * n_cols + u;
    const int vstride = n_cols + 1;

    if (helper) {
        const int c2 = (U <= T - 1) ? U + 1 : T - 1;
        int e = BETA ? nd - 1 : -1;
        int base = BETA ? T * m - 1 - U : 0;
        int tb = u <= U ? e - u : INT_MIN / 2;
        int sbase[R];
#pragma unroll
        for (int k = 0; k < R; ++k) sbase[k] = 0;
        auto issue = [&](int k) {
            sbase[k] = base;
            double *sb = st_b + k * n_cols, *sl = st_l + k * n_cols;
            if (!BETA) {
                if (unsigned(tb) < unsigned(T - 1)) cp_async8(sb, lpb + base + u); else *sb = 0.0;
                if (u >= 1 && unsigned(tb + 1) < unsigned(T)) cp_async8(sl, lpl + base + u - 1); else *sl = 0.0;
                if (e >= 0) base += min(min(e + 1, c2), U + T - 1 - e);
                ++e;
                ++tb;
            } else {
                const bool cell = unsigned(tb) < unsigned(T);
                if (cell) cp_async8(sb, lpb + base + u); else *sb = 0.0;
                if (cell && u < U) cp_async8(sl, lpl + base + u); else *sl = 0.0;
                --e;
                --tb;
                if (e >= 0) base -= min(min(e + 1, c2), U + T - 1 - e);
            }
        };
#pragma unroll
        for (int k = 0; k <= R - Q; ++k) issue(k);  // steps 0 .. R-Q
        cp_async_commit();
        cp_async_wait<0>();
        // frame index of this column at step x-1, for x = -(Q-1)
        int tprev = u <= U ? (BETA ? nd - u + (Q - 1) : -u - 1 - (Q - 1)) : INT_MIN / 2;
        int last_base = 0;
        asm volatile("bar.sync 1, %0;" ::"r"(n_sync) : "memory");
        asm volatile("bar.sync 1, %0;" ::"r"(n_sync) : "memory");
        // round r (compute runs steps Qr .. Qr+Q-1): x = Qr-(Q-1) .. Qr; store the result of step x-1 (previous round),
        // then refill the slot of step x with the operands of step x+R
        bool done = false;
        for (int s0 = 0; !done; s0 += R) {
#pragma unroll
            for (int q = 0; q < R / Q; ++q) {
                const bool drain = (s0 + Q * q) >= Q * n_rounds;
#pragma unroll
                for (int j = 0; j < Q; ++j) {
                    constexpr int RQ = R - Q + 1;
                    const int slot = (Q * q + j + RQ) % R;
                    const int row = (Q * q + j + V - Q) % V;
                    const int this_base = sbase[slot];
                    const int out_base = BETA ? last_base : this_base;
                    last_base = this_base;
                    if (unsigned(tprev) < unsigned(T)) out[out_base + u] = vbuf[row * vstride + u];
                    tprev += BETA ? -1 : 1;
                    if (!drain) issue(slot);
                }
                if (drain) { done = true; break; }
                cp_async_commit();
                cp_async_wait<2>();
                asm volatile("bar.sync 1, %0;" ::"r"(n_sync) : "memory");
            }
        }
        cp_async_wait<0>();
        return;
    }

#pragma unroll
    for (int i = 0; i < V; ++i) {
        vbuf[i * vstride + u] = -INFINITY;
        if (u == 0) vbuf[i * vstride + n_cols] = -INFINITY;
    }
    double prev = (u == (BETA ? U : 0)) ? 0.0 : -INFINITY;
    const int nb_col = BETA ? (u >= U ? n_cols : u + 1) : (u == 0 ? n_cols : u - 1);
    asm volatile("bar.sync 1, %0;" ::"r"(n_sync) : "memory");
    double cur_b = st_b[0], cur_l = st_l[0];
    asm volatile("bar.sync 1, %0;" ::"r"(n_sync) : "memory");
    for (int s0 = 0; s0 < nd; s0 += R) {
#pragma unroll
        for (int q = 0; q < R / Q; ++q) {
            if (s0 + Q * q >= nd) break;
#pragma unroll
            for (int j = 0; j < Q; ++j) {
                const int k = Q * q + j;
                if (s0 + k < nd) {
                    const double nxt_b = st_b[((k + 1) % R) * n_cols];
                    const double nxt_l = st_l[((k + 1) % R) * n_cols];
                    const double nb = vbuf[((k + V - 1) % V) * vstride + nb_col];
                    const double v = lse2_late<F64>(prev + cur_b, cur_l, nb, lse_tab);
                    vbuf[(k % V) * vstride + u] = v;
                    prev = v;
                    cur_b = nxt_b;
                    cur_l = nxt_l;
                }
                if (j < Q - 1) asm volatile("bar.sync 2, %0;" ::"r"(n_cols) : "memory");
            }
            asm volatile("bar.sync 1, %0;" ::"r"(n_sync) : "memory");
        }
    }
    if (!BETA) {
        if (u == U) *ll_out = prev + __ldg(lpb + int64_t(T) * m - 1);
    } else {
        if (u == 0) *ll_out = prev;
    }
}

template <int R, bool F64, bool ROUNDS>
__global__ void __launch_bounds__(1024)
wavefront_split_kernel(WaveArgs<typename std::conditional<F64, double, float>::type> g)
{
    extern __shared__ __align__(16) double stage[];
    __shared__ double edge[2][32];
    __shared__ float4 lse_tab[F64 ? 1 : kLseNodes];
    __shared__ int last_flag;
    __shared__ int diag_base[16];  // per ring slot: stream offset of the diagonal its operands come from
    const Workspace &w = g.w;
    if (w.status[0] & CWRNNT_ST_FATAL) return;

    const int n = w.order[blockIdx.x / g.n_dirs];
    // Another launch's sequence: leave at once. Only CTAs that run a sequence-direction take a completion ticket (each
    // sequence-direction runs in exactly one launch of the step), so leaving costs no atomic and no fence.
    if (other_group(g, n)) return;
    const bool beta_dir = (g.n_dirs == 1) || (blockIdx.x & 1);
    const int T = g.lx[n], U = g.ly[n];
    const int64_t off = w.off[n];
    const int half = blockDim.x >> 1;                 // compute threads launched (then as many helpers)
    const int n_cols = min(half, (U + 1 + 31) & ~31);  // columns padded to whole warps for this sequence
    // threads [0, n_cols) compute, [half, half + n_cols) help; the others leave (whole warps)
    const int tid = threadIdx.x;
    const bool is_helper = tid >= half;
    const int col = is_helper ? tid - half : tid;
    if (col >= n_cols) return;
    const int n_sync = 2 * n_cols;
    const int vtid = is_helper ? n_cols + col : col;  // dense numbering of the threads that stay
    if (!F64) build_lse_table(lse_tab, vtid, n_sync);
    asm volatile("bar.sync 1, %0;" ::"r"(n_sync) : "memory");
    double *vbuf = stage + 2 * R * n_cols;
    if constexpr (ROUNDS) {
        if (beta_dir)
            run_direction_rounds<F64, true>(T, U, w.lp_blank + off, w.lp_label + off, w.beta + off, w.ll_beta + n,
                                            n_cols, n_sync, stage, vbuf, lse_tab, is_helper, col);
        else
            run_direction_rounds<F64, false>(T, U, w.lp_blank + off, w.lp_label + off, w.alpha + off, w.ll_alpha + n,
                                             n_cols, n_sync, stage, vbuf, lse_tab, is_helper, col);
    } else {
        if (beta_dir)
            run_direction_split<R, F64, true>(T, U, w.lp_blank + off, w.lp_label + off, w.beta + off, w.ll_beta + n,
                                              n_cols, n_sync, stage, vbuf, diag_base, lse_tab, is_helper, col);
        else
            run_direction_split<R, F64, false>(T, U, w.lp_blank + off, w.lp_label + off, w.alpha + off,
                                               w.ll_alpha + n, n_cols, n_sync, stage, vbuf, diag_base, lse_tab,
                                               is_helper, col);
    }
    // the compute warps finalise (helpers are done; n_cols threads with dense ids 0..n_cols-1)
    if (is_helper) return;
    finalize_if_last(g, n_cols, edge, &last_flag);
}

// Dynamic shared memory above the default cap needs a per-kernel opt-in. It is asked for once per (device, kernel)
// and size, so that repeated launches - and launches under stream capture after a first plain call - make no
// attribute call at all.
static cudaError_t opt_in_smem_impl(const void *kernel, size_t smem, int threads)
{
    if (smem <= 32 * 1024) return cudaSuccess;  // default cap is 48 KB including ~9 KB of static arrays
    static std::mutex lock;
    static std::map<std::pair<int, const void *>, size_t> granted;
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    std::lock_guard<std::mutex> hold(lock);
    size_t &have = granted[std::make_pair(device, kernel)];
    if (have >= smem) return cudaSuccess;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e == cudaSuccess)
        have = smem;
    else
        std::fprintf(stderr, "cwrnnt: cannot opt in to %zu bytes of shared memory (%d threads): %s\n", smem, threads,
                     cudaGetErrorString(e));
    return e;
}
template <typename K>
static cudaError_t opt_in_smem(K kernel, size_t smem, int threads)
{
    return opt_in_smem_impl(reinterpret_cast<const void *>(kernel), smem, threads);
}

// True when `grid` CTAs of `kernel` with `threads` threads and `smem` bytes of dynamic shared memory are all resident
// at once (registers, shared memory and thread slots counted by the occupancy calculator; asked once per device and
// launch shape). The rounds variant takes 2.2 times the shared memory of the per-step one; on a launch that no longer
// fits the device in one wave the second wave costs more than the cheaper barrier saves (512 CTAs of 256 columns:
// 234 us against 213 us).
static bool one_wave(const void *kernel, int grid, int threads, size_t smem)
{
    struct Shape {
        int device, threads;
        size_t smem;
        bool operator<(const Shape &o) const
        {
            return device != o.device ? device < o.device : threads != o.threads ? threads < o.threads : smem < o.smem;
        }
    };
    static std::mutex lock;
    static std::map<Shape, int64_t> resident;  // CTAs the whole device holds at once
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return false;
    std::lock_guard<std::mutex> hold(lock);
    const Shape key{device, threads, smem};
    auto it = resident.find(key);
    if (it == resident.end()) {
        int sms = 0, per_sm = 0;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
        it = resident.emplace(key, int64_t(sms) * per_sm).first;
    }
    return int64_t(grid) <= it->second;
}

template <bool F64>
static cudaError_t launch_wavefront_t(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                                      void *costs, void *loss, const ShardOutput *shard, cudaStream_t s,
                                      GroupPlan plan, int group)
{
    using CostT = typename std::conditional<F64, double, float>::type;
    if (p.B == 0) return cudaSuccess;
    WaveArgs<CostT> g{};
    g.lx = lx;
    g.ly = ly;
    g.B = p.B;
    g.flags = p.flags;
    g.mean_den = p.mean_denominator;
    g.n_dirs = (p.flags & CWRNNT_COSTS_ONLY) ? 1 : 2;
    g.w = w;
    g.costs = static_cast<CostT *>(costs);
    g.loss = static_cast<CostT *>(loss);
    if (shard && shard->cost_vector) {
        g.global_ids = shard->global_ids;
        g.n_global = shard->n_global;
        g.cost_vec = static_cast<CostT *>(shard->cost_vector);
    }
    const int cols = p.max_u + 1;
    const int grid = p.B * g.n_dirs;
    g.plan = plan;
    g.group = group;
    g.ticket_total = unsigned(grid);  // one ticket per sequence-direction, whichever launch of the step runs it
    cudaError_t e = cudaSuccess;

    if (cols <= 512) {
        // split-role path: one compute and one helper thread per column
        constexpr int R = 8;
        const int half = (cols + 31) & ~31;
        const int threads = 2 * half;
        const size_t smem = (size_t(2 * R + 2) * half + 2) * sizeof(double);
        const size_t wide = (size_t(2 * kRoundsRing + kRoundsRows) * half + kRoundsRows) * sizeof(double);
        if constexpr (!F64) {
            if (half > kRoundsMinCols) {
                auto rounds = wavefront_split_kernel<kRoundsRing, false, true>;
                if ((e = opt_in_smem(rounds, wide, threads)) != cudaSuccess) return e;
                if (one_wave(reinterpret_cast<const void *>(rounds), grid, threads, wide)) {
                    rounds<<<grid, threads, wide, s>>>(g);
                    return cudaGetLastError();
                }
            }
        }
        if ((e = opt_in_smem(wavefront_split_kernel<R, F64, false>, smem, threads)) != cudaSuccess) return e;
        wavefront_split_kernel<R, F64, false><<<grid, threads, smem, s>>>(g);
        return cudaGetLastError();
    }
    const int C = cols <= 1024 ? 1 : (cols <= 2048 ? 4 : 8);
    const int per_thread_cols = (cols + C - 1) / C;
    const int threads = (per_thread_cols + 31) & ~31;
    const int R = C == 1 ? 8 : (threads * C <= 1280 ? 8 : (threads * C <= 2560 ? 4 : 2));  // deepest ring <= 160 KB
    const size_t smem = size_t(2) * R * C * threads * sizeof(double);
#define CWRNNT_LAUNCH_WAVEFRONT(CC, RR)                                                      \
    {                                                                                        \
        if ((e = opt_in_smem(wavefront_kernel<CC, RR, F64>, smem, threads)) != cudaSuccess) return e; \
        wavefront_kernel<CC, RR, F64><<<grid, threads, smem, s>>>(g);                        \
    }
#define CWRNNT_PICK_RING(CC)                                   \
    {                                                          \
        if (R == 8) CWRNNT_LAUNCH_WAVEFRONT(CC, 8)             \
        else if (R == 4) CWRNNT_LAUNCH_WAVEFRONT(CC, 4)        \
        else CWRNNT_LAUNCH_WAVEFRONT(CC, 2)                    \
    }
    if (C == 1) CWRNNT_LAUNCH_WAVEFRONT(1, 8)
    else if (C == 4) CWRNNT_PICK_RING(4)
    else CWRNNT_PICK_RING(8)
#undef CWRNNT_PICK_RING
#undef CWRNNT_LAUNCH_WAVEFRONT
    return cudaGetLastError();
}

cudaError_t launch_wavefront(const cwrnnt_problem &p, const int32_t *lx, const int32_t *ly, const Workspace &w,
                             void *costs, void *loss, const ShardOutput *shard, cudaStream_t s, GroupPlan plan,
                             int group)
{
    return p.dtype == CWRNNT_F64 ? launch_wavefront_t<true>(p, lx, ly, w, costs, loss, shard, s, plan, group)
                                 : launch_wavefront_t<false>(p, lx, ly, w, costs, loss, shard, s, plan, group);
}

}  // namespace cwrnnt
