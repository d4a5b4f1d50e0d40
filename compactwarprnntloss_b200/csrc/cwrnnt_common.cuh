// Shared device/host definitions of the sm_100a RNN-T loss engine: workspace layout, element-type traits,
// lattice index arithmetic. Internal; the public boundary is include/cwarp_rnnt_b200.h.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "cwarp_rnnt_b200.h"

namespace cwrnnt {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; persistent grids are sized in multiples of this
constexpr int kMaxGroups = 8;  // sequence groups of a pipelined step (cwrnnt_loss_grad)

// Pipelined step: the rows are cut into `count` nominal ranges of `range_rows` rows; a sequence belongs to the group
// of the range that holds its LAST row, so group g is complete as soon as ranges 0..g have been gathered.
struct GroupPlan {
    int count;           // 1 = no grouping
    int64_t range_rows;  // rows per nominal range (the last range may be shorter)
};
__host__ __device__ inline int group_of_row(int64_t row, const GroupPlan &plan)
{
    const int64_t g = row / plan.range_rows;
    return int(g < plan.count - 1 ? g : plan.count - 1);
}

// ------------------------------------------------------------------------------------------------ workspace
// One caller-provided allocation, carved deterministically from (n_rows, B) so forward and backward agree.
//   header   : 4 status words + completion ticket + row bounds of the sequence groups of a pipelined step
//   off      : int64 [B+1]   exclusive prefix sum of T_n*(U_n+1) (row offset of each sequence)
//   order    : int32 [B]     sequences by descending T_n+U_n (wavefront critical path), longest first
//   ll_alpha : double [B]    alpha(T-1,U) + blank(T-1,U)
//   ll_beta  : double [B]    beta(0,0)
//   lse      : double [rows] log-sum-exp of each logits row (0 for log-prob input)
//   lp_blank : double [rows] log P(blank | t,u), stored DIAGONAL-MAJOR inside each sequence (see diag_index)
//   lp_label : double [rows] log P(y_u   | t,u), same order
//   alpha    : double [rows] forward variables, diagonal-major like lp_blank
//   beta     : double [rows] backward variables, same order
struct Workspace {
    int32_t *status;
    unsigned int *ticket;
    int64_t *bounds;  // [kMaxGroups + 1] first row of each sequence group, then n_rows (written by K0)
    int64_t *off;
    int32_t *order;
    double *ll_alpha;
    double *ll_beta;
    double *lse;
    double *lp_blank;
    double *lp_label;
    double *alpha;
    double *beta;
};

__host__ __device__ inline int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

// Returns total bytes; fills `w` when base != nullptr.
__host__ inline int64_t carve_workspace(int64_t n_rows, int32_t B, void *base, Workspace *w)
{
    int64_t at = 0;
    auto take = [&](int64_t bytes) {
        int64_t here = at;
        at = align_up(at + bytes, 256);
        return here;
    };
    const int64_t rows = n_rows > 0 ? n_rows : 1;
    int64_t o_hdr = take(256);
    int64_t o_off = take(8 * (int64_t(B) + 1));
    int64_t o_ord = take(4 * int64_t(B));
    int64_t o_lla = take(8 * int64_t(B));
    int64_t o_llb = take(8 * int64_t(B));
    int64_t o_lse = take(8 * rows);
    int64_t o_lpb = take(8 * rows);
    int64_t o_lpl = take(8 * rows);
    int64_t o_alp = take(8 * rows);
    int64_t o_bet = take(8 * rows);
    if (base && w) {
        char *b = static_cast<char *>(base);
        w->status = reinterpret_cast<int32_t *>(b + o_hdr);
        w->ticket = reinterpret_cast<unsigned int *>(b + o_hdr + 16);
        w->bounds = reinterpret_cast<int64_t *>(b + o_hdr + 64);
        w->off = reinterpret_cast<int64_t *>(b + o_off);
        w->order = reinterpret_cast<int32_t *>(b + o_ord);
        w->ll_alpha = reinterpret_cast<double *>(b + o_lla);
        w->ll_beta = reinterpret_cast<double *>(b + o_llb);
        w->lse = reinterpret_cast<double *>(b + o_lse);
        w->lp_blank = reinterpret_cast<double *>(b + o_lpb);
        w->lp_label = reinterpret_cast<double *>(b + o_lpl);
        w->alpha = reinterpret_cast<double *>(b + o_alp);
        w->beta = reinterpret_cast<double *>(b + o_bet);
    }
    return at;
}

// ------------------------------------------------------------------------------------------------ lattice indexing
// Inside one sequence (T frames, m = U+1 columns) the gathered log-probs are stored diagonal by diagonal
// (d = t+u ascending, u ascending inside a diagonal) so that the wavefront kernel, whose thread u visits cell
// (d-u, u) at step d, reads one contiguous, fully coalesced stream. cells_before(d) counts the cells with t+u < d:
// inclusion-exclusion over the two box constraints t < T, u < m of the triangle count d(d+1)/2.
// (32-bit operands, one widening multiply each; a sequence has fewer than 2^31 cells.)
__host__ __device__ inline int64_t tri(int x)
{
    return x > 0 ? int64_t((uint64_t(uint32_t(x)) * uint64_t(uint32_t(x) + 1u)) >> 1) : 0;
}

__host__ __device__ inline int64_t cells_before(int d, int T, int m)
{
    return tri(d) - tri(d - T) - tri(d - m) + tri(d - T - m);
}

__host__ __device__ inline int64_t diag_index(int t, int u, int T, int m)
{
    const int d = t + u;
    const int lo = d - (T - 1) > 0 ? d - (T - 1) : 0;
    return cells_before(d, T, m) + (u - lo);
}

// Positions, inside a sequence's diagonal-major arrays, of cell (t,u) and of its successor (t+1,u) on the next
// diagonal; the other successor (t,u+1) sits right after the latter. The successor position is meaningful only when
// that cell exists.
__host__ __device__ inline void diag_cell_and_next(int t, int u, int T, int m, int64_t *cell, int64_t *next)
{
    const int d = t + u, U = m - 1;
    const int lo = d - (T - 1) > 0 ? d - (T - 1) : 0;
    const int hi = d < U ? d : U;
    const int lo1 = d + 1 - (T - 1) > 0 ? d + 1 - (T - 1) : 0;
    const int64_t before = cells_before(d, T, m);
    *cell = before + (u - lo);
    *next = before + (hi - lo + 1) + (u - lo1);
}

// ------------------------------------------------------------------------------------------------ element traits
template <typename T>
struct Elt;

template <>
struct Elt<float> {
    using acc = float;    // arithmetic type of the streaming kernels
    using cost = float;   // type of costs / loss / grad_costs
    static constexpr int VE = 4;  // elements per 16-byte vector
    static __device__ __forceinline__ void unpack(const uint4 &v, float (&e)[4])
    {
        e[0] = __uint_as_float(v.x);
        e[1] = __uint_as_float(v.y);
        e[2] = __uint_as_float(v.z);
        e[3] = __uint_as_float(v.w);
    }
    static __device__ __forceinline__ uint4 pack(const float (&e)[4])
    {
        return make_uint4(__float_as_uint(e[0]), __float_as_uint(e[1]), __float_as_uint(e[2]), __float_as_uint(e[3]));
    }
    static __device__ __forceinline__ float to_acc(float v) { return v; }
    static __device__ __forceinline__ float from_acc(float v) { return v; }
    // largest element of a vector (NaNs are skipped, as by a chain of `>` comparisons)
    static __device__ __forceinline__ float vec_max(const uint4 &v)
    {
        return fmaxf(fmaxf(__uint_as_float(v.x), __uint_as_float(v.y)),
                     fmaxf(__uint_as_float(v.z), __uint_as_float(v.w)));
    }
};

template <>
struct Elt<__half> {
    using acc = float;
    using cost = float;
    static constexpr int VE = 8;
    static __device__ __forceinline__ void unpack(const uint4 &v, float (&e)[8])
    {
        const unsigned int w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = *reinterpret_cast<const __half2 *>(&w[i]);
            float2 f = __half22float2(h);
            e[2 * i] = f.x;
            e[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ uint4 pack(const float (&e)[8])
    {
        unsigned int w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __half2 h = __floats2half2_rn(e[2 * i], e[2 * i + 1]);
            w[i] = *reinterpret_cast<unsigned int *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    static __device__ __forceinline__ float to_acc(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_acc(float v) { return __float2half_rn(v); }
    // the maximum is exact in any precision: three packed half2 maxima, then one widening
    static __device__ __forceinline__ float vec_max(const uint4 &v)
    {
        const __half2 a = *reinterpret_cast<const __half2 *>(&v.x), b = *reinterpret_cast<const __half2 *>(&v.y);
        const __half2 c = *reinterpret_cast<const __half2 *>(&v.z), d = *reinterpret_cast<const __half2 *>(&v.w);
        const float2 m = __half22float2(__hmax2(__hmax2(a, b), __hmax2(c, d)));
        return fmaxf(m.x, m.y);
    }
};

template <>
struct Elt<__nv_bfloat16> {
    using acc = float;
    using cost = float;
    static constexpr int VE = 8;
    static __device__ __forceinline__ void unpack(const uint4 &v, float (&e)[8])
    {
        const unsigned int w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            // a bf16 is the upper half of a float: widen by shifting
            e[2 * i] = __uint_as_float(w[i] << 16);
            e[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ uint4 pack(const float (&e)[8])
    {
        unsigned int w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(e[2 * i], e[2 * i + 1]);
            w[i] = *reinterpret_cast<unsigned int *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    static __device__ __forceinline__ float to_acc(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_acc(float v) { return __float2bfloat16_rn(v); }
    static __device__ __forceinline__ float vec_max(const uint4 &v)
    {
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162 *>(&v.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162 *>(&v.y);
        const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162 *>(&v.z);
        const __nv_bfloat162 d = *reinterpret_cast<const __nv_bfloat162 *>(&v.w);
        const __nv_bfloat162 m = __hmax2(__hmax2(a, b), __hmax2(c, d));
        const unsigned int w = *reinterpret_cast<const unsigned int *>(&m);
        return fmaxf(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    }
};

template <>
struct Elt<double> {
    using acc = double;
    using cost = double;
    static constexpr int VE = 2;
    static __device__ __forceinline__ void unpack(const uint4 &v, double (&e)[2])
    {
        e[0] = __hiloint2double(int(v.y), int(v.x));
        e[1] = __hiloint2double(int(v.w), int(v.z));
    }
    static __device__ __forceinline__ uint4 pack(const double (&e)[2])
    {
        return make_uint4(unsigned(__double2loint(e[0])), unsigned(__double2hiint(e[0])),
                          unsigned(__double2loint(e[1])), unsigned(__double2hiint(e[1])));
    }
    static __device__ __forceinline__ double to_acc(double v) { return v; }
    static __device__ __forceinline__ double from_acc(double v) { return v; }
    static __device__ __forceinline__ double vec_max(const uint4 &v)
    {
        return fmax(__hiloint2double(int(v.y), int(v.x)), __hiloint2double(int(v.w), int(v.z)));
    }
};

__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Softmax numerators exp(v - c) of one row and the matching log-sum-exp. Float: the shift is carried in base-2 units
// (c2 = c * log2 e, rounded once), each term is one FFMA and one MUFU ex2 (relative error ~2^-22; the FFMA rounds
// only the small difference v*log2e - c2), and the rounding of c2 is undone exactly when the row's log-sum-exp is
// assembled in double: lse = c2 * ln 2 + ln(sum).
template <typename A>
struct RowShift;
template <>
struct RowShift<float> {
    float c2;
    __device__ __forceinline__ explicit RowShift(float c) : c2(c * 1.4426950408889634f) {}
    __device__ __forceinline__ float term(float v) const { return ex2_approx(fmaf(v, 1.4426950408889634f, -c2)); }
    // ln(s) for s >= 1 with absolute error near 1e-7 even when the result is ~8: the binary exponent is split off
    // (exact in double) and logf sees only the mantissa in [0.5, 1).
    __device__ __forceinline__ double lse(float s) const
    {
        int e;
        const float f = frexpf(s, &e);
        return (double(c2) + double(e)) * 0.6931471805599453 + double(logf(f));
    }
};
template <>
struct RowShift<double> {
    double c;
    __device__ __forceinline__ explicit RowShift(double c_) : c(c_) {}
    __device__ __forceinline__ double term(double v) const { return exp(v - c); }
    __device__ __forceinline__ double lse(double s) const { return c + log(s); }
};

// exp(v - c) where c is a stored log-sum-exp (gradient kernel): subtract first, so the argument's rounding error
// scales with |v - c| and not with |v|.
__device__ __forceinline__ float exp_shifted(float v, float c) { return ex2_approx((v - c) * 1.4426950408889634f); }
__device__ __forceinline__ double exp_shifted(double v, double c) { return exp(v - c); }

// 128-bit global loads/stores with cache hints. `nc` = read-only path; `cs` = evict-first streaming.
__device__ __forceinline__ uint4 ld_nc(const uint4 *p) { return __ldg(p); }
__device__ __forceinline__ uint4 ld_stream(const uint4 *p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(uint4 *p, const uint4 &v) { __stcs(p, v); }

// Sequence lookup for a row: the largest n with off[n] <= r. `hint` is a running cursor (rows are visited in
// ascending order by each group), so the common case is zero or one step; falls back to bisection on a long jump.
__device__ __forceinline__ int find_sequence(const int64_t *__restrict__ off, int B, int64_t r, int hint)
{
    int n = hint;
    if (r < __ldg(off + n)) n = 0;
    int steps = 0;
    while (n + 1 < B && r >= __ldg(off + n + 1)) {
        ++n;
        if (++steps == 4) {  // long jump: bisect in (n, B)
            int lo = n, hi = B;  // invariant: off[lo] <= r < off[hi] (off[B] = total > r)
            while (hi - lo > 1) {
                int mid = (lo + hi) >> 1;
                if (r >= __ldg(off + mid))
                    lo = mid;
                else
                    hi = mid;
            }
            return lo;
        }
    }
    return n;
}

// Factor applied to a sequence's cost (and hence to its gradient weight) before any reduction.
__device__ __forceinline__ double sequence_scale(int flags, int T)
{
    return (flags & CWRNNT_AVERAGE_FRAMES) ? 1.0 / double(T) : 1.0;
}

// The reference's forward/backward consistency guard (cwarp_cuda_rnnt_kernel.cu:350-366): `a` = alpha(T-1,U) + the
// final blank, `b` = beta(0,0) are the same log-likelihood computed from both ends. When they differ by more than 1e-3
// relative to the larger one the reference prints a warning and uses their mean; here the mean is used and `gap` is
// raised (it becomes the CWRNNT_ST_FWD_BWD_GAP status bit). Otherwise beta's value stands.
__device__ __forceinline__ double guarded_loglik(double a, double b, bool &gap)
{
    const double big = fmax(a, b);
    if (fabs(a - b) / fabs(big) > 1e-3) {
        gap = true;
        return 0.5 * (a + b);
    }
    return b;
}

}  // namespace cwrnnt
