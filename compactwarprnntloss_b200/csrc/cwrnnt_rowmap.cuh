// Row -> (sequence, frame, column) bookkeeping and vector-shape dispatch shared by the two streaming kernels. Internal.
#pragma once
#include "cwrnnt_common.cuh"

namespace cwrnnt {

constexpr int kStreamThreads = 256;  // 8 warps per CTA in the streaming kernels

// Rows covered by one launch of a streaming kernel: [begin, end). A pipelined step knows the rows of a sequence group
// only on the device (K0 computes them): then `dev` points at the pair and begin/end are ignored.
struct RowRange {
    int64_t begin, end;
    const int64_t *dev;
    __device__ __forceinline__ void resolve(int64_t &b, int64_t &e) const
    {
        b = dev ? __ldg(dev) : begin;
        e = dev ? __ldg(dev + 1) : end;
    }
};

// Position of one lattice row while a group of lanes walks a contiguous run of rows. Found once per run by bisection
// and one division, then advanced with a handful of integer operations per row - rows are visited in memory order,
// which is (sequence, t, u) order.
struct RowWalker {
    int n;        // sequence
    int T, U;     // its lengths
    int t, u;     // lattice cell of the current row
    int64_t off;  // first row of the sequence (also the base of its diagonal-major arrays)
    int64_t at;   // diagonal-major position of (t,u) inside the sequence

    __device__ __forceinline__ void start(int64_t r, const int64_t *__restrict__ offs, int B,
                                          const int32_t *__restrict__ lx, const int32_t *__restrict__ ly)
    {
        int lo = 0, hi = B;  // invariant: offs[lo] <= r < offs[hi]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (r >= __ldg(offs + mid))
                lo = mid;
            else
                hi = mid;
        }
        n = lo;
        load_sequence(offs, lx, ly);
        const unsigned rel = unsigned(r - off);  // a sequence has fewer than 2^31 cells
        const unsigned m = unsigned(U) + 1u;
        t = int(rel / m);
        u = int(rel - unsigned(t) * m);
        at = diag_index(t, u, T, U + 1);
    }
    __device__ __forceinline__ void load_sequence(const int64_t *__restrict__ offs, const int32_t *__restrict__ lx,
                                                  const int32_t *__restrict__ ly)
    {
        off = __ldg(offs + n);
        T = __ldg(lx + n);
        U = __ldg(ly + n);
    }
    // Label of the current row clamped into [0,V), or -1 in the last column; reports an out-of-range label.
    __device__ __forceinline__ int label(const int32_t *__restrict__ y, int y_stride, int V, bool &bad) const
    {
        if (u >= U) return -1;
        int k = __ldg(y + int64_t(n) * y_stride + u);
        if (k < 0 || k >= V) {
            bad = true;
            k = k < 0 ? 0 : V - 1;
        }
        return k;
    }
    // Diagonal-major position of the successor (t+1,u); (t,u+1) is the element after it.
    __device__ __forceinline__ int64_t next_diag() const
    {
        const int d = t + u;
        const int lo0 = max(0, d - (T - 1)), lo1 = max(0, d + 1 - (T - 1));
        return at + (min(d, U) - lo0 + 1) - (lo1 - lo0);
    }
    // Move to the next row in memory order. `more` = the run continues (avoids reading past the last sequence).
    __device__ __forceinline__ void advance(const int64_t *__restrict__ offs, int B, const int32_t *__restrict__ lx,
                                            const int32_t *__restrict__ ly)
    {
        if (u < U) {
            // (t,u) on diagonal d -> (t,u+1) on diagonal d+1
            const int d = t + u;
            at += min(d, U) + 2 - max(0, d + 1 - (T - 1));
            ++u;
            return;
        }
        u = 0;
        if (++t == T) {
            t = 0;
            if (++n < B) load_sequence(offs, lx, ly);
        }
        at = diag_index(t, 0, T, U + 1);
    }
};

// Shape of the register-resident row: LPR lanes cooperate on one row, each holding NV 16-byte vectors.
// Chosen from the number of vectors in a row; returns false when the row does not fit (more than 512 vectors: the
// segment-wise long-row kernels take over).
struct RowShape {
    int lpr, nv;
};
__host__ inline bool pick_row_shape(int64_t nvec, RowShape *s)
{
    // short rows: few lanes per row, so that one warp instruction of the per-row bookkeeping serves 8 rows
    if (nvec <= 4) *s = {4, 1};
    else if (nvec <= 8) *s = {4, 2};
    else if (nvec <= 16) *s = {4, 4};
    else if (nvec <= 32) *s = {8, 4};
    else if (nvec <= 64) *s = {16, 4};
    else if (nvec <= 128) *s = {32, 4};
    else if (nvec <= 256) *s = {32, 8};
    else if (nvec <= 512) *s = {32, 16};
    else return false;
    return true;
}

// Expands `CALL(LPR, NV)` for the shape picked at run time.
#define CWRNNT_DISPATCH_SHAPE(shape, CALL)                      \
    do {                                                        \
        if ((shape).lpr == 4 && (shape).nv == 1) { CALL(4, 1); }        \
        else if ((shape).lpr == 4 && (shape).nv == 2) { CALL(4, 2); }   \
        else if ((shape).lpr == 4 && (shape).nv == 4) { CALL(4, 4); }   \
        else if ((shape).lpr == 8 && (shape).nv == 4) { CALL(8, 4); }   \
        else if ((shape).lpr == 16 && (shape).nv == 4) { CALL(16, 4); } \
        else if ((shape).lpr == 32 && (shape).nv == 4) { CALL(32, 4); } \
        else if ((shape).lpr == 32 && (shape).nv == 8) { CALL(32, 8); } \
        else { CALL(32, 16); }                                  \
    } while (0)

// Non-persistent grid for the streaming kernels: one tile of `rows_per_cta` consecutive rows per CTA. The hardware
// dispatches CTAs in order, so the CTAs in flight sweep the matrix as one compact front; a persistent grid-stride loop
// over the same tiles measured 15 % less bandwidth on B200.
__host__ inline unsigned tiled_grid(int64_t n_rows, int64_t rows_per_cta)
{
    const int64_t g = (n_rows + rows_per_cta - 1) / rows_per_cta;
    return unsigned(g < 1 ? 1 : (g > 0x7fffffff ? 0x7fffffff : g));
}

template <int LPR, typename A>
__device__ __forceinline__ A group_max(A v)
{
#pragma unroll
    for (int s = LPR / 2; s > 0; s >>= 1) {
        A o = __shfl_xor_sync(0xffffffffu, v, s);
        v = o > v ? o : v;
    }
    return v;
}
template <int LPR, typename A>
__device__ __forceinline__ A group_sum(A v)
{
#pragma unroll
    for (int s = LPR / 2; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
    return v;
}

}  // namespace cwrnnt
