// Row -> (sequence, frame, column) bookkeeping and vector-shape dispatch shared by the two streaming kernels. Internal.
#pragma once
#include "cwrnnt_common.cuh"

namespace cwrnnt {

constexpr int kStreamThreads = 256;  // 8 warps per CTA in the streaming kernels

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
    // Same for a later row when the walker already stands on an earlier one: a short forward walk over the sequence
    // boundaries (rows visited with a fixed stride usually stay in the same sequence or move to the next), bisection
    // only after a long jump.
    __device__ __forceinline__ void restart(int64_t r, const int64_t *__restrict__ offs, int B,
                                            const int32_t *__restrict__ lx, const int32_t *__restrict__ ly)
    {
        int steps = 0;
        while (n + 1 < B && r >= __ldg(offs + n + 1)) {
            ++n;
            if (++steps == 4) {
                start(r, offs, B, lx, ly);
                return;
            }
        }
        if (steps) load_sequence(offs, lx, ly);
        const unsigned rel = unsigned(r - off);
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
// Chosen from the number of vectors in a row; returns false when the row does not fit (generic path).
struct RowShape {
    int lpr, nv;
};
__host__ inline bool pick_row_shape(int64_t nvec, RowShape *s)
{
    if (nvec <= 8) *s = {8, 1};
    else if (nvec <= 16) *s = {8, 2};
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
        if ((shape).lpr == 8 && (shape).nv == 1) { CALL(8, 1); }        \
        else if ((shape).lpr == 8 && (shape).nv == 2) { CALL(8, 2); }   \
        else if ((shape).lpr == 8 && (shape).nv == 4) { CALL(8, 4); }   \
        else if ((shape).lpr == 16 && (shape).nv == 4) { CALL(16, 4); } \
        else if ((shape).lpr == 32 && (shape).nv == 4) { CALL(32, 4); } \
        else if ((shape).lpr == 32 && (shape).nv == 8) { CALL(32, 8); } \
        else { CALL(32, 16); }                                  \
    } while (0)

// Persistent grid: as many CTAs as are resident at once (148 SMs x occupancy), so that the static, perfectly balanced
// split of rows over lane groups runs as a single wave.
template <typename K>
__host__ inline int resident_grid(K kernel, int threads)
{
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0) != cudaSuccess || per_sm < 1)
        per_sm = 4;
    return kNumSMs * per_sm;
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
