// Row -> (sequence, frame, column) mapping and vector-shape dispatch shared by the two streaming kernels. Internal.
#pragma once
#include "cwrnnt_common.cuh"

namespace cwrnnt {

constexpr int kStreamThreads = 256;  // 8 warps per CTA in the streaming kernels

struct RowInfo {
    int n;        // sequence
    int T, U;     // its lengths
    int t, u;     // lattice cell of this row
    int64_t off;  // first row of the sequence
    int label;    // y[n][u] clamped into [0,V), or -1 when u == U
    bool bad_label;
};

__device__ __forceinline__ RowInfo locate_row(int64_t r, int &cursor, const int64_t *__restrict__ off, int B,
                                              const int32_t *__restrict__ lx, const int32_t *__restrict__ ly,
                                              const int32_t *__restrict__ y, int y_stride, int V)
{
    RowInfo ri;
    ri.n = cursor = find_sequence(off, B, r, cursor);
    ri.off = __ldg(off + ri.n);
    ri.T = __ldg(lx + ri.n);
    ri.U = __ldg(ly + ri.n);
    const unsigned rel = unsigned(r - ri.off);  // a sequence has fewer than 2^31 cells
    const unsigned m = unsigned(ri.U) + 1u;
    ri.t = int(rel / m);
    ri.u = int(rel - unsigned(ri.t) * m);
    ri.label = -1;
    ri.bad_label = false;
    if (ri.u < ri.U) {
        int k = __ldg(y + int64_t(ri.n) * y_stride + ri.u);
        if (k < 0 || k >= V) {
            ri.bad_label = true;
            k = k < 0 ? 0 : V - 1;
        }
        ri.label = k;
    }
    return ri;
}

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
