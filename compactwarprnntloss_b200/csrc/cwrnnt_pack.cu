// Padded [B, Tmax, Umax+1, V] joint output  <->  compact [sum_n T_n*(U_n+1), V] rows.
//
// The reference accepts 4-D input and compacts it with the third-party gather.cat on the flattened [T*(U+1)] axis
// (cwarp_rnnt/__init__.py:52-59), which keeps the first T_n*(U_n+1) rows of each block and is therefore only right
// when every U_n equals Umax. These two kernels implement the layout the reference's own test defines
// (test/test.py:45-46): sequence n contributes x[n, :T_n, :U_n+1, :], rows in (t,u) order - and the transpose of that
// copy for the gradient, which also zero-fills the padding. Pure streaming copies, one warp per row, 128-bit when the
// row allows it.
#include "cwrnnt_kernels.h"
#include "cwrnnt_rowmap.cuh"

namespace cwrnnt {

template <typename Vec>
__device__ __forceinline__ void copy_row(const char *__restrict__ src, char *__restrict__ dst, int row_bytes, int lane)
{
    const Vec *s = reinterpret_cast<const Vec *>(src);
    Vec *d = reinterpret_cast<Vec *>(dst);
    for (int i = lane; i < row_bytes / int(sizeof(Vec)); i += 32) d[i] = __ldg(s + i);
}

// compact[r] = padded[n, t, u] for every compact row r = off[n] + t*(U_n+1) + u
template <typename Vec>
__global__ void __launch_bounds__(kStreamThreads)
pack_kernel(const char *__restrict__ padded, char *__restrict__ compact, int row_bytes, int64_t n_rows, int B,
            int t_max, int u_max1, const int32_t *__restrict__ lx, const int32_t *__restrict__ ly,
            const int64_t *__restrict__ off)
{
    if (off[B] != n_rows) return;  // lengths and row count disagree: leave the output untouched
    const int lane = threadIdx.x & 31;
    const int64_t n_warps = (int64_t(gridDim.x) * kStreamThreads) >> 5;
    const int64_t per_warp = (n_rows + n_warps - 1) / n_warps;
    const int64_t r_begin = ((int64_t(blockIdx.x) * kStreamThreads + threadIdx.x) >> 5) * per_warp;
    const int64_t r_end = r_begin + per_warp < n_rows ? r_begin + per_warp : n_rows;
    if (r_begin >= r_end) return;
    RowWalker rw;
    rw.start(r_begin, off, B, lx, ly);
    for (int64_t r = r_begin; r < r_end; ++r) {
        if (rw.t < t_max && rw.u < u_max1) {
            const int64_t pr = (int64_t(rw.n) * t_max + rw.t) * u_max1 + rw.u;
            copy_row<Vec>(padded + pr * row_bytes, compact + r * row_bytes, row_bytes, lane);
        }
        rw.advance(off, B, lx, ly);
    }
}

// padded[n, t, u] = compact[r] inside the lattice of sequence n, zero outside
template <typename Vec>
__global__ void __launch_bounds__(kStreamThreads)
unpack_kernel(const char *__restrict__ compact, char *__restrict__ padded, int row_bytes, int64_t n_rows, int B,
              int t_max, int u_max1, const int32_t *__restrict__ lx, const int32_t *__restrict__ ly,
              const int64_t *__restrict__ off)
{
    const bool consistent = off[B] == n_rows;
    const int lane = threadIdx.x & 31;
    const int64_t total = int64_t(B) * t_max * u_max1;
    const int64_t n_warps = (int64_t(gridDim.x) * kStreamThreads) >> 5;
    for (int64_t pr = (int64_t(blockIdx.x) * kStreamThreads + threadIdx.x) >> 5; pr < total; pr += n_warps) {
        const int u = int(pr % u_max1);
        const int64_t nt = pr / u_max1;
        const int t = int(nt % t_max), n = int(nt / t_max);
        const int T = lx[n], U = ly[n];
        char *dst = padded + pr * row_bytes;
        if (consistent && t < T && u <= U) {
            const int64_t r = off[n] + int64_t(t) * (U + 1) + u;
            copy_row<Vec>(compact + r * row_bytes, dst, row_bytes, lane);
        } else {
            Vec zero{};
            Vec *d = reinterpret_cast<Vec *>(dst);
            for (int i = lane; i < row_bytes / int(sizeof(Vec)); i += 32) d[i] = zero;
        }
    }
}

static size_t elt_bytes(int dtype) { return dtype == CWRNNT_F32 ? 4 : (dtype == CWRNNT_F64 ? 8 : 2); }

cudaError_t launch_pack(const cwrnnt_problem &p, bool to_compact, const void *src, void *dst, int32_t t_max,
                        int32_t u_max1, const int32_t *lx, const int32_t *ly, int64_t *off_scratch, cudaStream_t s)
{
    cudaError_t e = launch_offsets_only(lx, ly, p.B, p.max_u, off_scratch, s);
    if (e != cudaSuccess) return e;
    const int row_bytes = int(int64_t(p.V) * int64_t(elt_bytes(p.dtype)));
    const bool vec = row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(src) % 16 == 0 &&
                     reinterpret_cast<uintptr_t>(dst) % 16 == 0;
    // otherwise 2-byte units: every supported element type has an even size
    const int64_t rows = to_compact ? p.n_rows : int64_t(p.B) * t_max * u_max1;
    if (rows == 0) return cudaSuccess;
    const unsigned grid = tiled_grid(rows, 8 * 4);
    const char *cs = static_cast<const char *>(src);
    char *cd = static_cast<char *>(dst);
    if (to_compact) {
        if (vec)
            pack_kernel<uint4><<<grid, kStreamThreads, 0, s>>>(cs, cd, row_bytes, p.n_rows, p.B, t_max, u_max1, lx, ly,
                                                               off_scratch);
        else
            pack_kernel<unsigned short><<<grid, kStreamThreads, 0, s>>>(cs, cd, row_bytes, p.n_rows, p.B, t_max,
                                                                        u_max1, lx, ly, off_scratch);
    } else {
        if (vec)
            unpack_kernel<uint4><<<grid, kStreamThreads, 0, s>>>(cs, cd, row_bytes, p.n_rows, p.B, t_max, u_max1, lx,
                                                                 ly, off_scratch);
        else
            unpack_kernel<unsigned short><<<grid, kStreamThreads, 0, s>>>(cs, cd, row_bytes, p.n_rows, p.B, t_max,
                                                                          u_max1, lx, ly, off_scratch);
    }
    return cudaGetLastError();
}

}  // namespace cwrnnt
