// The joint network's broadcast-add, written straight into the compact layout (the step in front of the loss):
//     h[off_n + t*(U_n+1) + u][:] = act(enc[n][t][:] + pred[n][u][:]),   act = identity | relu | tanh
// from the padded encoder output enc [B, t_max, H] and predictor output pred [B, u_max1, H]. The reference leaves this
// to the caller, who builds the padded [N, T, U+1, H] tensor and compacts it (test/test.py:34-48 shows that layout;
// cwarp_rnnt/__init__.py:52-59 compacts a padded 4-D input). Producing the compact rows directly never materialises
// the padding: on the ragged workload the padded tensor is 20 times the compact one.
//
// Forward: one warp per run of rows; enc/pred rows are re-read from L2 (each is used U+1 / T times); the output is
// written once with 128-bit stores. Bound: HBM write, H * sizeof(element) bytes per lattice node.
// Backward: grad_enc[n][t] = sum_u g * act', grad_pred[n][u] = sum_t g * act' - two reductions over the same
// [n_rows, H] gradient, one warp per (n, t, 32-vector chunk) and per (n, u, chunk). Fixed summation order
// (deterministic, no atomics); act' is recomputed from enc + pred, so the forward output is not read. The padding of
// grad_enc / grad_pred is zero-filled by the same kernels. Bound: HBM read, 2 * H * sizeof(element) per node.
#include "cwrnnt_kernels.h"
#include "cwrnnt_rowmap.cuh"

namespace cwrnnt {

enum { kActNone = CWRNNT_ACT_NONE, kActRelu = CWRNNT_ACT_RELU, kActTanh = CWRNNT_ACT_TANH };

// tanh in the arithmetic the storage type deserves: 16-bit rows (8 or 11 significant bits) take the hardware
// approximation (one MUFU instruction, relative error about 2^-11), float rows tanhf, double rows tanh.
template <bool FAST>
__device__ __forceinline__ float tanh_of(float s)
{
    if (FAST) {
        float y;
        asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(s));
        return y;
    }
    return tanhf(s);
}
template <bool FAST>
__device__ __forceinline__ double tanh_of(double s)
{
    return tanh(s);
}

template <int ACT, bool FAST, typename A>
__device__ __forceinline__ A activate(A s)
{
    if (ACT == kActRelu) return s > A(0) ? s : A(0);
    if (ACT == kActTanh) return tanh_of<FAST>(s);
    return s;
}
// d act(s) / d s
template <int ACT, bool FAST, typename A>
__device__ __forceinline__ A activate_slope(A s)
{
    if (ACT == kActRelu) return s > A(0) ? A(1) : A(0);
    if (ACT == kActTanh) {
        const A h = tanh_of<FAST>(s);
        return A(1) - h * h;
    }
    return A(1);
}

// VEC: rows are whole 16-byte vectors and all bases are 16-byte aligned; otherwise element by element.
template <typename T, int ACT, bool VEC>
__global__ void __launch_bounds__(kStreamThreads)
joint_rows_kernel(const T *__restrict__ enc, const T *__restrict__ pred, T *__restrict__ out, int H, int64_t n_rows,
                  int B, int t_max, int u_max1, const int32_t *__restrict__ lx, const int32_t *__restrict__ ly,
                  const int64_t *__restrict__ off, int run_len)
{
    using E = Elt<T>;
    using A = typename E::acc;
    constexpr int VE = E::VE;
    if (off[B] != n_rows) return;  // lengths and row count disagree: leave the output untouched
    const int lane = threadIdx.x & 31;
    const int64_t first = ((int64_t(blockIdx.x) * kStreamThreads + threadIdx.x) >> 5) * run_len;
    const int64_t limit = first + run_len < n_rows ? first + run_len : n_rows;
    RowWalker rw;
    for (int64_t r = first; r < limit; ++r) {
        if (r == first) rw.start(r, off, B, lx, ly);
        if (rw.t < t_max && rw.u < u_max1) {
            const T *e = enc + (int64_t(rw.n) * t_max + rw.t) * H;
            const T *q = pred + (int64_t(rw.n) * u_max1 + rw.u) * H;
            T *o = out + r * int64_t(H);
            if (VEC) {
                const uint4 *ev = reinterpret_cast<const uint4 *>(e), *qv = reinterpret_cast<const uint4 *>(q);
                uint4 *ov = reinterpret_cast<uint4 *>(o);
                for (int i = lane; i < H / VE; i += 32) {
                    A a[VE], b[VE];
                    E::unpack(__ldg(ev + i), a);
                    E::unpack(__ldg(qv + i), b);
#pragma unroll
                    for (int c = 0; c < VE; ++c) a[c] = activate<ACT, sizeof(T) == 2>(a[c] + b[c]);
                    ov[i] = E::pack(a);
                }
            } else {
                for (int i = lane; i < H; i += 32) {
                    const A sum = E::to_acc(__ldg(e + i)) + E::to_acc(__ldg(q + i));
                    o[i] = E::from_acc(activate<ACT, sizeof(T) == 2>(sum));
                }
            }
        }
        rw.advance(off, B, lx, ly);
    }
}

// One warp per (n, fixed index, chunk of 32 vectors or 32 elements): the sum over the other lattice axis.
// OVER_U: fixed t, sum over u = 0..U (consecutive rows) -> grad_enc[n][t]; else fixed u, sum over t -> grad_pred[n][u].
template <typename T, int ACT, bool VEC, bool OVER_U>
__global__ void __launch_bounds__(kStreamThreads)
joint_reduce_kernel(const T *__restrict__ enc, const T *__restrict__ pred, const T *__restrict__ g,
                    T *__restrict__ dst, int H, int64_t n_rows, int B, int t_max, int u_max1,
                    const int32_t *__restrict__ lx, const int32_t *__restrict__ ly, const int64_t *__restrict__ off,
                    int n_chunks)
{
    using E = Elt<T>;
    using A = typename E::acc;
    constexpr int VE = VEC ? E::VE : 1;
    const bool consistent = off[B] == n_rows;
    const int lane = threadIdx.x & 31;
    const int fixed_max = OVER_U ? t_max : u_max1;
    const int64_t total = int64_t(B) * fixed_max * n_chunks;
    const int64_t n_warps = (int64_t(gridDim.x) * kStreamThreads) >> 5;
    const int width = VEC ? H / E::VE : H;  // units (vectors or elements) per row
    for (int64_t item = (int64_t(blockIdx.x) * kStreamThreads + threadIdx.x) >> 5; item < total; item += n_warps) {
        const int chunk = int(item % n_chunks);
        const int64_t nf = item / n_chunks;
        const int fixed = int(nf % fixed_max), n = int(nf / fixed_max);
        const int idx = chunk * 32 + lane;  // this lane's unit inside the row
        if (idx >= width) continue;
        const int T_n = lx[n], U_n = ly[n];
        A acc[VE];
#pragma unroll
        for (int c = 0; c < VE; ++c) acc[c] = A(0);
        const bool inside = consistent && (OVER_U ? fixed < T_n : fixed <= U_n);
        if (inside) {
            const int64_t base = off[n];
            const int m = U_n + 1;
            const int count = OVER_U ? min(m, u_max1) : min(T_n, t_max);
            A fix[VE];  // the operand that does not change along the sum
            {
                const T *row = OVER_U ? enc + (int64_t(n) * t_max + fixed) * H
                                      : pred + (int64_t(n) * u_max1 + fixed) * H;
                if (VEC) {
                    A tmp[E::VE];
                    E::unpack(__ldg(reinterpret_cast<const uint4 *>(row) + idx), tmp);
#pragma unroll
                    for (int c = 0; c < VE; ++c) fix[c] = tmp[c];
                } else {
                    fix[0] = E::to_acc(__ldg(row + idx));
                }
            }
            for (int k = 0; k < count; ++k) {
                const int t = OVER_U ? fixed : k, u = OVER_U ? k : fixed;
                const int64_t r = base + int64_t(t) * m + u;
                const T *other = OVER_U ? pred + (int64_t(n) * u_max1 + u) * H : enc + (int64_t(n) * t_max + t) * H;
                if (VEC) {
                    A gv[E::VE], ov[E::VE];
                    E::unpack(__ldg(reinterpret_cast<const uint4 *>(g + r * int64_t(H)) + idx), gv);
                    E::unpack(__ldg(reinterpret_cast<const uint4 *>(other) + idx), ov);
#pragma unroll
                    for (int c = 0; c < VE; ++c) acc[c] += gv[c] * activate_slope<ACT, sizeof(T) == 2>(fix[c] + ov[c]);
                } else {
                    acc[0] += E::to_acc(__ldg(g + r * int64_t(H) + idx)) *
                              activate_slope<ACT, sizeof(T) == 2>(fix[0] + E::to_acc(__ldg(other + idx)));
                }
            }
        }
        T *d = dst + (int64_t(n) * fixed_max + fixed) * H;
        if (VEC) {
            A outv[E::VE];
#pragma unroll
            for (int c = 0; c < VE; ++c) outv[c] = acc[c];
            reinterpret_cast<uint4 *>(d)[idx] = E::pack(outv);
        } else {
            d[idx] = E::from_acc(acc[0]);
        }
    }
}

template <typename T, int ACT, bool VEC>
static cudaError_t launch_joint_t(const cwrnnt_problem &p, bool backward, const T *enc, int t_max, const T *pred,
                                  int u_max1, const int32_t *lx, const int32_t *ly, const int64_t *off,
                                  const T *grad_out, T *out_or_genc, T *gpred, cudaStream_t s)
{
    const int H = p.V;
    if (!backward) {
        if (p.n_rows == 0) return cudaSuccess;
        const int run_len = 8;
        const unsigned grid = tiled_grid(p.n_rows, int64_t(kStreamThreads / 32) * run_len);
        joint_rows_kernel<T, ACT, VEC><<<grid, kStreamThreads, 0, s>>>(enc, pred, out_or_genc, H, p.n_rows, p.B, t_max,
                                                                       u_max1, lx, ly, off, run_len);
        return cudaGetLastError();
    }
    const int width = VEC ? H / Elt<T>::VE : H;
    const int n_chunks = (width + 31) / 32;
    const int64_t items_enc = int64_t(p.B) * t_max * n_chunks, items_pred = int64_t(p.B) * u_max1 * n_chunks;
    auto grid_for = [](int64_t warps) {
        const int64_t ctas = (warps + kStreamThreads / 32 - 1) / (kStreamThreads / 32);
        return unsigned(ctas < 1 ? 1 : (ctas > kNumSMs * 64 ? kNumSMs * 64 : ctas));
    };
    if (items_enc > 0)
        joint_reduce_kernel<T, ACT, VEC, true><<<grid_for(items_enc), kStreamThreads, 0, s>>>(
            enc, pred, grad_out, out_or_genc, H, p.n_rows, p.B, t_max, u_max1, lx, ly, off, n_chunks);
    if (items_pred > 0)
        joint_reduce_kernel<T, ACT, VEC, false><<<grid_for(items_pred), kStreamThreads, 0, s>>>(
            enc, pred, grad_out, gpred, H, p.n_rows, p.B, t_max, u_max1, lx, ly, off, n_chunks);
    return cudaGetLastError();
}

template <typename T>
static cudaError_t launch_joint_act(const cwrnnt_problem &p, int activation, bool backward, const void *enc, int t_max,
                                    const void *pred, int u_max1, const int32_t *lx, const int32_t *ly,
                                    const int64_t *off, const void *grad_out, void *a, void *b, cudaStream_t s)
{
    const T *e = static_cast<const T *>(enc), *q = static_cast<const T *>(pred), *g = static_cast<const T *>(grad_out);
    T *pa = static_cast<T *>(a), *pb = static_cast<T *>(b);
    auto aligned = [](const void *ptr) { return reinterpret_cast<uintptr_t>(ptr) % 16 == 0; };
    const bool vec = p.V % Elt<T>::VE == 0 && aligned(enc) && aligned(pred) && aligned(a) &&
                     (!backward || (aligned(b) && aligned(grad_out)));
#define CWRNNT_JOINT(ACT)                                                                                         \
    return vec ? launch_joint_t<T, ACT, true>(p, backward, e, t_max, q, u_max1, lx, ly, off, g, pa, pb, s)         \
               : launch_joint_t<T, ACT, false>(p, backward, e, t_max, q, u_max1, lx, ly, off, g, pa, pb, s)
    if (activation == kActRelu) CWRNNT_JOINT(kActRelu);
    if (activation == kActTanh) CWRNNT_JOINT(kActTanh);
    CWRNNT_JOINT(kActNone);
#undef CWRNNT_JOINT
}

cudaError_t launch_joint(const cwrnnt_problem &p, int activation, bool backward, const void *enc, int32_t t_max,
                         const void *pred, int32_t u_max1, const int32_t *lx, const int32_t *ly, int64_t *off_scratch,
                         const void *grad_out, void *out_or_grad_enc, void *grad_pred, cudaStream_t s)
{
    cudaError_t e = launch_offsets_only(lx, ly, p.B, p.max_u, off_scratch, s);
    if (e != cudaSuccess) return e;
    switch (p.dtype) {
    case CWRNNT_F32:
        return launch_joint_act<float>(p, activation, backward, enc, t_max, pred, u_max1, lx, ly, off_scratch,
                                       grad_out, out_or_grad_enc, grad_pred, s);
    case CWRNNT_F16:
        return launch_joint_act<__half>(p, activation, backward, enc, t_max, pred, u_max1, lx, ly, off_scratch,
                                        grad_out, out_or_grad_enc, grad_pred, s);
    case CWRNNT_BF16:
        return launch_joint_act<__nv_bfloat16>(p, activation, backward, enc, t_max, pred, u_max1, lx, ly, off_scratch,
                                               grad_out, out_or_grad_enc, grad_pred, s);
    case CWRNNT_F64:
        return launch_joint_act<double>(p, activation, backward, enc, t_max, pred, u_max1, lx, ly, off_scratch,
                                        grad_out, out_or_grad_enc, grad_pred, s);
    }
    return cudaErrorInvalidValue;
}

}  // namespace cwrnnt
