// Host-buffer pipeline: logits in host memory -> costs / loss / gradients in host memory.
//
// The batch is cut into chunks of whole sequences (a lattice is never split: the recursion needs all of it). Three
// streams form a software pipeline over a ring of device slots:
//     upload(c+1)  ||  prep+gather+wavefront+grad(c)  ||  download(c-1)
// so that with pinned host buffers both PCIe directions and the SMs are busy at once and the device never holds more
// than kSlots chunks. Events order the stages; nothing spins on the device.
#include <cstdio>
#include <cstring>
#include <vector>

#include "cwrnnt_kernels.h"

using namespace cwrnnt;

namespace {
constexpr int kSlots = 3;

size_t elt_size(int dtype) { return dtype == CWRNNT_F32 ? 4 : (dtype == CWRNNT_F64 ? 8 : 2); }
size_t cost_size(int dtype) { return dtype == CWRNNT_F64 ? 8 : 4; }

struct Slot {
    void *x = nullptr, *g = nullptr, *ws = nullptr;
    cudaEvent_t free_ev = nullptr;  // all work that used this slot has finished
};
}  // namespace

struct cwrnnt_host_ctx {
    int device = 0;
    cudaStream_t s_up = nullptr, s_run = nullptr, s_down = nullptr;
    Slot slot[kSlots];
    int64_t cap_chunk_bytes = 0, cap_ws_bytes = 0;
    bool cap_grad = false;
    int32_t *lens = nullptr;  // lx | ly | y on the device
    int64_t cap_lens = 0;
    void *costs = nullptr, *gc = nullptr;
    int64_t cap_costs = 0;
    int32_t *status_h = nullptr;  // pinned, 4 words per chunk
    int64_t cap_status = 0;
    std::vector<cudaEvent_t> up_ev, run_ev;
    char err[256] = "";
};

#define CK(call)                                                                                   \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) {                                                                   \
            std::snprintf(ctx->err, sizeof ctx->err, "%s: %s", #call, cudaGetErrorString(e_));     \
            return CWRNNT_ERR_LAUNCH;                                                              \
        }                                                                                          \
    } while (0)

// Waits for everything queued on the context's streams; the results are ignored (the caller is already failing).
static void drain(cwrnnt_host_ctx *ctx)
{
    cudaStreamSynchronize(ctx->s_up);
    cudaStreamSynchronize(ctx->s_run);
    cudaStreamSynchronize(ctx->s_down);
}

#define CKD(call)                                                                                  \
    do {                                                                                           \
        cudaError_t e_ = (call);                                                                   \
        if (e_ != cudaSuccess) {                                                                   \
            std::snprintf(ctx->err, sizeof ctx->err, "%s: %s", #call, cudaGetErrorString(e_));     \
            drain(ctx);                                                                            \
            return CWRNNT_ERR_LAUNCH;                                                              \
        }                                                                                          \
    } while (0)

extern "C" {

int cwrnnt_host_ctx_create(cwrnnt_host_ctx **out)
{
    if (!out) return CWRNNT_ERR_ARGUMENT;
    cwrnnt_host_ctx *ctx = new cwrnnt_host_ctx();
    *out = ctx;
    CK(cudaGetDevice(&ctx->device));
    CK(cudaStreamCreateWithFlags(&ctx->s_up, cudaStreamNonBlocking));
    CK(cudaStreamCreateWithFlags(&ctx->s_run, cudaStreamNonBlocking));
    CK(cudaStreamCreateWithFlags(&ctx->s_down, cudaStreamNonBlocking));
    for (auto &s : ctx->slot) CK(cudaEventCreateWithFlags(&s.free_ev, cudaEventDisableTiming));
    return CWRNNT_OK;
}

void cwrnnt_host_ctx_destroy(cwrnnt_host_ctx *ctx)
{
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    cudaDeviceSynchronize();
    for (auto &s : ctx->slot) {
        cudaFree(s.x);
        cudaFree(s.g);
        cudaFree(s.ws);
        if (s.free_ev) cudaEventDestroy(s.free_ev);
    }
    cudaFree(ctx->lens);
    cudaFree(ctx->costs);
    cudaFree(ctx->gc);
    if (ctx->status_h) cudaFreeHost(ctx->status_h);
    for (auto e : ctx->up_ev) cudaEventDestroy(e);
    for (auto e : ctx->run_ev) cudaEventDestroy(e);
    if (ctx->s_up) cudaStreamDestroy(ctx->s_up);
    if (ctx->s_run) cudaStreamDestroy(ctx->s_run);
    if (ctx->s_down) cudaStreamDestroy(ctx->s_down);
    delete ctx;
}

const char *cwrnnt_host_ctx_error(const cwrnnt_host_ctx *ctx) { return ctx ? ctx->err : ""; }

int cwrnnt_loss_grad_host(cwrnnt_host_ctx *ctx, const cwrnnt_problem *p, const void *x_host, const int32_t *lx_host,
                          const int32_t *ly_host, const int32_t *y_host, const void *grad_costs_host,
                          int32_t grad_costs_stride, void *costs_host, void *loss_host, void *grad_x_host,
                          int64_t chunk_rows, int32_t status_out[4])
{
    if (!ctx || !p || !lx_host || !ly_host || !costs_host) return CWRNNT_ERR_ARGUMENT;
    if (cwrnnt_workspace_bytes(p) < 0) return CWRNNT_ERR_ARGUMENT;
    if ((p->n_rows > 0 && !x_host) || (p->max_u > 0 && !y_host)) return CWRNNT_ERR_ARGUMENT;
    if (grad_costs_stride != 0 && grad_costs_stride != 1) return CWRNNT_ERR_ARGUMENT;
    const bool want_grad = grad_x_host != nullptr && !(p->flags & CWRNNT_COSTS_ONLY);
    const int B = p->B;
    const size_t es = elt_size(p->dtype), cs = cost_size(p->dtype);
    const int64_t row_bytes = int64_t(p->V) * int64_t(es);
    if (status_out) status_out[0] = status_out[2] = status_out[3] = 0, status_out[1] = -1;
    if (B == 0) return CWRNNT_OK;
    CK(cudaSetDevice(ctx->device));

    // ---- host-side validation and chunk plan (lengths are host data here, so this costs nothing)
    int64_t total = 0;
    for (int n = 0; n < B; ++n) {
        if (lx_host[n] < 1 || ly_host[n] < 0 || ly_host[n] > p->max_u) {
            if (status_out) status_out[0] = CWRNNT_ST_BAD_LENGTH, status_out[1] = n;
            return CWRNNT_ERR_ARGUMENT;
        }
        total += int64_t(lx_host[n]) * (int64_t(ly_host[n]) + 1);
    }
    if (total != p->n_rows) {
        if (status_out) status_out[0] = CWRNNT_ST_ROW_MISMATCH;
        return CWRNNT_ERR_ARGUMENT;
    }
    if (chunk_rows <= 0) chunk_rows = (int64_t(48) << 20) / row_bytes + 1;  // ~48 MB of logits per chunk
    struct Chunk {
        int seq0, nseq;
        int64_t row0, rows;
    };
    std::vector<Chunk> chunks;
    {
        int64_t row = 0;
        int n = 0;
        while (n < B) {
            Chunk c{n, 0, row, 0};
            while (n < B) {
                int64_t r = int64_t(lx_host[n]) * (int64_t(ly_host[n]) + 1);
                if (c.nseq > 0 && c.rows + r > chunk_rows) break;
                c.rows += r;
                ++c.nseq;
                ++n;
            }
            row += c.rows;
            chunks.push_back(c);
        }
    }
    int64_t max_rows = 0;
    int max_seq = 0;
    for (auto &c : chunks) {
        max_rows = c.rows > max_rows ? c.rows : max_rows;
        max_seq = c.nseq > max_seq ? c.nseq : max_seq;
    }

    // ---- capacity
    const int64_t need_chunk = max_rows * row_bytes;
    const int64_t need_ws = carve_workspace(max_rows, max_seq, nullptr, nullptr);
    if (need_chunk > ctx->cap_chunk_bytes || need_ws > ctx->cap_ws_bytes || (want_grad && !ctx->cap_grad)) {
        CK(cudaDeviceSynchronize());
        for (auto &s : ctx->slot) {
            cudaFree(s.x);
            cudaFree(s.g);
            cudaFree(s.ws);
            s.x = s.g = s.ws = nullptr;
        }
        ctx->cap_chunk_bytes = need_chunk > ctx->cap_chunk_bytes ? need_chunk : ctx->cap_chunk_bytes;
        ctx->cap_ws_bytes = need_ws > ctx->cap_ws_bytes ? need_ws : ctx->cap_ws_bytes;
        ctx->cap_grad = ctx->cap_grad || want_grad;
        for (auto &s : ctx->slot) {
            CK(cudaMalloc(&s.x, size_t(ctx->cap_chunk_bytes)));
            if (ctx->cap_grad) CK(cudaMalloc(&s.g, size_t(ctx->cap_chunk_bytes)));
            CK(cudaMalloc(&s.ws, size_t(ctx->cap_ws_bytes)));
        }
    }
    const int64_t need_lens = (2 * int64_t(B) + int64_t(B) * p->y_stride) * 4;
    if (need_lens > ctx->cap_lens) {
        CK(cudaDeviceSynchronize());
        cudaFree(ctx->lens);
        CK(cudaMalloc(reinterpret_cast<void **>(&ctx->lens), size_t(need_lens)));
        ctx->cap_lens = need_lens;
    }
    if (int64_t(B) * 8 > ctx->cap_costs) {
        CK(cudaDeviceSynchronize());
        cudaFree(ctx->costs);
        cudaFree(ctx->gc);
        CK(cudaMalloc(&ctx->costs, size_t(B) * 8));
        CK(cudaMalloc(&ctx->gc, size_t(B) * 8));
        ctx->cap_costs = int64_t(B) * 8;
    }
    if (int64_t(chunks.size()) > ctx->cap_status) {
        CK(cudaDeviceSynchronize());
        if (ctx->status_h) cudaFreeHost(ctx->status_h);
        CK(cudaMallocHost(reinterpret_cast<void **>(&ctx->status_h), chunks.size() * 16));
        ctx->cap_status = int64_t(chunks.size());
    }
    while (ctx->up_ev.size() < chunks.size()) {
        cudaEvent_t a, b;
        CK(cudaEventCreateWithFlags(&a, cudaEventDisableTiming));
        CK(cudaEventCreateWithFlags(&b, cudaEventDisableTiming));
        ctx->up_ev.push_back(a);
        ctx->run_ev.push_back(b);
    }

    // ---- small inputs first, on the upload stream. From here on copies from and into the caller's host buffers are in
    // flight: a failure drains the three streams before returning (CKD), so that the caller may free or reuse those
    // buffers and the context's slots are idle for the next call.
    int32_t *d_lx = ctx->lens, *d_ly = ctx->lens + B, *d_y = ctx->lens + 2 * int64_t(B);
    CKD(cudaMemcpyAsync(d_lx, lx_host, size_t(B) * 4, cudaMemcpyHostToDevice, ctx->s_up));
    CKD(cudaMemcpyAsync(d_ly, ly_host, size_t(B) * 4, cudaMemcpyHostToDevice, ctx->s_up));
    if (p->y_stride > 0)
        CKD(cudaMemcpyAsync(d_y, y_host, size_t(B) * p->y_stride * 4, cudaMemcpyHostToDevice, ctx->s_up));
    if (grad_costs_host)
        CKD(cudaMemcpyAsync(ctx->gc, grad_costs_host, (grad_costs_stride ? size_t(B) : 1) * cs, cudaMemcpyHostToDevice,
                           ctx->s_up));

    // ---- the pipeline
    const char *xh = static_cast<const char *>(x_host);
    char *gh = static_cast<char *>(grad_x_host);
    for (size_t c = 0; c < chunks.size(); ++c) {
        const Chunk &ch = chunks[c];
        Slot &sl = ctx->slot[c % kSlots];
        if (c >= size_t(kSlots)) CKD(cudaStreamWaitEvent(ctx->s_up, sl.free_ev, 0));
        CKD(cudaMemcpyAsync(sl.x, xh + ch.row0 * row_bytes, size_t(ch.rows * row_bytes), cudaMemcpyHostToDevice,
                           ctx->s_up));
        CKD(cudaEventRecord(ctx->up_ev[c], ctx->s_up));

        cwrnnt_problem sub = *p;
        sub.n_rows = ch.rows;
        sub.B = ch.nseq;
        sub.mean_denominator = p->mean_denominator > 0 ? p->mean_denominator : B;
        char *costs_c = static_cast<char *>(ctx->costs) + size_t(ch.seq0) * cs;
        const char *gc_c = grad_costs_host
                               ? static_cast<const char *>(ctx->gc) + (grad_costs_stride ? size_t(ch.seq0) * cs : 0)
                               : nullptr;
        CKD(cudaStreamWaitEvent(ctx->s_run, ctx->up_ev[c], 0));
        int st = cwrnnt_forward(&sub, sl.x, d_lx + ch.seq0, d_ly + ch.seq0, d_y + int64_t(ch.seq0) * p->y_stride,
                                sl.ws, ctx->cap_ws_bytes, costs_c, nullptr,
                                reinterpret_cast<cwrnnt_stream_t>(ctx->s_run));
        if (st) {
            drain(ctx);
            return st;
        }
        if (want_grad) {
            st = cwrnnt_backward(&sub, sl.x, d_lx + ch.seq0, d_ly + ch.seq0, d_y + int64_t(ch.seq0) * p->y_stride,
                                 sl.ws, gc_c, grad_costs_stride, sl.g, reinterpret_cast<cwrnnt_stream_t>(ctx->s_run));
            if (st) {
            drain(ctx);
            return st;
        }
        }
        CKD(cudaMemcpyAsync(ctx->status_h + 4 * c, sl.ws, 16, cudaMemcpyDeviceToHost, ctx->s_run));
        CKD(cudaEventRecord(ctx->run_ev[c], ctx->s_run));

        CKD(cudaStreamWaitEvent(ctx->s_down, ctx->run_ev[c], 0));
        if (want_grad)
            CKD(cudaMemcpyAsync(gh + ch.row0 * row_bytes, sl.g, size_t(ch.rows * row_bytes), cudaMemcpyDeviceToHost,
                               ctx->s_down));
        CKD(cudaEventRecord(sl.free_ev, ctx->s_down));
    }
    CKD(cudaStreamWaitEvent(ctx->s_down, ctx->run_ev[chunks.size() - 1], 0));
    CKD(cudaMemcpyAsync(costs_host, ctx->costs, size_t(B) * cs, cudaMemcpyDeviceToHost, ctx->s_down));
    CKD(cudaStreamSynchronize(ctx->s_down));
    CKD(cudaStreamSynchronize(ctx->s_run));
    CKD(cudaStreamSynchronize(ctx->s_up));

    // ---- status and reduction on the host (B numbers)
    if (status_out) {
        for (size_t c = 0; c < chunks.size(); ++c) {
            const int32_t *s = ctx->status_h + 4 * c;
            status_out[0] |= s[0];
            if (s[1] >= 0 && status_out[1] < 0) status_out[1] = chunks[c].seq0 + s[1];
        }
        status_out[2] = int32_t(total & 0x7fffffff);
    }
    if (loss_host && (p->flags & (CWRNNT_REDUCE_MEAN | CWRNNT_REDUCE_SUM))) {
        double tot = 0.0;
        for (int n = 0; n < B; ++n)
            tot += cs == 8 ? static_cast<const double *>(costs_host)[n] : double(static_cast<const float *>(costs_host)[n]);
        if (p->flags & CWRNNT_REDUCE_MEAN) tot /= double(p->mean_denominator > 0 ? p->mean_denominator : B);
        if (cs == 8)
            *static_cast<double *>(loss_host) = tot;
        else
            *static_cast<float *>(loss_host) = float(tot);
    }
    return CWRNNT_OK;
}

}  // extern "C"
