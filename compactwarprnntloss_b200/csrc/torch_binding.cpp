// Thin torch extension over the C ABI (include/cwarp_rnnt_b200.h): the replacement of the reference's cwarp_cuda.cpp.
// It owns tensors, the device guard and the current stream; all arithmetic lives in libcwarp_rnnt_b200.so.
//
// Exports the reference module's three functions with the reference's argument order and result shapes
// (cwarp_cuda.cpp:138-153) for callers of `cwarp_rnnt._C`, plus the fused entry points the autograd function uses.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <string>
#include <tuple>
#include <vector>

#include "cwarp_rnnt_b200.h"

namespace {

// Same wording as the reference's checks (cwarp_cuda.cpp:46-52).
#define CHECK_CUDA(x) TORCH_CHECK(x.device().is_cuda(), #x " must be a CUDA tensor")
#define CHECK_CONTIGUOUS(x) TORCH_CHECK(x.is_contiguous(), #x " must be contiguous")
#define CHECK_TYPE(x, T) TORCH_CHECK(x.scalar_type() == T, #x " must be " #T)
#define CHECK_INPUT(x, T) \
    CHECK_CUDA(x);        \
    CHECK_CONTIGUOUS(x);  \
    CHECK_TYPE(x, T)

int dtype_code(const torch::Tensor &x)
{
    switch (x.scalar_type()) {
    case torch::ScalarType::Float: return CWRNNT_F32;
    case torch::ScalarType::Half: return CWRNNT_F16;
    case torch::ScalarType::BFloat16: return CWRNNT_BF16;
    case torch::ScalarType::Double: return CWRNNT_F64;
    default: TORCH_CHECK(false, "xs must be float32, float16, bfloat16 or float64, got ", x.scalar_type());
    }
    return -1;
}

torch::ScalarType cost_type(const torch::Tensor &x)
{
    return x.scalar_type() == torch::ScalarType::Double ? torch::ScalarType::Double : torch::ScalarType::Float;
}

void check_status(int st, const char *what)
{
    if (st == CWRNNT_OK) return;
    std::string msg = std::string(what) + ": " + cwrnnt_status_string(st);
    if (st == CWRNNT_ERR_LAUNCH) msg += std::string(" (") + cwrnnt_last_error() + ")";
    TORCH_CHECK(false, msg);
}

cwrnnt_problem describe(const torch::Tensor &xs, const torch::Tensor &lx, const torch::Tensor &ys, int64_t blank,
                        int64_t flags, int64_t mean_denominator)
{
    TORCH_CHECK(xs.dim() == 2, "xs must be 2-D [sum_i T_i*(U_i+1), V]");
    TORCH_CHECK(ys.dim() == 2 && ys.size(0) == lx.size(0), "ys must be [N, Umax]");
    cwrnnt_problem p{};
    p.n_rows = xs.size(0);
    p.V = static_cast<int32_t>(xs.size(1));
    p.B = static_cast<int32_t>(lx.size(0));
    p.y_stride = static_cast<int32_t>(ys.size(1));
    p.max_u = static_cast<int32_t>(ys.size(1));
    p.blank = static_cast<int32_t>(blank);
    p.dtype = dtype_code(xs);
    p.flags = static_cast<int32_t>(flags);
    p.mean_denominator = static_cast<int32_t>(mean_denominator);
    return p;
}

void check_inputs(const torch::Tensor &xs, const torch::Tensor &lx, const torch::Tensor &ys, const torch::Tensor &ly)
{
    CHECK_CONTIGUOUS(xs);
    CHECK_CUDA(xs);
    CHECK_INPUT(lx, torch::ScalarType::Int);
    CHECK_INPUT(ys, torch::ScalarType::Int);
    CHECK_INPUT(ly, torch::ScalarType::Int);
    TORCH_CHECK(lx.device() == xs.device() && ly.device() == xs.device() && ys.device() == xs.device(),
                "xs, lx, ys, ly must live on the same device");
    TORCH_CHECK(lx.dim() == 1 && ly.dim() == 1 && lx.size(0) == ly.size(0), "lx and ly must be [N]");
}

torch::Tensor make_workspace(const cwrnnt_problem &p, const torch::Tensor &like)
{
    const int64_t bytes = cwrnnt_workspace_bytes(&p);
    TORCH_CHECK(bytes >= 0, "invalid problem: check blank in [0,V), label length <= ", CWRNNT_MAX_COLUMNS - 1);
    return torch::empty({bytes}, like.options().dtype(torch::kUInt8));
}

cwrnnt_stream_t current_stream()
{
    return reinterpret_cast<cwrnnt_stream_t>(at::cuda::getCurrentCUDAStream().stream());
}

const int32_t *i32(const torch::Tensor &t) { return t.numel() ? t.data_ptr<int32_t>() : nullptr; }

// ---------------------------------------------------------------------------------------------- fused entry points

// Forward. Returns (costs [N], loss [] (zero unless a reduce flag is set), workspace bytes).
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> rnnt_forward(const torch::Tensor &xs, const torch::Tensor &lx,
                                                                     const torch::Tensor &ys, const torch::Tensor &ly,
                                                                     int64_t blank, int64_t flags,
                                                                     int64_t mean_denominator)
{
    check_inputs(xs, lx, ys, ly);
    const c10::cuda::CUDAGuard guard(xs.device());
    cwrnnt_problem p = describe(xs, lx, ys, blank, flags, mean_denominator);
    auto ws = make_workspace(p, xs);
    auto costs = torch::empty({lx.size(0)}, xs.options().dtype(cost_type(xs)));
    // written by the kernels whenever a reduction is asked for on a non-empty batch (NaN on invalid lengths)
    auto loss = ((flags & (CWRNNT_REDUCE_MEAN | CWRNNT_REDUCE_SUM)) && lx.size(0) > 0) ? torch::empty({}, costs.options())
                                                                   : torch::zeros({}, costs.options());
    check_status(cwrnnt_forward(&p, xs.data_ptr(), i32(lx), i32(ly), i32(ys), ws.data_ptr(), ws.numel(),
                                costs.data_ptr(), loss.data_ptr(), current_stream()),
                 "cwrnnt_forward");
    return {costs, loss, ws};
}

// Backward. grad_costs: [] or [1] (gradient of the reduced loss) or [N] (per-sequence), costs dtype.
torch::Tensor rnnt_backward(const torch::Tensor &xs, const torch::Tensor &lx, const torch::Tensor &ys,
                            const torch::Tensor &ly, int64_t blank, int64_t flags, int64_t mean_denominator,
                            const torch::Tensor &workspace, const torch::Tensor &grad_costs)
{
    check_inputs(xs, lx, ys, ly);
    CHECK_CUDA(grad_costs);
    const c10::cuda::CUDAGuard guard(xs.device());
    cwrnnt_problem p = describe(xs, lx, ys, blank, flags, mean_denominator);
    auto gc = grad_costs.to(cost_type(xs)).contiguous();
    TORCH_CHECK(gc.numel() == 1 || gc.numel() == lx.size(0), "grad_costs must have 1 or N elements");
    auto gx = torch::empty_like(xs);
    check_status(cwrnnt_backward(&p, xs.data_ptr(), i32(lx), i32(ly), i32(ys), workspace.data_ptr(), gc.data_ptr(),
                                 gc.numel() == 1 ? 0 : 1, gx.data_ptr(), current_stream()),
                 "cwrnnt_backward");
    return gx;
}

// Side streams of the pipelined step: one set per device and host thread (a pipe serves one call at a time), created
// on first use and kept for the life of the thread's process.
cwrnnt_pipe *pipe_of(int device_index)
{
    static thread_local std::vector<cwrnnt_pipe *> pipes;
    if (device_index >= static_cast<int>(pipes.size())) pipes.resize(device_index + 1, nullptr);
    if (!pipes[device_index]) check_status(cwrnnt_pipe_create(&pipes[device_index]), "cwrnnt_pipe_create");
    return pipes[device_index];
}

// Forward and gradient in one pipelined call, for an upstream gradient of 1 (scaled later by rnnt_scale_grad if the
// real one differs). Returns (costs [N], loss [], workspace bytes, grad_x like xs).
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor>
rnnt_loss_grad(const torch::Tensor &xs, const torch::Tensor &lx, const torch::Tensor &ys, const torch::Tensor &ly,
               int64_t blank, int64_t flags, int64_t mean_denominator, int64_t groups)
{
    check_inputs(xs, lx, ys, ly);
    const c10::cuda::CUDAGuard guard(xs.device());
    cwrnnt_problem p = describe(xs, lx, ys, blank, flags, mean_denominator);
    auto ws = make_workspace(p, xs);
    auto costs = torch::empty({lx.size(0)}, xs.options().dtype(cost_type(xs)));
    // written by the kernels whenever a reduction is asked for on a non-empty batch (NaN on invalid lengths)
    auto loss = ((flags & (CWRNNT_REDUCE_MEAN | CWRNNT_REDUCE_SUM)) && lx.size(0) > 0) ? torch::empty({}, costs.options())
                                                                   : torch::zeros({}, costs.options());
    auto gx = torch::empty_like(xs);
    check_status(cwrnnt_loss_grad(pipe_of(xs.get_device()), &p, xs.data_ptr(), i32(lx), i32(ly), i32(ys),
                                  ws.data_ptr(), ws.numel(), costs.data_ptr(), loss.data_ptr(), nullptr, 0,
                                  gx.data_ptr(), nullptr, 0, nullptr, static_cast<int32_t>(groups), current_stream()),
                 "cwrnnt_loss_grad");
    return {costs, loss, ws, gx};
}

// grad_x *= factor in place; factor holds one element of the costs dtype on the same device.
void rnnt_scale_grad(torch::Tensor grad_x, const torch::Tensor &factor)
{
    CHECK_CONTIGUOUS(grad_x);
    CHECK_CUDA(grad_x);
    CHECK_CUDA(factor);
    TORCH_CHECK(grad_x.dim() == 2 && factor.numel() == 1, "grad_x must be 2-D and factor a single element");
    const c10::cuda::CUDAGuard guard(grad_x.device());
    cwrnnt_problem p{};
    p.n_rows = grad_x.size(0);
    p.V = static_cast<int32_t>(grad_x.size(1));
    p.dtype = dtype_code(grad_x);
    auto f = factor.to(cost_type(grad_x)).contiguous();
    check_status(cwrnnt_scale_grad(&p, grad_x.data_ptr(), f.data_ptr(), current_stream()), "cwrnnt_scale_grad");
}

// Input validation ahead of the heavy kernels: [status bits, first bad sequence, max(lx), max(ly)]; one short sync.
std::vector<int64_t> rnnt_validate(const torch::Tensor &lx, const torch::Tensor &ys, const torch::Tensor &ly,
                                   int64_t n_rows, int64_t V)
{
    CHECK_INPUT(lx, torch::ScalarType::Int);
    CHECK_INPUT(ys, torch::ScalarType::Int);
    CHECK_INPUT(ly, torch::ScalarType::Int);
    TORCH_CHECK(ys.dim() == 2 && ys.size(0) == lx.size(0) && ly.size(0) == lx.size(0), "ys must be [N, Umax]");
    const c10::cuda::CUDAGuard guard(lx.device());
    cwrnnt_problem p{};
    p.n_rows = n_rows;
    p.V = static_cast<int32_t>(V);
    p.B = static_cast<int32_t>(lx.size(0));
    p.y_stride = p.max_u = static_cast<int32_t>(ys.size(1));
    auto scratch = torch::empty({4}, lx.options());
    int32_t st[4] = {0, 0, 0, 0};
    check_status(cwrnnt_validate(&p, i32(lx), i32(ly), i32(ys), scratch.data_ptr(), st, current_stream()),
                 "cwrnnt_validate");
    return {st[0], st[1], st[2], st[3]};
}

// The same validation queued without waiting: returns the four words as a pinned host tensor that is filled once the
// current stream has passed this point. The caller records an event, queues the loss kernels, then waits on the event.
torch::Tensor rnnt_validate_begin(const torch::Tensor &lx, const torch::Tensor &ys, const torch::Tensor &ly,
                                  int64_t n_rows, int64_t V)
{
    CHECK_INPUT(lx, torch::ScalarType::Int);
    CHECK_INPUT(ys, torch::ScalarType::Int);
    CHECK_INPUT(ly, torch::ScalarType::Int);
    TORCH_CHECK(ys.dim() == 2 && ys.size(0) == lx.size(0) && ly.size(0) == lx.size(0), "ys must be [N, Umax]");
    const c10::cuda::CUDAGuard guard(lx.device());
    cwrnnt_problem p{};
    p.n_rows = n_rows;
    p.V = static_cast<int32_t>(V);
    p.B = static_cast<int32_t>(lx.size(0));
    p.y_stride = p.max_u = static_cast<int32_t>(ys.size(1));
    auto scratch = torch::empty({4}, lx.options());  // freed stream-ordered by the caching allocator
    auto out = torch::empty({4}, torch::TensorOptions().dtype(torch::kInt32).pinned_memory(true));
    check_status(cwrnnt_validate_async(&p, i32(lx), i32(ly), i32(ys), scratch.data_ptr(), out.data_ptr<int32_t>(),
                                       current_stream()),
                 "cwrnnt_validate_async");
    return out;
}

// Device status words of a workspace: synchronises the current stream. [bits, first bad sequence, rows, 0].
std::vector<int64_t> rnnt_status(const torch::Tensor &workspace)
{
    CHECK_CUDA(workspace);
    const c10::cuda::CUDAGuard guard(workspace.device());
    int32_t st[4] = {0, 0, 0, 0};
    check_status(cwrnnt_read_status(workspace.data_ptr(), st, current_stream()), "cwrnnt_read_status");
    return {st[0], st[1], st[2], st[3]};
}

// Padded [N, T, U+1, V] -> compact [n_rows, V] (n_rows = sum T_n*(U_n+1), computed by the caller) and back.
torch::Tensor pack_padded(const torch::Tensor &padded, const torch::Tensor &lx, const torch::Tensor &ly,
                          int64_t n_rows)
{
    CHECK_CUDA(padded);
    CHECK_CONTIGUOUS(padded);
    CHECK_INPUT(lx, torch::ScalarType::Int);
    CHECK_INPUT(ly, torch::ScalarType::Int);
    TORCH_CHECK(padded.dim() == 4 && padded.size(0) == lx.size(0), "padded must be [N, T, U+1, V]");
    const c10::cuda::CUDAGuard guard(padded.device());
    cwrnnt_problem p{};
    p.n_rows = n_rows;
    p.V = static_cast<int32_t>(padded.size(3));
    p.B = static_cast<int32_t>(padded.size(0));
    p.y_stride = p.max_u = static_cast<int32_t>(padded.size(2) - 1);
    p.dtype = dtype_code(padded);
    auto scratch = torch::empty({cwrnnt_scatter_scratch_bytes(p.B)}, padded.options().dtype(torch::kUInt8));
    auto out = torch::empty({n_rows, padded.size(3)}, padded.options());
    check_status(cwrnnt_pack_padded(&p, padded.data_ptr(), static_cast<int32_t>(padded.size(1)),
                                    static_cast<int32_t>(padded.size(2)), i32(lx), i32(ly), scratch.data_ptr(),
                                    scratch.numel(), out.data_ptr(), current_stream()),
                 "cwrnnt_pack_padded");
    return out;
}

torch::Tensor unpack_padded(const torch::Tensor &compact, const torch::Tensor &lx, const torch::Tensor &ly,
                            int64_t T, int64_t Up)
{
    CHECK_CUDA(compact);
    CHECK_INPUT(lx, torch::ScalarType::Int);
    CHECK_INPUT(ly, torch::ScalarType::Int);
    TORCH_CHECK(compact.dim() == 2, "compact must be [n_rows, V]");
    const c10::cuda::CUDAGuard guard(compact.device());
    auto c = compact.contiguous();
    cwrnnt_problem p{};
    p.n_rows = c.size(0);
    p.V = static_cast<int32_t>(c.size(1));
    p.B = static_cast<int32_t>(lx.size(0));
    p.y_stride = p.max_u = static_cast<int32_t>(Up - 1);
    p.dtype = dtype_code(c);
    auto scratch = torch::empty({cwrnnt_scatter_scratch_bytes(p.B)}, c.options().dtype(torch::kUInt8));
    auto out = torch::empty({lx.size(0), T, Up, c.size(1)}, c.options());
    check_status(cwrnnt_unpack_padded(&p, c.data_ptr(), static_cast<int32_t>(T), static_cast<int32_t>(Up), i32(lx),
                                      i32(ly), scratch.data_ptr(), scratch.numel(), out.data_ptr(), current_stream()),
                 "cwrnnt_unpack_padded");
    return out;
}

// ------------------------------------------------------------------- the reference module's functions, same shapes

// cwarp_cuda.cpp:84-108. xs are log-probabilities. Returns (costs [N], grads [STU,2], alphas, betas [N,Tmax,Umax+1]).
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor, torch::Tensor>
compact_rnnt_loss_forward(const torch::Tensor xs, const torch::Tensor lx, const torch::Tensor ys,
                          const torch::Tensor ly, const int blank)
{
    check_inputs(xs, lx, ys, ly);
    TORCH_CHECK(xs.scalar_type() == torch::ScalarType::Float || xs.scalar_type() == torch::ScalarType::Double,
                "the reference-shaped entry points take float32 or float64 log-probabilities");
    const c10::cuda::CUDAGuard guard(xs.device());
    cwrnnt_problem p = describe(xs, lx, ys, blank, 0, 0);
    auto ws = make_workspace(p, xs);
    auto costs = torch::empty({lx.size(0)}, xs.options());
    check_status(cwrnnt_forward(&p, xs.data_ptr(), i32(lx), i32(ly), i32(ys), ws.data_ptr(), ws.numel(),
                                costs.data_ptr(), nullptr, current_stream()),
                 "cwrnnt_forward");
    auto grads = torch::empty({xs.size(0), 2}, xs.options());
    check_status(cwrnnt_pair_grads(&p, xs.data_ptr(), i32(lx), i32(ly), i32(ys), ws.data_ptr(), grads.data_ptr(),
                                   current_stream()),
                 "cwrnnt_pair_grads");
    // padded debug outputs need max T on the host, like the reference (cwarp_cuda_rnnt_kernel.cu:395-396)
    const int64_t t_max = lx.numel() ? lx.max().item<int64_t>() : 0;
    const int64_t u_max1 = ys.size(1) + 1;
    auto alphas = torch::empty({lx.size(0), t_max, u_max1}, xs.options());
    auto betas = torch::empty_like(alphas);
    check_status(cwrnnt_export_alpha_beta(&p, i32(lx), i32(ly), ws.data_ptr(), static_cast<int32_t>(t_max),
                                          static_cast<int32_t>(u_max1), alphas.data_ptr(), betas.data_ptr(),
                                          current_stream()),
                 "cwrnnt_export_alpha_beta");
    return {costs, grads, alphas, betas};
}

// cwarp_cuda.cpp:58-82. Costs only.
torch::Tensor compact_rnnt_loss(const torch::Tensor xs, const torch::Tensor lx, const torch::Tensor ys,
                                const torch::Tensor ly, const int blank)
{
    check_inputs(xs, lx, ys, ly);
    TORCH_CHECK(xs.scalar_type() == torch::ScalarType::Float || xs.scalar_type() == torch::ScalarType::Double,
                "the reference-shaped entry points take float32 or float64 log-probabilities");
    const c10::cuda::CUDAGuard guard(xs.device());
    cwrnnt_problem p = describe(xs, lx, ys, blank, CWRNNT_COSTS_ONLY, 0);
    auto ws = make_workspace(p, xs);
    auto costs = torch::empty({lx.size(0)}, xs.options());
    check_status(cwrnnt_forward(&p, xs.data_ptr(), i32(lx), i32(ly), i32(ys), ws.data_ptr(), ws.numel(),
                                costs.data_ptr(), nullptr, current_stream()),
                 "cwrnnt_forward");
    return costs;
}

// cwarp_cuda.cpp:110-136. grad_in [STU,2] is NOT modified (the reference scales it in place).
torch::Tensor compact_rnnt_loss_backward(torch::Tensor grad_in, const torch::Tensor grad_costs,
                                         const torch::Tensor labels, const torch::Tensor lx, const torch::Tensor ly,
                                         const int blank, const int V)
{
    CHECK_CUDA(grad_costs);
    CHECK_CUDA(grad_in);
    CHECK_INPUT(labels, torch::ScalarType::Int);
    CHECK_INPUT(lx, torch::ScalarType::Int);
    CHECK_INPUT(ly, torch::ScalarType::Int);
    TORCH_CHECK(grad_in.dim() == 2 && grad_in.size(1) == 2, "grad_in must be [STU, 2]");
    TORCH_CHECK(grad_in.scalar_type() == torch::ScalarType::Float || grad_in.scalar_type() == torch::ScalarType::Double,
                "grad_in must be float32 or float64");
    const c10::cuda::CUDAGuard guard(grad_in.device());
    auto g = grad_in.contiguous();
    auto gc = grad_costs.to(g.scalar_type()).contiguous();
    TORCH_CHECK(gc.numel() == lx.size(0), "grad_costs must be [N]");
    cwrnnt_problem p{};
    p.n_rows = g.size(0);
    p.V = V;
    p.B = static_cast<int32_t>(lx.size(0));
    p.y_stride = p.max_u = static_cast<int32_t>(labels.size(1));
    p.blank = blank;
    p.dtype = g.scalar_type() == torch::ScalarType::Double ? CWRNNT_F64 : CWRNNT_F32;
    auto scratch = torch::empty({cwrnnt_scatter_scratch_bytes(p.B)}, g.options().dtype(torch::kUInt8));
    auto dense = torch::empty({g.size(0), static_cast<int64_t>(V)}, g.options());
    check_status(cwrnnt_scatter_backward(&p, g.data_ptr(), gc.data_ptr(), i32(lx), i32(ly), i32(labels),
                                         scratch.data_ptr(), scratch.numel(), dense.data_ptr(), current_stream()),
                 "cwrnnt_scatter_backward");
    return dense;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m)
{
    m.def("_cwarp_rnnt_forward", &compact_rnnt_loss_forward,
          "Transducer loss forward for compact layout (reference shapes): (costs, grads[STU,2], alphas, betas).");
    m.def("_cwarp_rnnt_backward", &compact_rnnt_loss_backward,
          "Transducer loss backward for compact layout (reference shapes): dense [STU,V] gradient.");
    m.def("_cwarp_rnnt_loss", &compact_rnnt_loss, "Transducer costs without gradients.");
    m.def("_rnnt_forward", &rnnt_forward, "Fused forward: (costs, loss, workspace).");
    m.def("_rnnt_backward", &rnnt_backward, "Fused backward: gradient w.r.t. xs.");
    m.def("_rnnt_loss_grad", &rnnt_loss_grad,
          "Pipelined forward + gradient for an upstream gradient of 1: (costs, loss, workspace, grad_x).");
    m.def("_rnnt_scale_grad", &rnnt_scale_grad, "In-place grad_x *= factor (device scalar); free when the factor is 1.");
    m.def("_rnnt_validate", &rnnt_validate,
          "Validates lengths, row count and labels: [bits, first bad sequence, max lx, max ly] (one short sync).");
    m.def("_rnnt_validate_begin", &rnnt_validate_begin,
          "Queues the validation and returns a pinned int32[4] tensor filled once the current stream gets there.");
    m.def("_rnnt_status", &rnnt_status, "Status words of a workspace (synchronises).");
    m.def("_pack_padded", &pack_padded, "Padded [N,T,U+1,V] -> compact [n_rows,V].");
    m.def("_unpack_padded", &unpack_padded, "Compact [n_rows,V] -> zero-padded [N,T,U+1,V].");
    m.attr("FUSED_LOG_SOFTMAX") = static_cast<int>(CWRNNT_FUSED_LOG_SOFTMAX);
    m.attr("COSTS_ONLY") = static_cast<int>(CWRNNT_COSTS_ONLY);
    m.attr("REDUCE_MEAN") = static_cast<int>(CWRNNT_REDUCE_MEAN);
    m.attr("REDUCE_SUM") = static_cast<int>(CWRNNT_REDUCE_SUM);
    m.attr("AVERAGE_FRAMES") = static_cast<int>(CWRNNT_AVERAGE_FRAMES);
    m.attr("ST_BAD_LENGTH") = static_cast<int>(CWRNNT_ST_BAD_LENGTH);
    m.attr("ST_ROW_MISMATCH") = static_cast<int>(CWRNNT_ST_ROW_MISMATCH);
    m.attr("ST_BAD_LABEL") = static_cast<int>(CWRNNT_ST_BAD_LABEL);
    m.attr("ST_FWD_BWD_GAP") = static_cast<int>(CWRNNT_ST_FWD_BWD_GAP);
}
