"""ctypes view of the C ABI in include/cwarp_rnnt_b200.h, operating on torch CUDA tensors by raw pointer.

This is the same boundary a foreign-language binding would use: every call passes plain device pointers, sizes and the
current CUDA stream. There is no fallback: if the CUDA library has not been built the import of :func:`lib` raises.
"""
import ctypes
import os
from typing import Optional

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("CWRNNT_LIB") or os.path.join(_PKG, "libcwarp_rnnt_b200.so")  # override: another build

F32, F16, BF16, F64 = 0, 1, 2, 3
FUSED_LOG_SOFTMAX, COSTS_ONLY, REDUCE_MEAN, REDUCE_SUM, AVERAGE_FRAMES = 0x01, 0x02, 0x04, 0x08, 0x10
ST_BAD_LENGTH, ST_ROW_MISMATCH, ST_BAD_LABEL, ST_FWD_BWD_GAP = 0x01, 0x02, 0x04, 0x08
MAX_COLUMNS = 4096
STATIC_MAX_ROWS, STATIC_MAX_SEQUENCES = 131072, 1024
ERR_CAPACITY = 5

_DTYPES = {torch.float32: F32, torch.float16: F16, torch.bfloat16: BF16, torch.float64: F64}

EXPORTS = [
    "cwrnnt_abi_version", "cwrnnt_status_string", "cwrnnt_last_error", "cwrnnt_workspace_bytes", "cwrnnt_forward",
    "cwrnnt_backward", "cwrnnt_pair_grads", "cwrnnt_export_alpha_beta", "cwrnnt_scatter_scratch_bytes",
    "cwrnnt_scatter_backward", "cwrnnt_read_status", "cwrnnt_host_ctx_create", "cwrnnt_host_ctx_destroy",
    "cwrnnt_host_ctx_error", "cwrnnt_loss_grad_host", "cwrnnt_costs_static", "cwrnnt_forward_sharded",
    "cwrnnt_pack_padded", "cwrnnt_unpack_padded", "cwrnnt_pipe_create", "cwrnnt_pipe_destroy", "cwrnnt_loss_grad",
    "cwrnnt_scale_grad", "cwrnnt_pipeline_groups", "cwrnnt_joint_forward", "cwrnnt_joint_backward",
    "cwrnnt_pipe_wait_costs", "cwrnnt_validate", "cwrnnt_validate_async", "cwrnnt_static_status", "cwrnnt_fill_costs", "cwrnnt_recursion", "cwrnnt_alignment_scratch_bytes", "cwrnnt_export_alignment",
    "cwrnnt_export_posteriors", "cwrnnt_pipe_create_traced", "cwrnnt_pipe_timeline",
]


class Problem(ctypes.Structure):
    _fields_ = [("n_rows", ctypes.c_int64), ("V", ctypes.c_int32), ("B", ctypes.c_int32),
                ("y_stride", ctypes.c_int32), ("max_u", ctypes.c_int32), ("blank", ctypes.c_int32),
                ("dtype", ctypes.c_int32), ("flags", ctypes.c_int32), ("mean_denominator", ctypes.c_int32)]


class CwrnntError(RuntimeError):
    pass


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m compactwarprnntloss_b200.build` "
                              "(there is no CPU or PyTorch fallback)")
        L = ctypes.CDLL(LIB_PATH)
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
        pp = ctypes.POINTER(Problem)
        L.cwrnnt_abi_version.restype = ctypes.c_int
        L.cwrnnt_status_string.restype = ctypes.c_char_p
        L.cwrnnt_status_string.argtypes = [ctypes.c_int]
        L.cwrnnt_last_error.restype = ctypes.c_char_p
        L.cwrnnt_workspace_bytes.restype = i64
        L.cwrnnt_workspace_bytes.argtypes = [pp]
        L.cwrnnt_forward.argtypes = [pp, vp, vp, vp, vp, vp, i64, vp, vp, vp]
        L.cwrnnt_forward_sharded.argtypes = [pp, vp, vp, vp, vp, vp, i64, vp, vp, vp, i32, vp, vp]
        L.cwrnnt_backward.argtypes = [pp, vp, vp, vp, vp, vp, vp, i32, vp, vp]
        L.cwrnnt_pipe_create.argtypes = [ctypes.POINTER(vp)]
        L.cwrnnt_pipe_create_traced.argtypes = [ctypes.POINTER(vp)]
        L.cwrnnt_pipe_timeline.argtypes = [vp, ctypes.POINTER(ctypes.c_float), i32]
        L.cwrnnt_pipe_destroy.argtypes = [vp]
        L.cwrnnt_pipe_destroy.restype = None
        L.cwrnnt_pipe_wait_costs.argtypes = [vp, vp]
        L.cwrnnt_loss_grad.argtypes = [vp, pp, vp, vp, vp, vp, vp, i64, vp, vp, vp, i32, vp, vp, i32, vp, i32, vp]
        L.cwrnnt_scale_grad.argtypes = [pp, vp, vp, vp]
        L.cwrnnt_joint_forward.argtypes = [pp, i32, vp, i32, vp, i32, vp, vp, vp, i64, vp, vp]
        L.cwrnnt_joint_backward.argtypes = [pp, i32, vp, i32, vp, i32, vp, vp, vp, vp, i64, vp, vp, vp]
        L.cwrnnt_pipeline_groups.restype = i32
        L.cwrnnt_pipeline_groups.argtypes = [pp, i32]
        L.cwrnnt_pair_grads.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp]
        L.cwrnnt_export_alpha_beta.argtypes = [pp, vp, vp, vp, i32, i32, vp, vp, vp]
        L.cwrnnt_scatter_scratch_bytes.restype = i64
        L.cwrnnt_scatter_scratch_bytes.argtypes = [i32]
        L.cwrnnt_scatter_backward.argtypes = [pp, vp, vp, vp, vp, vp, vp, i64, vp, vp]
        L.cwrnnt_pack_padded.argtypes = [pp, vp, i32, i32, vp, vp, vp, i64, vp, vp]
        L.cwrnnt_unpack_padded.argtypes = [pp, vp, i32, i32, vp, vp, vp, i64, vp, vp]
        L.cwrnnt_costs_static.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp]
        L.cwrnnt_alignment_scratch_bytes.restype = i64
        L.cwrnnt_alignment_scratch_bytes.argtypes = [pp]
        L.cwrnnt_export_alignment.argtypes = [pp, vp, vp, vp, vp, i64, i32, vp, vp, vp]
        L.cwrnnt_export_posteriors.argtypes = [pp, vp, vp, vp, i32, i32, vp, vp]
        L.cwrnnt_recursion.argtypes = [pp, vp, vp, vp, i64, vp, vp, vp]
        L.cwrnnt_fill_costs.argtypes = [pp, vp, vp, vp, vp, vp, vp]
        L.cwrnnt_static_status.argtypes = [ctypes.POINTER(i32 * 4), vp]
        L.cwrnnt_read_status.argtypes = [vp, ctypes.POINTER(i32 * 4), vp]
        L.cwrnnt_validate.argtypes = [pp, vp, vp, vp, vp, ctypes.POINTER(i32 * 4), vp]
        L.cwrnnt_validate_async.argtypes = [pp, vp, vp, vp, vp, vp, vp]
        L.cwrnnt_host_ctx_create.argtypes = [ctypes.POINTER(vp)]
        L.cwrnnt_host_ctx_destroy.argtypes = [vp]
        L.cwrnnt_host_ctx_destroy.restype = None
        L.cwrnnt_host_ctx_error.restype = ctypes.c_char_p
        L.cwrnnt_host_ctx_error.argtypes = [vp]
        L.cwrnnt_loss_grad_host.argtypes = [vp, pp, vp, vp, vp, vp, vp, i32, vp, vp, vp, i64, ctypes.POINTER(i32 * 4)]
        _lib = L
    return _lib


def check(status: int, what: str = "cwrnnt") -> None:
    if status != 0:
        L = lib()
        msg = L.cwrnnt_status_string(status).decode()
        if status in (4, 5):
            msg += ": " + L.cwrnnt_last_error().decode()
        raise CwrnntError(f"{what}: {msg} (status {status})")


def dtype_code(dt: torch.dtype) -> int:
    if dt not in _DTYPES:
        raise TypeError(f"unsupported logits dtype {dt}; expected float32, float16, bfloat16 or float64")
    return _DTYPES[dt]


def cost_dtype(dt: torch.dtype) -> torch.dtype:
    return torch.float64 if dt == torch.float64 else torch.float32


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def make_problem(x: torch.Tensor, lx: torch.Tensor, y: torch.Tensor, blank: int, flags: int,
                 mean_denominator: int = 0, max_u: Optional[int] = None) -> Problem:
    ys = y.size(1) if y.dim() == 2 else 0
    return Problem(n_rows=x.size(0), V=x.size(1), B=lx.numel(), y_stride=ys, max_u=ys if max_u is None else max_u,
                   blank=blank, dtype=dtype_code(x.dtype), flags=flags, mean_denominator=mean_denominator)


def workspace_bytes(p: Problem) -> int:
    n = lib().cwrnnt_workspace_bytes(ctypes.byref(p))
    if n < 0:
        raise CwrnntError("invalid problem description")
    return int(n)


def alloc_workspace(p: Problem, device) -> torch.Tensor:
    # torch's caching allocator hands out 512-byte aligned blocks; the ABI needs 256
    return torch.empty(workspace_bytes(p), dtype=torch.uint8, device=device)


def forward(p: Problem, x, lx, ly, y, workspace, costs, loss=None) -> None:
    with torch.cuda.device(x.device):
        check(lib().cwrnnt_forward(ctypes.byref(p), _ptr(x), _ptr(lx), _ptr(ly), _ptr(y), _ptr(workspace),
                                   workspace.numel(), _ptr(costs), _ptr(loss), _stream(x.device)), "cwrnnt_forward")


def forward_sharded(p: Problem, x, lx, ly, y, workspace, costs, loss, global_ids, n_global, cost_vector) -> None:
    """Forward of this rank's shard; also fills cost_vector [n_global + 1] for one all-reduce(sum) across ranks."""
    with torch.cuda.device(x.device):
        check(lib().cwrnnt_forward_sharded(ctypes.byref(p), _ptr(x), _ptr(lx), _ptr(ly), _ptr(y), _ptr(workspace),
                                           workspace.numel(), _ptr(costs), _ptr(loss), _ptr(global_ids), n_global,
                                           _ptr(cost_vector), _stream(x.device)), "cwrnnt_forward_sharded")


def recursion(p: Problem, lx, ly, workspace, costs, loss=None) -> None:
    """The alpha/beta wavefront and the cost step alone, on a workspace a forward has already filled (same problem)."""
    with torch.cuda.device(lx.device):
        check(lib().cwrnnt_recursion(ctypes.byref(p), _ptr(lx), _ptr(ly), _ptr(workspace), workspace.numel(),
                                     _ptr(costs), _ptr(loss), _stream(lx.device)), "cwrnnt_recursion")


def backward(p: Problem, x, lx, ly, y, workspace, grad_costs, grad_costs_stride, grad_x) -> None:
    with torch.cuda.device(x.device):
        check(lib().cwrnnt_backward(ctypes.byref(p), _ptr(x), _ptr(lx), _ptr(ly), _ptr(y), _ptr(workspace),
                                    _ptr(grad_costs), grad_costs_stride, _ptr(grad_x), _stream(x.device)),
              "cwrnnt_backward")


class Pipe:
    """Side streams and events of the pipelined step (cwrnnt_pipe_create); bound to one device, one call at a time."""

    def __init__(self, device, traced: bool = False):
        self.device = torch.device("cuda", device) if not isinstance(device, torch.device) else device
        self._h = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            torch.cuda.current_stream()  # make sure the primary context exists
            make = lib().cwrnnt_pipe_create_traced if traced else lib().cwrnnt_pipe_create
            check(make(ctypes.byref(self._h)), "cwrnnt_pipe_create")

    def timeline(self):
        """Per sequence group of the last step (traced pipes, after a synchronise): [ms since the fork point at which
        its range was gathered, its wavefront was done, its gradient was done]."""
        buf = (ctypes.c_float * 24)()
        n = lib().cwrnnt_pipe_timeline(self._h, buf, 24)
        if n < 0:
            raise CwrnntError("cwrnnt_pipe_timeline: the pipe is not traced")
        return [[buf[3 * g + k] for k in range(3)] for g in range(n)]

    def wait_costs(self, stream: torch.cuda.Stream) -> None:
        """`stream` waits until the costs / loss / cost vector of the last loss_grad on this pipe are written (its
        gradient kernels may still be running): the place to start an all-reduce of the cost vector."""
        check(lib().cwrnnt_pipe_wait_costs(self._h, ctypes.c_void_p(stream.cuda_stream)), "cwrnnt_pipe_wait_costs")

    def close(self):
        if self._h:
            lib().cwrnnt_pipe_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def loss_grad(p: Problem, x, lx, ly, y, workspace, costs, loss, grad_costs, grad_costs_stride, grad_x, pipe=None,
              groups=0, global_ids=None, n_global=0, cost_vector=None) -> None:
    """Costs, loss and gradient in one call (cwrnnt_loss_grad): with a Pipe, the wavefront of each sequence group
    runs on a side stream underneath the gather and gradient passes; without, the same work on the current stream."""
    with torch.cuda.device(x.device):
        check(lib().cwrnnt_loss_grad(pipe._h if pipe is not None else None, ctypes.byref(p), _ptr(x), _ptr(lx),
                                     _ptr(ly), _ptr(y), _ptr(workspace), workspace.numel(), _ptr(costs), _ptr(loss),
                                     _ptr(grad_costs), grad_costs_stride, _ptr(grad_x), _ptr(global_ids), n_global,
                                     _ptr(cost_vector), groups, _stream(x.device)), "cwrnnt_loss_grad")


def pipeline_groups(p: Problem, groups: int = 0) -> int:
    """Sequence groups a pipelined step of this problem runs with (1 + 3 * groups kernel launches)."""
    n = lib().cwrnnt_pipeline_groups(ctypes.byref(p), groups)
    if n < 0:
        raise CwrnntError("cwrnnt_pipeline_groups: invalid argument")
    return n


def scale_grad(p: Problem, grad_x, factor) -> None:
    """grad_x *= factor[0] in place (factor: device scalar of the costs dtype); free on the device when it is 1."""
    with torch.cuda.device(grad_x.device):
        check(lib().cwrnnt_scale_grad(ctypes.byref(p), _ptr(grad_x), _ptr(factor), _stream(grad_x.device)),
              "cwrnnt_scale_grad")


def pair_grads(p: Problem, x, lx, ly, y, workspace, grads) -> None:
    with torch.cuda.device(grads.device):
        check(lib().cwrnnt_pair_grads(ctypes.byref(p), _ptr(x), _ptr(lx), _ptr(ly), _ptr(y), _ptr(workspace),
                                      _ptr(grads), _stream(grads.device)), "cwrnnt_pair_grads")


def export_alpha_beta(p: Problem, lx, ly, workspace, t_max, u_max1, alphas, betas) -> None:
    with torch.cuda.device(lx.device):
        check(lib().cwrnnt_export_alpha_beta(ctypes.byref(p), _ptr(lx), _ptr(ly), _ptr(workspace), t_max, u_max1,
                                             _ptr(alphas), _ptr(betas), _stream(lx.device)),
              "cwrnnt_export_alpha_beta")


def export_alignment(p: Problem, lx, ly, workspace, path_stride: int):
    """Best path of every sequence from a forward's workspace: (moves [B, path_stride] int32 - 0 blank move, 1 label
    move, -1 padding - and scores [B], the paths' log-probabilities)."""
    dev = lx.device
    n = lib().cwrnnt_alignment_scratch_bytes(ctypes.byref(p))
    scratch = torch.empty(n, dtype=torch.uint8, device=dev)
    moves = torch.empty(p.B, path_stride, dtype=torch.int32, device=dev)
    scores = torch.empty(p.B, dtype=torch.float64 if p.dtype == F64 else torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib().cwrnnt_export_alignment(ctypes.byref(p), _ptr(lx), _ptr(ly), _ptr(workspace), _ptr(scratch), n,
                                            path_stride, _ptr(moves), _ptr(scores), _stream(dev)),
              "cwrnnt_export_alignment")
    return moves, scores


def export_posteriors(p: Problem, lx, ly, workspace, t_max: int, u_max1: int):
    """Node posteriors exp(alpha + beta - log P) as a zero-padded [B, t_max, u_max1] tensor of the costs dtype."""
    dev = lx.device
    post = torch.empty(p.B, t_max, u_max1, dtype=torch.float64 if p.dtype == F64 else torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib().cwrnnt_export_posteriors(ctypes.byref(p), _ptr(lx), _ptr(ly), _ptr(workspace), t_max, u_max1,
                                             _ptr(post), _stream(dev)), "cwrnnt_export_posteriors")
    return post


def scatter_backward(p: Problem, grads, grad_costs, lx, ly, y, dense) -> None:
    n = lib().cwrnnt_scatter_scratch_bytes(p.B)
    scratch = torch.empty(n, dtype=torch.uint8, device=grads.device)
    with torch.cuda.device(grads.device):
        check(lib().cwrnnt_scatter_backward(ctypes.byref(p), _ptr(grads), _ptr(grad_costs), _ptr(lx), _ptr(ly),
                                            _ptr(y), _ptr(scratch), n, _ptr(dense), _stream(grads.device)),
              "cwrnnt_scatter_backward")


def pack_padded(padded: torch.Tensor, lx, ly, n_rows: int) -> torch.Tensor:
    """[B, T, U+1, V] -> compact [n_rows, V] keeping padded[n, :lx[n], :ly[n]+1] of every sequence."""
    B, T, Up, V = padded.shape
    out = torch.empty(n_rows, V, dtype=padded.dtype, device=padded.device)
    p = Problem(n_rows=n_rows, V=V, B=B, y_stride=Up - 1, max_u=Up - 1, blank=0, dtype=dtype_code(padded.dtype))
    n = lib().cwrnnt_scatter_scratch_bytes(B)
    scratch = torch.empty(n, dtype=torch.uint8, device=padded.device)
    with torch.cuda.device(padded.device):
        check(lib().cwrnnt_pack_padded(ctypes.byref(p), _ptr(padded), T, Up, _ptr(lx), _ptr(ly), _ptr(scratch), n,
                                       _ptr(out), _stream(padded.device)), "cwrnnt_pack_padded")
    return out


def unpack_padded(compact: torch.Tensor, lx, ly, B: int, T: int, Up: int) -> torch.Tensor:
    """Transpose of pack_padded: compact rows back into a zero-padded [B, T, U+1, V] tensor."""
    V = compact.size(1)
    out = torch.empty(B, T, Up, V, dtype=compact.dtype, device=compact.device)
    p = Problem(n_rows=compact.size(0), V=V, B=B, y_stride=Up - 1, max_u=Up - 1, blank=0,
                dtype=dtype_code(compact.dtype))
    n = lib().cwrnnt_scatter_scratch_bytes(B)
    scratch = torch.empty(n, dtype=torch.uint8, device=compact.device)
    with torch.cuda.device(compact.device):
        check(lib().cwrnnt_unpack_padded(ctypes.byref(p), _ptr(compact), T, Up, _ptr(lx), _ptr(ly), _ptr(scratch), n,
                                         _ptr(out), _stream(compact.device)), "cwrnnt_unpack_padded")
    return out


ACTIVATIONS = {None: 0, "none": 0, "relu": 1, "tanh": 2}


def _joint_problem(enc, pred, lx, n_rows):
    return Problem(n_rows, enc.size(2), lx.numel(), pred.size(1) - 1, pred.size(1) - 1, 0, dtype_code(enc.dtype), 0, 0)


def joint_forward(enc: torch.Tensor, pred: torch.Tensor, lx, ly, n_rows: int, activation="tanh") -> torch.Tensor:
    """act(enc[n,t] + pred[n,u]) for every lattice node, as compact rows [n_rows, H] (cwrnnt_joint_forward).
    enc [B, t_max, H], pred [B, u_max1, H], contiguous, same dtype and device."""
    out = torch.empty(n_rows, enc.size(2), dtype=enc.dtype, device=enc.device)
    p = _joint_problem(enc, pred, lx, n_rows)
    with torch.cuda.device(enc.device):
        scratch = torch.empty(lib().cwrnnt_scatter_scratch_bytes(p.B), dtype=torch.uint8, device=enc.device)
        check(lib().cwrnnt_joint_forward(ctypes.byref(p), ACTIVATIONS[activation], _ptr(enc), enc.size(1), _ptr(pred),
                                         pred.size(1), _ptr(lx), _ptr(ly), _ptr(scratch), scratch.numel(), _ptr(out),
                                         _stream(enc.device)), "cwrnnt_joint_forward")
    return out


def joint_backward(enc, pred, lx, ly, grad_out, activation="tanh"):
    """(grad_enc like enc, grad_pred like pred) from grad_out [n_rows, H] (cwrnnt_joint_backward)."""
    genc, gpred = torch.empty_like(enc), torch.empty_like(pred)
    p = _joint_problem(enc, pred, lx, grad_out.size(0))
    with torch.cuda.device(enc.device):
        scratch = torch.empty(lib().cwrnnt_scatter_scratch_bytes(p.B), dtype=torch.uint8, device=enc.device)
        check(lib().cwrnnt_joint_backward(ctypes.byref(p), ACTIVATIONS[activation], _ptr(enc), enc.size(1), _ptr(pred),
                                          pred.size(1), _ptr(lx), _ptr(ly), _ptr(grad_out), _ptr(scratch),
                                          scratch.numel(), _ptr(genc), _ptr(gpred), _stream(enc.device)),
              "cwrnnt_joint_backward")
    return genc, gpred


def costs_static(p: Problem, x, lx, ly, y, costs, loss=None) -> None:
    """Costs-only forward on the library's built-in scratch: no workspace argument, nothing allocated. Problems above
    STATIC_MAX_ROWS rows / STATIC_MAX_SEQUENCES sequences raise CwrnntError (status 5). Calls on one device share the
    scratch, so keep them on one stream."""
    with torch.cuda.device(x.device):
        check(lib().cwrnnt_costs_static(ctypes.byref(p), _ptr(x), _ptr(lx), _ptr(ly), _ptr(y), _ptr(costs),
                                        _ptr(loss), _stream(x.device)), "cwrnnt_costs_static")


def fill_costs(p: Problem, lx, ll_alpha, ll_beta, costs, status) -> None:
    """costs[n] = -guarded(ll_alpha[n], ll_beta[n]); ORs ST_FWD_BWD_GAP into the device int32 word `status`."""
    with torch.cuda.device(lx.device):
        check(lib().cwrnnt_fill_costs(ctypes.byref(p), _ptr(lx), _ptr(ll_alpha), _ptr(ll_beta), _ptr(costs),
                                      _ptr(status), _stream(lx.device)), "cwrnnt_fill_costs")


def static_status(device):
    """Status words of the last costs_static call on `device` (synchronises its current stream)."""
    out = (ctypes.c_int32 * 4)()
    with torch.cuda.device(device):
        check(lib().cwrnnt_static_status(ctypes.byref(out), _stream(device)), "cwrnnt_static_status")
    return list(out)


def read_status(workspace: torch.Tensor):
    out = (ctypes.c_int32 * 4)()
    with torch.cuda.device(workspace.device):
        check(lib().cwrnnt_read_status(_ptr(workspace), ctypes.byref(out), _stream(workspace.device)),
              "cwrnnt_read_status")
    return list(out)


def validate(p: Problem, lx, ly, y):
    """[status bits, first bad sequence, max(lx), max(ly)] from one small kernel and one short synchronisation."""
    out = (ctypes.c_int32 * 4)()
    with torch.cuda.device(lx.device):
        scratch = torch.empty(4, dtype=torch.int32, device=lx.device)
        check(lib().cwrnnt_validate(ctypes.byref(p), _ptr(lx), _ptr(ly), _ptr(y) if y is not None and y.numel() else None,
                                    _ptr(scratch), ctypes.byref(out), _stream(lx.device)), "cwrnnt_validate")
    return list(out)


def validate_async(p: Problem, lx, ly, y, out_pinned: torch.Tensor, scratch: torch.Tensor) -> None:
    """Queues the validation on the current stream and returns; `out_pinned` (pinned int32[4] CPU tensor) holds
    [status bits, first bad sequence, max(lx), max(ly)] once the stream - or an event recorded after this call - is
    waited for. `scratch`: int32[4] on the device, kept alive by the caller until then."""
    assert out_pinned.is_pinned() and out_pinned.dtype == torch.int32 and out_pinned.numel() >= 4
    with torch.cuda.device(lx.device):
        check(lib().cwrnnt_validate_async(ctypes.byref(p), _ptr(lx), _ptr(ly),
                                          _ptr(y) if y is not None and y.numel() else None, _ptr(scratch),
                                          _ptr(out_pinned), _stream(lx.device)), "cwrnnt_validate_async")


class HostPipeline:
    """Host-buffer entry point (cwrnnt_loss_grad_host): CPU tensors in, CPU tensors out, chunked over PCIe."""

    def __init__(self, device=0):
        self.device = torch.device("cuda", device) if not isinstance(device, torch.device) else device
        self._ctx = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            torch.cuda.current_stream()  # make sure the primary context exists
            check(lib().cwrnnt_host_ctx_create(ctypes.byref(self._ctx)), "cwrnnt_host_ctx_create")

    def close(self):
        if self._ctx:
            lib().cwrnnt_host_ctx_destroy(self._ctx)
            self._ctx = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def run(self, x, lx, ly, y, blank=0, flags=FUSED_LOG_SOFTMAX, grad_costs=None, grad_x=None, chunk_rows=0,
            mean_denominator=0):
        """All tensors on the CPU (pin them for overlap). Returns (costs, loss or None, status words)."""
        assert not x.is_cuda and x.is_contiguous()
        p = make_problem(x, lx, y, blank, flags, mean_denominator)
        ct = cost_dtype(x.dtype)
        costs = torch.empty(p.B, dtype=ct)
        loss = torch.zeros((), dtype=ct) if flags & (REDUCE_MEAN | REDUCE_SUM) else None
        st = (ctypes.c_int32 * 4)()
        stride = 0
        if grad_costs is not None:
            grad_costs = grad_costs.to(ct).contiguous()
            stride = 0 if grad_costs.numel() == 1 else 1
        rc = lib().cwrnnt_loss_grad_host(self._ctx, ctypes.byref(p), _ptr(x), _ptr(lx), _ptr(ly),
                                         _ptr(y) if y.numel() else None, _ptr(grad_costs), stride, _ptr(costs),
                                         _ptr(loss), _ptr(grad_x), chunk_rows, ctypes.byref(st))
        if rc == 4:
            raise CwrnntError("cwrnnt_loss_grad_host: " + lib().cwrnnt_host_ctx_error(self._ctx).decode())
        check(rc, "cwrnnt_loss_grad_host")
        return costs, loss, list(st)
