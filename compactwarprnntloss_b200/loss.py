"""`transducer_loss`: the reference's Python entry point (cwarp_rnnt/__init__.py:32-73) on the B200 engine.

Same positional signature and argument contract; keyword-only additions:

gather              accepted for callers that pass ``gather=True`` to comparable packages; the compact engine always
                    gathers the blank and label columns internally, so both values give the same result.
average_frames      divide each sequence's cost (and its gradient) by its frame count T_n before the reduction.
fused_log_softmax   False (default, the reference contract): ``x`` holds log-probabilities and the gradient is zero
                    except at the blank and label columns. True: ``x`` holds raw logits; the row-wise log-softmax and
                    its backward are fused into the loss kernels and the gradient is dense. On already-normalised
                    input both settings return the same loss.
eager_grad          True (default): when ``x`` requires a gradient and the reduction is 'mean' or 'sum', the gradient
                    is computed inside the forward call, as the reference does (its forward returns the gradients,
                    cwarp_rnnt/__init__.py:14-16), by the pipelined single-call step: the alpha/beta wavefront of each
                    group of sequences runs on a side stream underneath the two bandwidth-bound passes. ``backward``
                    then only scales the stored gradient (a no-op on the device when the upstream gradient is 1).
                    False: the gradient pass runs inside ``backward`` with the upstream gradient folded in - one pass
                    less when that gradient is not 1 (loss scaling), no overlap, and nothing computed if ``backward``
                    is never called.
check               True (default): the reference's assertions, including ``y.size(1) == ly.max()``, plus checks the
                    reference lacks (lengths, row count, label range). All of them that need device data come from
                    one small validation kernel queued BEFORE the loss kernels; the host waits for its four words
                    only after the loss kernels are queued as well, so neither the GPU nor the loss waits for the
                    check, and a bad batch still raises before a loss is returned. False: no host synchronisation at
                    all; invalid lengths then surface as NaN costs, NaN loss and a NaN gradient.

The CUDA extension is mandatory: importing this module without it raises ImportError (no CPU or PyTorch fallback).
"""
from typing import Any, Literal, Optional

import torch

try:
    from . import _C as core
except ImportError as e:  # pragma: no cover - exercised only on a box without the built extension
    raise ImportError("compactwarprnntloss_b200._C is not built; run `python -m compactwarprnntloss_b200.build` "
                      "(the package has no CPU or PyTorch fallback)") from e

__all__ = ["transducer_loss", "TransducerLoss", "compact_from_padded"]


class _TransLoss(torch.autograd.Function):
    """forward -> (costs [N], loss []); only one of the two is consumed, depending on the reduction."""

    @staticmethod
    def forward(ctx: Any, xs, lx, ys, ly, blank, flags, mean_denominator, check, eager_grad):
        needs_grad = xs.requires_grad
        ctx.grad_x = None
        if needs_grad and eager_grad and flags & (core.REDUCE_MEAN | core.REDUCE_SUM):
            costs, loss, ws, ctx.grad_x = core._rnnt_loss_grad(xs, lx, ys, ly, blank, flags, mean_denominator, 0)
        else:
            run_flags = flags if needs_grad else (flags | core.COSTS_ONLY)
            costs, loss, ws = core._rnnt_forward(xs, lx, ys, ly, blank, run_flags, mean_denominator)
        if check:
            st = core._rnnt_status(ws)
            if st[0] & core.ST_BAD_LENGTH:
                raise ValueError(f"invalid length at sequence {st[1]}: need lx >= 1 and 0 <= ly <= y.size(1)")
            if st[0] & core.ST_ROW_MISMATCH:
                raise ValueError(f"x has {xs.size(0)} rows but sum(lx*(ly+1)) is different")
            if st[0] & core.ST_BAD_LABEL:
                raise ValueError("a label lies outside [0, V)")
        if needs_grad:
            ctx.save_for_backward(xs, lx, ys, ly, ws)
            ctx.blank, ctx.flags, ctx.mean_denominator = blank, flags, mean_denominator
        ctx.mark_non_differentiable(*(() if needs_grad else (costs, loss)))
        return costs, loss

    @staticmethod
    def backward(ctx: Any, grad_costs, grad_loss):
        xs, lx, ys, ly, ws = ctx.saved_tensors
        reduced = ctx.flags & (core.REDUCE_MEAN | core.REDUCE_SUM)
        g = grad_loss if reduced else grad_costs
        if ctx.grad_x is not None:
            # computed during forward for an upstream gradient of 1; handed over once (a second backward over a
            # retained graph recomputes it below from the saved workspace)
            grad_x, ctx.grad_x = ctx.grad_x, None
            core._rnnt_scale_grad(grad_x, g)
        else:
            grad_x = core._rnnt_backward(xs, lx, ys, ly, ctx.blank, ctx.flags, ctx.mean_denominator, ws,
                                         g.contiguous())
        return grad_x, None, None, None, None, None, None, None, None


class _PackPadded(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x, lx, ly, n_rows):
        ctx.save_for_backward(lx, ly)
        ctx.shape = x.shape
        return core._pack_padded(x.contiguous(), lx, ly, n_rows)

    @staticmethod
    def backward(ctx: Any, grad):
        lx, ly = ctx.saved_tensors
        return core._unpack_padded(grad, lx, ly, ctx.shape[1], ctx.shape[2]), None, None, None


def compact_from_padded(x: torch.Tensor, lx: torch.Tensor, ly: torch.Tensor) -> torch.Tensor:
    """[N, T, U+1, V] padded joint output -> compact [sum_i T_i*(U_i+1), V], keeping x[i, :T_i, :U_i+1] of every
    sequence in (t, u) row-major order (the layout of the reference's test/test.py:34-48). Differentiable: the
    gradient is scattered back into a zero-padded tensor. Reads the lengths on the host once for the row count."""
    n_rows = int((lx.long() * (ly.long() + 1)).sum())
    return _PackPadded.apply(x, lx, ly, n_rows)


def transducer_loss(x: torch.Tensor, lx: torch.Tensor, y: torch.Tensor, ly: torch.Tensor, blank: int = 0,
                    reduction: Optional[Literal["mean", "sum", "none"]] = "mean", *, gather: bool = True,
                    average_frames: bool = False, fused_log_softmax: bool = False, check: bool = True,
                    mean_denominator: int = 0, eager_grad: bool = True) -> torch.Tensor:
    """Transducer loss with compact layout. See the module docstring for the keyword-only options."""
    del gather  # always on
    assert lx.dtype == torch.int32
    assert ly.dtype == torch.int32
    assert y.dtype == torch.int32
    assert reduction in ["mean", "sum", "none"] or reduction is None
    # y: (N, U)
    assert y.dim() == 2
    assert y.size(0) == lx.size(0)
    assert y.size(0) == ly.size(0)
    assert blank >= 0 and blank < x.size(-1)

    def _raise_on(st, rows):
        if st[0] & core.ST_BAD_LENGTH:
            raise ValueError(f"invalid length at sequence {st[1]}: need lx >= 1 and 0 <= ly <= y.size(1)")
        if st[0] & core.ST_ROW_MISMATCH:
            raise ValueError(f"x has {rows} rows but sum(lx*(ly+1)) is different")
        if st[0] & core.ST_BAD_LABEL:
            raise ValueError("a label lies outside [0, V)")

    y = y.contiguous()
    pending = None  # (pinned status words, event): a validation that is queued but not yet waited for
    if x.dim() == 4:
        print("WARNING: it seems your input is not compact... would try to compact the input.")
        N, T, Up, V = x.size()
        assert y.size(1) + 1 == Up
        # the compaction reads the lengths on the host anyway (row count), so this path validates them first, with a
        # wait, before any kernel indexes the padded tensor with them
        n_rows = int((lx.long() * (ly.long() + 1)).sum())
        if check:
            st = core._rnnt_validate(lx, y, ly, n_rows, V)
            assert y.size(1) == st[3]                               # reference: y.size(1) == ly.max()
            assert st[2] == T                                       # reference: lx.max() == T for 4-D input
            _raise_on(st, n_rows)
        x = _PackPadded.apply(x, lx, ly, n_rows)
    elif check:
        # bits, first bad sequence, max(lx), max(ly): everything the assertions below need from the device, queued
        # AHEAD of the loss kernels and waited for only after they are queued too - the kernels protect themselves
        # (invalid lengths: they return at once and the results are NaN; labels are clamped), so the GPU does not
        # idle for the round trip and a bad batch still raises before a loss is returned
        words = core._rnnt_validate_begin(lx, y, ly, x.size(0), x.size(1))
        done = torch.cuda.Event()
        done.record(torch.cuda.current_stream(lx.device))
        pending = (words, done)

    # x: (STU, V)
    assert x.dim() == 2

    flags = 0
    if fused_log_softmax:
        flags |= core.FUSED_LOG_SOFTMAX
    if average_frames:
        flags |= core.AVERAGE_FRAMES
    if reduction == "mean":
        flags |= core.REDUCE_MEAN
    elif reduction == "sum":
        flags |= core.REDUCE_SUM
    elif not (reduction == "none" or reduction is None):
        raise ValueError

    # validated here: the autograd function itself does not read the device status back
    costs, loss = _TransLoss.apply(x.contiguous(), lx, y, ly, blank, flags, mean_denominator, False, eager_grad)
    if pending is not None:
        words, done = pending
        done.synchronize()
        st = words.tolist()
        assert y.size(1) == st[3]                                   # reference: y.size(1) == ly.max()
        _raise_on(st, x.size(0))
    return loss if reduction in ("mean", "sum") else costs


class TransducerLoss(torch.nn.Module):
    """Module form of :func:`transducer_loss`."""

    def __init__(self, blank: int = 0, reduction: Optional[str] = "mean", average_frames: bool = False,
                 fused_log_softmax: bool = False, check: bool = True, eager_grad: bool = True):
        super().__init__()
        self.blank, self.reduction = blank, reduction
        self.average_frames, self.fused_log_softmax, self.check = average_frames, fused_log_softmax, check
        self.eager_grad = eager_grad

    def forward(self, x, lx, y, ly):
        return transducer_loss(x, lx, y, ly, self.blank, self.reduction, average_frames=self.average_frames,
                               fused_log_softmax=self.fused_log_softmax, check=self.check,
                               eager_grad=self.eager_grad)
