"""`compact_joint`: the joint network's broadcast-add written straight into the compact layout the loss takes.

    h = compact_joint(enc, pred, lx, ly, activation="tanh")     # [sum_n T_n*(U_n+1), H]
    logits = h @ W.t() + b                                      # a library GEMM, [n_rows, V], any of f32/f16/bf16
    loss = transducer_loss(logits, lx, y, ly, fused_log_softmax=True)

The reference leaves this step to its callers, who build the padded [N, T, U+1, H] tensor first and compact it
afterwards (test/test.py:34-48; cwarp_rnnt/__init__.py:52-59 for 4-D input). Here the padded tensor never exists.
The CUDA library is mandatory (no CPU or PyTorch fallback).
"""
from typing import Any, Optional

import torch

from . import capi

__all__ = ["compact_joint"]


class _CompactJoint(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, enc, pred, lx, ly, n_rows, activation):
        enc, pred = enc.contiguous(), pred.contiguous()
        ctx.save_for_backward(enc, pred, lx, ly)
        ctx.activation = activation
        return capi.joint_forward(enc, pred, lx, ly, n_rows, activation)

    @staticmethod
    def backward(ctx: Any, grad_out):
        enc, pred, lx, ly = ctx.saved_tensors
        genc, gpred = capi.joint_backward(enc, pred, lx, ly, grad_out.contiguous(), ctx.activation)
        return genc, gpred, None, None, None, None


def compact_joint(enc: torch.Tensor, pred: torch.Tensor, lx: torch.Tensor, ly: torch.Tensor,
                  activation: Optional[str] = "tanh", n_rows: Optional[int] = None) -> torch.Tensor:
    """enc [N, Tmax, H] (encoder frames), pred [N, Umax+1, H] (predictor states, position 0 = start symbol),
    lx, ly int32 [N] on the same device. Returns act(enc[n,t] + pred[n,u]) for t < lx[n], u <= ly[n] as compact rows.
    `n_rows` = sum(lx*(ly+1)); when omitted it is read from the device once (one synchronisation)."""
    assert enc.dim() == 3 and pred.dim() == 3 and enc.size(0) == pred.size(0) and enc.size(2) == pred.size(2)
    assert enc.dtype == pred.dtype and enc.is_cuda and pred.device == enc.device
    assert lx.dtype == torch.int32 and ly.dtype == torch.int32 and lx.numel() == enc.size(0) == ly.numel()
    assert activation in capi.ACTIVATIONS
    if n_rows is None:
        n_rows = int((lx.long() * (ly.long() + 1)).sum())
    return _CompactJoint.apply(enc, pred, lx, ly, n_rows, activation)
