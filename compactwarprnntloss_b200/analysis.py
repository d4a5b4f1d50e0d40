"""Lattice analysis on top of a forward pass: best alignment, node posteriors, padded alpha / beta.

The reference returns its alpha and beta arrays "for debugging or analysis" (cwarp_cuda_rnnt_kernel.cu:383-384,
returned at :496) and leaves the analysis to the caller; `analyse` runs the engine's forward on compact inputs and
returns what such a caller computes from them, all on the device, through the C ABI
(`cwrnnt_export_alignment`, `cwrnnt_export_posteriors`, `cwrnnt_export_alpha_beta`). There is no CPU fallback.
"""
from dataclasses import dataclass
from typing import Optional

import torch

from . import capi


@dataclass
class LatticeAnalysis:
    costs: torch.Tensor                  # [N]  -log P(y|x)
    moves: torch.Tensor                  # [N, max(T+U)] int32: 0 = blank move (next frame), 1 = label move, -1 padding
    path_log_prob: torch.Tensor          # [N]  log-probability of the best path
    posteriors: Optional[torch.Tensor]   # [N, Tmax, Umax+1] probability that the alignment passes through (t,u)
    alphas: Optional[torch.Tensor]       # [N, Tmax, Umax+1] zero-padded, as the reference returns them
    betas: Optional[torch.Tensor]

    def emission_frames(self, n: int) -> torch.Tensor:
        """Frame index at which each label of sequence n is emitted on the best path ([U_n] int64)."""
        mv = self.moves[n]
        mv = mv[mv >= 0]
        frames = torch.cumsum((mv == 0).long(), 0)  # frames completed before each move
        return frames[mv == 1]


def analyse(x: torch.Tensor, lx: torch.Tensor, y: torch.Tensor, ly: torch.Tensor, blank: int = 0, *,
            fused_log_softmax: bool = False, want_posteriors: bool = True, want_alpha_beta: bool = False,
            t_max: Optional[int] = None) -> LatticeAnalysis:
    """Forward pass on compact `x [sum_i T_i*(U_i+1), V]` (log-probabilities, or raw logits with
    ``fused_log_softmax=True``) followed by the analysis exports. `lx`, `ly` int32 [N], `y` int32 [N, Umax] as for
    `transducer_loss`. Reads `lx.max()` on the host once (the padded outputs need it) unless `t_max` is given."""
    assert x.dim() == 2 and y.dim() == 2 and lx.dtype == torch.int32 and ly.dtype == torch.int32
    x, y = x.contiguous(), y.contiguous()
    flags = capi.FUSED_LOG_SOFTMAX if fused_log_softmax else 0
    p = capi.make_problem(x, lx, y, blank, flags)
    ws = capi.alloc_workspace(p, x.device)
    costs = torch.empty(p.B, dtype=capi.cost_dtype(x.dtype), device=x.device)
    capi.forward(p, x, lx, ly, y if y.numel() else None, ws, costs)
    if t_max is None:
        t_max = int(lx.max()) if lx.numel() else 0
    u_max1 = y.size(1) + 1
    moves, scores = capi.export_alignment(p, lx, ly, ws, max(t_max + y.size(1), 1))
    post = capi.export_posteriors(p, lx, ly, ws, t_max, u_max1) if want_posteriors else None
    alphas = betas = None
    if want_alpha_beta:
        alphas = torch.empty(p.B, t_max, u_max1, dtype=costs.dtype, device=x.device)
        betas = torch.empty_like(alphas)
        capi.export_alpha_beta(p, lx, ly, ws, t_max, u_max1, alphas, betas)
    st = capi.read_status(ws)
    if st[0] & (capi.ST_BAD_LENGTH | capi.ST_ROW_MISMATCH):
        raise ValueError(f"invalid lengths (status {st}): need lx >= 1, 0 <= ly <= y.size(1) and sum(lx*(ly+1)) == x.size(0)")
    return LatticeAnalysis(costs, moves, scores, post, alphas, betas)
