"""Seeded synthetic workloads with the shapes of the five benchmark configurations.

They stand in for a Conformer-transducer ASR joint-network output: no dataset is read. Lengths and labels come from
``torch.Generator('cpu').manual_seed(1000 * cfg)``; the logits of sequence ``i`` come from a generator seeded
``1000 * cfg + 1 + i``, so a sequence has the same data whichever rank or chunk it lands in. ``N(0, s)`` means
standard deviation ``s``. Logits are drawn in float32 and then cast. All ranges are inclusive.
"""
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch


@dataclass(frozen=True)
class Workload:
    cfg: int
    name: str
    B: int
    V: int
    dtype: torch.dtype
    sigma: float
    reduction: str


WORKLOADS = {
    1: Workload(1, "tiny B=4 T~U[20,50] U~U[5,15] V=64 fp32", 4, 64, torch.float32, 1.0, "mean"),
    2: Workload(2, "conformer B=32 T~U[150,250] U~U[20,80] V=1024 fp32", 32, 1024, torch.float32, 2.0, "mean"),
    3: Workload(3, "large-vocab B=16 T~U[300,500] U~U[50,150] V=4096 bf16", 16, 4096, torch.bfloat16, 3.0, "sum"),
    4: Workload(4, "long-form B=4 T~U[1000,1500] U~U[200,400] V=512 fp32", 4, 512, torch.float32, 1.0, "mean"),
    5: Workload(5, "ragged B=256 T~lognormal(ln200,0.6) clip[20,1200] U=round(T*U[.05,.3])+1 V=128 fp16",
                256, 128, torch.float16, 1.0, "mean"),
}


def lengths_and_labels(cfg: int, B: Optional[int] = None):
    """Returns (lx[B] int32, ly[B] int32, y[B, max ly] int32 zero-padded) on the CPU."""
    w = WORKLOADS[cfg]
    B = w.B if B is None else B
    g = torch.Generator("cpu").manual_seed(1000 * cfg)
    if cfg == 1:
        lx = torch.randint(20, 51, (B,), generator=g)
        ly = torch.randint(5, 16, (B,), generator=g)
    elif cfg == 2:
        lx = torch.randint(150, 251, (B,), generator=g)
        ly = torch.randint(20, 81, (B,), generator=g)
    elif cfg == 3:
        lx = torch.randint(300, 501, (B,), generator=g)
        ly = torch.randint(50, 151, (B,), generator=g)
    elif cfg == 4:
        lx = torch.randint(1000, 1501, (B,), generator=g)
        ly = torch.randint(200, 401, (B,), generator=g)
    elif cfg == 5:
        z = torch.randn(B, generator=g, dtype=torch.float64)
        lx = torch.exp(torch.log(torch.tensor(200.0, dtype=torch.float64)) + 0.6 * z).round().clamp(20, 1200).long()
        frac = 0.05 + 0.25 * torch.rand(B, generator=g, dtype=torch.float64)
        ly = (lx.double() * frac).round().long() + 1
    else:
        raise ValueError(f"unknown workload {cfg}")
    umax = int(ly.max())
    y = torch.randint(1, w.V, (B, umax), generator=g)
    y = y * (torch.arange(umax)[None, :] < ly[:, None])
    return lx.int(), ly.int(), y.int()


def sequence_logits(cfg: int, i: int, T: int, U: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Logits of global sequence ``i``: [T*(U+1), V] in the workload's dtype, rows in (t, u) row-major order."""
    w = WORKLOADS[cfg]
    g = torch.Generator("cpu").manual_seed(1000 * cfg + 1 + i)
    rows = T * (U + 1)
    if out is not None and out.dtype == torch.float32:
        out.normal_(0.0, w.sigma, generator=g)
        return out
    x = torch.empty(rows, w.V, dtype=torch.float32).normal_(0.0, w.sigma, generator=g)
    if out is not None:
        out.copy_(x)
        return out
    return x.to(w.dtype)


def compact_logits(cfg: int, lx: torch.Tensor, ly: torch.Tensor, ids: Optional[Sequence[int]] = None,
                   pin: bool = False) -> torch.Tensor:
    """Compact [sum_i T_i*(U_i+1), V] logits of the listed global sequences (default: all), on the CPU."""
    w = WORKLOADS[cfg]
    ids = list(range(len(lx))) if ids is None else list(ids)
    rows = [int(lx[i]) * (int(ly[i]) + 1) for i in ids]
    x = torch.empty(sum(rows), w.V, dtype=w.dtype, pin_memory=pin)
    at = 0
    for i, r in zip(ids, rows):
        sequence_logits(cfg, i, int(lx[i]), int(ly[i]), out=x[at:at + r])
        at += r
    return x


def lattice_nodes(lx: torch.Tensor, ly: torch.Tensor, ids: Optional[List[int]] = None) -> int:
    n = lx.long() * (ly.long() + 1)
    return int(n.sum() if ids is None else n[list(ids)].sum())
