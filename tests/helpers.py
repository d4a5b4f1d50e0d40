"""Shared input generators for the CPU and GPU tests."""
import numpy as np


def ragged_case(seed, N, Tr, Ur, V, sigma=1.0, blank=0, dtype=np.float32, allow_blank_label=False):
    """Random ragged batch: returns dict(x [STU,V] logits, lx, ly, y [N,max U] int32, blank, V)."""
    rng = np.random.default_rng(seed)
    lx = rng.integers(Tr[0], Tr[1] + 1, size=N).astype(np.int32)
    ly = rng.integers(Ur[0], Ur[1] + 1, size=N).astype(np.int32)
    umax = max(int(ly.max()), 0)
    lo = 0 if allow_blank_label else 1
    y = rng.integers(lo, V, size=(N, umax)).astype(np.int32) if umax > 0 else np.zeros((N, 0), np.int32)
    if blank != 0 and not allow_blank_label:
        y[y == blank] = 0
    rows = int((lx.astype(np.int64) * (ly.astype(np.int64) + 1)).sum())
    x = (rng.standard_normal((rows, V)) * sigma).astype(dtype)
    return dict(x=x, lx=lx, ly=ly, y=y, blank=blank, V=V)
