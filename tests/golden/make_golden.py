"""Generates the golden fixtures in this folder from the reference's own CUDA kernels.

Run on a machine with a B200 after `python oracle/build_ref.py` has produced oracle/_ref/cwarp_rnnt_ref_C.so (the
reference's three unmodified source files compiled for sm_100a):

    python tests/golden/make_golden.py <output-folder>

and copy the resulting ref_*.npz files here. Inputs are regenerated from seeds (tests/helpers.ragged_case); the
float32 log-probabilities fed to the reference are stored too, so the CPU checker consumes bit-identical inputs.
Stored per case: lx, ly, y, blank, lp (small cases) or the gathered pair g [STU,2], and the reference outputs
costs [N], grads [STU,2], alphas/betas [N,Tmax,Umax+1], cost-only costs, dense backward [STU,V] (small cases).
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle.build_ref import load_ref  # noqa: E402
from tests.helpers import ragged_case  # noqa: E402

# name, seed, N, T range, U range, V, sigma, store_full_lp
CASES = [
    ("v3_small", 101, 6, (2, 30), (1, 14), 3, 1.0, True),      # the reference's own test uses V = 3
    ("v16_ragged", 102, 5, (1, 40), (1, 20), 16, 2.0, True),
    ("v8_tiles", 103, 3, (60, 100), (30, 45), 8, 1.0, True),     # several 32-frame tiles per sequence
    ("v64_tiny_cfg", 104, 4, (20, 50), (5, 15), 64, 1.0, False),  # shape of the tiny benchmark configuration
    ("v32_long", 105, 2, (180, 250), (40, 80), 32, 2.0, False),   # lattice of the Conformer-shape configuration
]


def main(out_dir):
    ref = load_ref()
    if ref is None:
        raise SystemExit("oracle/_ref/cwarp_rnnt_ref_C.so not built")
    os.makedirs(out_dir, exist_ok=True)
    dev = torch.device("cuda:0")
    for name, seed, N, Tr, Ur, V, sigma, full in CASES:
        c = ragged_case(seed, N, Tr, Ur, V=V, sigma=sigma)  # every U range starts at 1: the reference needs max U >= 1
        x = torch.tensor(c["x"], device=dev)
        lp = torch.log_softmax(x, -1).contiguous()
        lx = torch.tensor(c["lx"], device=dev)
        ly = torch.tensor(c["ly"], device=dev)
        y = torch.tensor(c["y"], device=dev).contiguous()
        costs, grads, alphas, betas = ref._cwarp_rnnt_forward(lp, lx, y, ly, 0)
        costs_only = ref._cwarp_rnnt_loss(lp, lx, y, ly, 0)
        torch.cuda.synchronize()
        rng = np.random.default_rng(seed + 1)
        gc = torch.tensor(rng.uniform(0.5, 2.0, size=N).astype(np.float32), device=dev)
        dense = ref._cwarp_rnnt_backward(grads.clone(), gc, y, lx, ly, 0, V)
        torch.cuda.synchronize()
        # gathered pair exactly as the reference sees it
        off = np.concatenate([[0], np.cumsum(c["lx"].astype(np.int64) * (c["ly"].astype(np.int64) + 1))])
        lp_h = lp.cpu().numpy()
        g = np.zeros((lp_h.shape[0], 2), np.float32)
        for n in range(N):
            T, m = int(c["lx"][n]), int(c["ly"][n]) + 1
            blk = lp_h[off[n]:off[n + 1]].reshape(T, m, V)
            g[off[n]:off[n + 1], 0] = blk[:, :, 0].reshape(-1)
            lab = np.zeros((T, m), np.float32)
            for u in range(m - 1):
                lab[:, u] = blk[:, u, c["y"][n, u]]
            g[off[n]:off[n + 1], 1] = lab.reshape(-1)
        rec = dict(seed=seed, N=N, Tr=Tr, Ur=Ur, V=V, sigma=sigma, lx=c["lx"], ly=c["ly"], y=c["y"], blank=0, g=g,
                   costs=costs.cpu().numpy(), grads=grads.cpu().numpy(), alphas=alphas.cpu().numpy(),
                   betas=betas.cpu().numpy(), costs_only=costs_only.cpu().numpy(), grad_costs=gc.cpu().numpy())
        if full:
            rec["lp"] = lp_h
            rec["dense"] = dense.cpu().numpy()
        else:
            rec["dense_abs_sum"] = dense.abs().sum(-1).cpu().numpy()
        np.savez_compressed(os.path.join(out_dir, f"ref_{name}.npz"), **rec)
        print(name, "rows", lp_h.shape[0], "costs", costs.cpu().numpy()[:3])


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "golden_out"))
