"""Pins the CPU checker to the reference itself: fixtures in tests/golden/ are outputs of the reference's own CUDA
kernels (its three source files compiled unmodified for sm_100a and run on a B200 by tests/golden/make_golden.py).

The float32 "as the reference computes it" flavour of the checker must reproduce them to float32 rounding (costs come
out bit-identical; exp/log1p differ by an ulp between libm and CUDA, so alphas and gradients get a few-ulp band). The
double flavour, which is what the CUDA engine is held to, must agree within the reference's own float32 error.
"""
import glob
import os

import numpy as np
import pytest

GOLD = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "ref_*.npz")))


def _compact(padded, lx, ly):
    out = []
    for n in range(len(lx)):
        T, m = int(lx[n]), int(ly[n]) + 1
        out.append(padded[n, :T, :m].reshape(-1))
    return np.concatenate(out)


def test_fixtures_present():
    assert len(GOLD) >= 5


@pytest.mark.parametrize("path", GOLD, ids=[os.path.basename(p)[4:-4] for p in GOLD])
def test_ref32_flavour_reproduces_reference_outputs(oracle, path):
    z = np.load(path)
    lx, ly = z["lx"], z["ly"]
    got = oracle.forward_ref32(z["g"], lx, ly, want_ab=True)
    np.testing.assert_allclose(got["costs"], z["costs"], rtol=2e-7, atol=0)
    np.testing.assert_allclose(z["costs_only"], z["costs"], rtol=2e-6)  # reference: beta-only path == full path
    scale = np.abs(z["costs"]).max()
    assert np.abs(got["alpha"] - _compact(z["alphas"], lx, ly)).max() <= 4e-7 * scale
    assert np.abs(got["beta"] - _compact(z["betas"], lx, ly)).max() <= 4e-7 * scale
    assert np.abs(got["grads"] - z["grads"]).max() <= 1e-5
    # padding of the reference's [N, Tmax, Umax+1] outputs is zero
    for n in range(len(lx)):
        assert np.all(z["alphas"][n, int(lx[n]):] == 0) and np.all(z["alphas"][n, :, int(ly[n]) + 1:] == 0)


@pytest.mark.parametrize("path", GOLD, ids=[os.path.basename(p)[4:-4] for p in GOLD])
def test_double_flavour_within_reference_float_error(oracle, path):
    z = np.load(path)
    f64 = oracle.forward(z["g"].astype(np.float64), z["lx"], z["ly"])
    np.testing.assert_allclose(f64["costs"], z["costs"], rtol=1e-6)
    # the reference's float32 recursion drifts with lattice size: 4e-6 (T+U ~ 40) ... 9e-4 (T+U ~ 330)
    diag = int((z["lx"] + z["ly"]).max())
    assert np.abs(f64["grads"] - z["grads"]).max() <= 5e-6 * diag


@pytest.mark.parametrize("path", [p for p in GOLD if "lp" in np.load(p).files],
                         ids=lambda p: os.path.basename(p)[4:-4])
def test_gather_and_backward_match_reference(oracle, path):
    """cwarp_cuda_gather_kernel.cu forward (checked through g) and the scale+scatter backward (dense [STU,V])."""
    z = np.load(path)
    lx, ly, y, V = z["lx"], z["ly"], z["y"], int(z["V"])
    g = oracle.gather(z["lp"].astype(np.float64), lx, ly, y, 0)
    assert np.array_equal(g.astype(np.float32), z["g"])
    dense = oracle.backward(z["grads"].astype(np.float64), z["grad_costs"].astype(np.float64), lx, ly, y, 0, V,
                            accumulate_equal=False)
    np.testing.assert_allclose(dense, z["dense"], rtol=2e-7, atol=1e-12)
