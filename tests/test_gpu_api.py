"""GPU tests of the reference-facing Python surface: `cwarp_rnnt.transducer_loss`, the `cwarp_rnnt._C` functions with
the reference's shapes, autograd, and - when oracle/_ref was built - the reference's own CUDA kernels run live on the
same inputs.

Bounds against the reference are triangle bounds: the reference computes alpha/beta in float32, and its own distance
to the double-precision truth grows with lattice size (4e-6 at 40 diagonals, 9e-4 at 330, see tests/test_golden.py);
this engine stays within 1e-5 of the truth, so |ours - ref| <= |ref - truth| + 1e-5.
"""
import glob
import os

import numpy as np
import pytest
import torch

from tests.helpers import ragged_case

pytestmark = pytest.mark.gpu
GOLD = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "ref_*.npz")))
DEV = "cuda:0"


def _tensors(case, dtype=torch.float32, x=None):
    x = torch.as_tensor(case["x"] if x is None else x).to(dtype).to(DEV)
    return (x, torch.as_tensor(case["lx"]).to(DEV), torch.as_tensor(case["y"]).to(DEV).contiguous(),
            torch.as_tensor(case["ly"]).to(DEV))


@pytest.mark.parametrize("reduction", ["mean", "sum", "none", None])
def test_drop_in_log_prob_contract(oracle, reduction):
    import cwarp_rnnt
    case = ragged_case(3, 5, (2, 25), (1, 10), V=12, sigma=1.5)
    lp = oracle.log_softmax(case["x"]).astype(np.float32)
    x, lx, y, ly = _tensors(case, x=lp)
    x.requires_grad_(True)
    out = cwarp_rnnt.transducer_loss(x, lx, y, ly, 0, reduction)
    g = oracle.gather(lp.astype(np.float64), case["lx"], case["ly"], case["y"], 0)
    fw = oracle.forward(g, case["lx"], case["ly"])
    if reduction in ("none", None):
        assert out.shape == (5,)
        np.testing.assert_allclose(out.detach().cpu().numpy(), fw["costs"], rtol=1e-5)
        w = torch.linspace(0.5, 2.0, 5, device=DEV)
        (out * w).sum().backward()
        weights = w.cpu().numpy().astype(np.float64)
    else:
        want = fw["costs"].mean() if reduction == "mean" else fw["costs"].sum()
        assert out.dim() == 0 and abs(float(out) - want) <= 1e-5 * abs(want)
        out.backward()
        weights = np.full(5, 1.0 / 5 if reduction == "mean" else 1.0)
    dense = oracle.backward(fw["grads"], weights, case["lx"], case["ly"], case["y"], 0, 12, accumulate_equal=True)
    assert np.abs(x.grad.cpu().numpy() - dense).max() <= 2e-5


def test_fused_equals_log_softmax_then_loss(oracle):
    """fused_log_softmax=True on logits == torch.log_softmax followed by the log-prob contract, loss and gradient."""
    import cwarp_rnnt
    case = ragged_case(8, 4, (3, 30), (0, 12), V=40, sigma=2.0)
    x, lx, y, ly = _tensors(case)
    a = x.clone().requires_grad_(True)
    b = x.clone().requires_grad_(True)
    la = cwarp_rnnt.transducer_loss(a, lx, y, ly, 0, "mean", fused_log_softmax=True, average_frames=True)
    lb = cwarp_rnnt.transducer_loss(torch.log_softmax(b, -1), lx, y, ly, 0, "mean", average_frames=True)
    la.backward()
    lb.backward()
    assert abs(float(la) - float(lb)) <= 1e-5 * abs(float(lb))
    assert (a.grad - b.grad).abs().max().item() <= 1e-5
    w = np.full(4, 0.25) / case["lx"]
    costs, dense = oracle.fused(case["x"], case["lx"], case["ly"], case["y"], 0, weights=w)
    assert abs(float(la) - (costs / case["lx"]).mean()) <= 1e-5 * abs(float(la))
    assert np.abs(a.grad.cpu().numpy() - dense).max() <= 1e-5


def test_no_grad_path_and_unchecked_path(oracle):
    import cwarp_rnnt
    case = ragged_case(13, 6, (2, 18), (1, 9), V=16)
    x, lx, y, ly = _tensors(case)
    costs, _ = oracle.fused(case["x"], case["lx"], case["ly"], case["y"], 0, want_grad=False)
    out = cwarp_rnnt.transducer_loss(x, lx, y, ly, 0, "none", fused_log_softmax=True)
    assert not out.requires_grad
    np.testing.assert_allclose(out.cpu().numpy(), costs, rtol=1e-5)
    out2 = cwarp_rnnt.transducer_loss(x, lx, y, ly, 0, "none", fused_log_softmax=True, check=False, gather=True)
    assert torch.equal(out, out2)


def test_padded_4d_input_is_compacted_per_sequence(oracle, capsys):
    import cwarp_rnnt
    case = ragged_case(17, 3, (4, 9), (1, 5), V=7)
    lx, ly = case["lx"], case["ly"]
    lx[0], ly[1] = 9, 5  # maxima attained, as the entry point asserts
    case = ragged_case(17, 3, (4, 9), (1, 5), V=7)
    case["lx"][0], case["ly"][1] = 9, 5
    N, T, Up, V = 3, 9, 6, 7
    rng = np.random.default_rng(0)
    xp = rng.standard_normal((N, T, Up, V)).astype(np.float32)
    y = rng.integers(1, V, size=(N, Up - 1)).astype(np.int32)
    rows = [xp[n, :case["lx"][n], :case["ly"][n] + 1].reshape(-1, V) for n in range(N)]
    compact = np.concatenate(rows)
    costs, _ = oracle.fused(compact, case["lx"], case["ly"], y, 0, want_grad=False)
    x4 = torch.tensor(xp, device=DEV, requires_grad=True)
    out = cwarp_rnnt.transducer_loss(x4, torch.tensor(case["lx"], device=DEV), torch.tensor(y, device=DEV),
                                     torch.tensor(case["ly"], device=DEV), 0, "sum", fused_log_softmax=True)
    assert "not compact" in capsys.readouterr().out
    assert abs(float(out) - costs.sum()) <= 1e-5 * costs.sum()
    out.backward()
    g = x4.grad.cpu().numpy()
    assert np.all(g[1, case["lx"][1]:] == 0) and np.abs(g[0, :case["lx"][0], :case["ly"][0] + 1]).max() > 0


def test_error_behaviour_matches_reference():
    import cwarp_rnnt
    case = ragged_case(19, 2, (3, 6), (1, 3), V=5)
    x, lx, y, ly = _tensors(case)
    with pytest.raises(AssertionError):
        cwarp_rnnt.transducer_loss(x, lx.long(), y, ly)          # lx must be int32   (reference __init__.py:41)
    with pytest.raises(AssertionError):
        cwarp_rnnt.transducer_loss(x, lx, y, ly, blank=5)        # blank < V          (reference __init__.py:50)
    with pytest.raises(AssertionError):
        cwarp_rnnt.transducer_loss(x, lx, y[:, :-1].contiguous(), ly)  # y.size(1) == ly.max()  (:49)
    with pytest.raises(AssertionError):
        cwarp_rnnt.transducer_loss(x, lx, y, ly, reduction="avg")
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        cwarp_rnnt.transducer_loss(x.cpu(), lx, y, ly)           # reference cwarp_cuda.cpp:46
    with pytest.raises(ValueError, match="rows"):
        cwarp_rnnt.transducer_loss(x[:-1].contiguous(), lx, y, ly)   # the reference would read out of bounds here
    with pytest.raises(TypeError):
        cwarp_rnnt.transducer_loss(x, lx, y, ly, 0, "mean", True)    # the extras are keyword-only


def test_gradcheck_double_fused():
    import cwarp_rnnt
    case = ragged_case(23, 2, (2, 4), (1, 3), V=4)
    x, lx, y, ly = _tensors(case, dtype=torch.float64)
    x.requires_grad_(True)
    f = lambda t: cwarp_rnnt.transducer_loss(t, lx, y, ly, 0, "none", fused_log_softmax=True, check=False)  # noqa: E731
    assert torch.autograd.gradcheck(f, (x,), eps=1e-6, atol=1e-6, rtol=1e-5, nondet_tol=0.0)


@pytest.mark.parametrize("path", GOLD, ids=[os.path.basename(p)[4:-4] for p in GOLD])
def test_extension_functions_against_golden_reference_outputs(oracle, path):
    """`cwarp_rnnt._C` with the reference's shapes on the inputs the reference itself was run on (fixtures)."""
    import cwarp_rnnt._C as core
    z = np.load(path)
    if "lp" not in z.files:
        pytest.skip("fixture stores the gathered pair only")
    lx, ly = torch.tensor(z["lx"], device=DEV), torch.tensor(z["ly"], device=DEV)
    y = torch.tensor(z["y"], device=DEV).contiguous()
    lp = torch.tensor(z["lp"], device=DEV)
    costs, grads, alphas, betas = core._cwarp_rnnt_forward(lp, lx, y, ly, 0)
    costs_only = core._cwarp_rnnt_loss(lp, lx, y, ly, 0)
    f64 = oracle.forward(z["g"].astype(np.float64), z["lx"], z["ly"])
    ref_err = np.abs(z["grads"] - f64["grads"]).max()
    assert costs.shape == z["costs"].shape and grads.shape == z["grads"].shape
    assert alphas.shape == z["alphas"].shape and betas.shape == z["betas"].shape
    np.testing.assert_allclose(costs.cpu().numpy(), z["costs"], rtol=1e-5)
    np.testing.assert_allclose(costs_only.cpu().numpy(), z["costs"], rtol=1e-5)
    assert np.abs(grads.cpu().numpy() - f64["grads"]).max() <= 1e-5
    assert np.abs(grads.cpu().numpy() - z["grads"]).max() <= ref_err + 1e-5
    scale = np.abs(z["costs"]).max()
    assert np.abs(alphas.cpu().numpy() - z["alphas"]).max() <= 2e-6 * scale
    assert np.abs(betas.cpu().numpy() - z["betas"]).max() <= 2e-6 * scale
    saved = grads.clone()
    dense = core._cwarp_rnnt_backward(grads, torch.tensor(z["grad_costs"], device=DEV), y, lx, ly, 0, int(z["V"]))
    assert torch.equal(grads, saved)  # not scaled in place, unlike the reference
    assert np.abs(dense.cpu().numpy() - z["dense"]).max() <= 2.0 * ref_err + 2e-5


def test_live_reference_cuda_kernels_when_built(oracle):
    """ours vs the reference's CUDA kernels (oracle/_ref, sm_100a build of its unmodified sources) on a Conformer-shape
    lattice: costs within 1e-5 relative; gradients within the reference's own float32 error + 1e-5.

    The reference's tile hand-over is racy on B200 (on large batches its own forward/backward guard fires and it returns
    a wrong cost for the affected sequence), so sequences on which the reference disagrees with the double oracle by
    more than 1e-4 relative are left out of the reference comparison; this engine is held to the oracle on all of them."""
    from oracle.build_ref import load_ref
    import cwarp_rnnt
    ref = load_ref()
    if ref is None:
        pytest.skip("oracle/_ref not built on this machine")
    case = ragged_case(29, 4, (150, 250), (20, 80), V=32, sigma=2.0)
    x, lx, y, ly = _tensors(case)
    a = x.clone().requires_grad_(True)
    lp = torch.log_softmax(a, -1)
    costs_r, grads_r, _, _ = ref._cwarp_rnnt_forward(lp.detach().contiguous(), lx, y, ly, 0)
    dense_r = ref._cwarp_rnnt_backward(grads_r.clone(), torch.full((4,), 0.25, device=DEV), y, lx, ly, 0, 32)
    lp.backward(dense_r)
    b = x.clone().requires_grad_(True)
    ours = cwarp_rnnt.transducer_loss(b, lx, y, ly, 0, "none", fused_log_softmax=True)
    (ours * 0.25).sum().backward()
    costs64, dense64 = oracle.fused(case["x"], case["lx"], case["ly"], case["y"], 0, weights=np.full(4, 0.25))
    np.testing.assert_allclose(ours.detach().cpu().numpy(), costs64, rtol=1e-5)
    our_err = np.abs(b.grad.cpu().numpy() - dense64).max()
    assert our_err <= 1e-5
    sane = np.abs(costs_r.cpu().numpy() - costs64) <= 1e-4 * np.abs(costs64)
    off = np.concatenate([[0], np.cumsum(case["lx"].astype(np.int64) * (case["ly"] + 1))])
    for n in np.nonzero(sane)[0]:
        rows = slice(off[n], off[n + 1])
        assert abs(float(ours[n]) - float(costs_r[n])) <= 1e-5 * abs(float(ours[n]))
        ref_err = np.abs(a.grad[rows].cpu().numpy() - dense64[rows]).max()
        assert (a.grad[rows] - b.grad[rows]).abs().max().item() <= ref_err + 1e-5
    print(f"|ours-f64| {our_err:.2e}; reference consistent on {int(sane.sum())} of 4 sequences")


def test_forward_backward_capture_in_a_cuda_graph(oracle):
    """The C-ABI calls allocate nothing and never synchronise, so a whole step can be captured once and replayed on
    new data of the same shapes (lengths included, since they live on the device)."""
    from compactwarprnntloss_b200 import capi
    case = ragged_case(37, 6, (4, 30), (1, 12), V=64, sigma=1.5)
    x, lx, y, ly = _tensors(case)
    p = capi.make_problem(x, lx, y, 0, capi.FUSED_LOG_SOFTMAX | capi.REDUCE_MEAN)
    ws = capi.alloc_workspace(p, x.device)
    costs = torch.empty(6, device=DEV)
    loss = torch.empty((), device=DEV)
    gx = torch.empty_like(x)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        capi.forward(p, x, lx, ly, y, ws, costs, loss)   # first use outside capture (module load, smem opt-in)
        capi.backward(p, x, lx, ly, y, ws, None, 0, gx)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            capi.forward(p, x, lx, ly, y, ws, costs, loss)
            capi.backward(p, x, lx, ly, y, ws, None, 0, gx)
    torch.cuda.synchronize()
    for seed in (1, 2):
        fresh = torch.randn(x.shape, generator=torch.Generator().manual_seed(seed)) * 1.5
        x.copy_(fresh.to(DEV))
        graph.replay()
        torch.cuda.synchronize()
        c64, d64 = oracle.fused(fresh.numpy(), case["lx"], case["ly"], case["y"], 0, weights=np.full(6, 1 / 6))
        np.testing.assert_allclose(costs.cpu().numpy(), c64, rtol=1e-5)
        assert abs(float(loss) - c64.mean()) <= 1e-5 * c64.mean()
        assert np.abs(gx.cpu().numpy() - d64).max() <= 1e-5


@pytest.mark.parametrize("dtype,V", [(torch.float32, 7), (torch.float32, 64), (torch.bfloat16, 40), (torch.float64, 6)])
def test_pack_and_unpack_padded_through_the_c_abi(dtype, V):
    """Padded [N,T,U+1,V] -> compact rows (x[n, :T_n, :U_n+1] per sequence, reference test/test.py:45-46) and the
    transpose used for the gradient, which zero-fills the padding. Bit-exact copies."""
    from compactwarprnntloss_b200 import capi
    rng = np.random.default_rng(V)
    N, T, Up = 5, 11, 6
    lx = rng.integers(1, T + 1, size=N).astype(np.int32)
    ly = rng.integers(0, Up, size=N).astype(np.int32)
    xp = torch.tensor(rng.standard_normal((N, T, Up, V))).to(dtype).to(DEV)
    want = torch.cat([xp[n, :lx[n], :ly[n] + 1].reshape(-1, V) for n in range(N)])
    got = capi.pack_padded(xp, torch.tensor(lx, device=DEV), torch.tensor(ly, device=DEV), want.shape[0])
    assert torch.equal(got, want)
    back = capi.unpack_padded(got, torch.tensor(lx, device=DEV), torch.tensor(ly, device=DEV), N, T, Up)
    for n in range(N):
        assert torch.equal(back[n, :lx[n], :ly[n] + 1], xp[n, :lx[n], :ly[n] + 1])
        assert back[n, lx[n]:].abs().sum() == 0 and back[n, :, ly[n] + 1:].abs().sum() == 0


def test_validate_reports_lengths_rows_labels_and_maxima():
    """cwrnnt_validate: the device-side facts behind the reference's host assertions, from one small kernel."""
    from compactwarprnntloss_b200 import capi
    case = ragged_case(5, 300, (1, 40), (0, 17), V=33)
    x, lx, y, ly = _tensors(case)
    p = capi.make_problem(x, lx, y, 0, capi.FUSED_LOG_SOFTMAX)
    assert capi.validate(p, lx, ly, y) == [0, -1, int(case["lx"].max()), int(case["ly"].max())]
    bad = y.clone()
    n = int(np.argmax(case["ly"]))
    bad[n, 0] = 33                                        # one label out of range, inside the used part of its row
    assert capi.validate(p, lx, ly, bad)[0] == capi.ST_BAD_LABEL
    bad = y.clone()
    short = int(np.argmin(case["ly"]))
    bad[short, int(case["ly"][short]):] = -7                # padding beyond ly[n] is never looked at
    assert capi.validate(p, lx, ly, bad)[0] == 0
    lx2 = lx.clone()
    lx2[7] = 0
    st = capi.validate(p, lx2, ly, y)
    assert st[0] & capi.ST_BAD_LENGTH and st[1] == 7 and st[0] & capi.ST_ROW_MISMATCH
    q = capi.make_problem(x[:-1], lx, y, 0, capi.FUSED_LOG_SOFTMAX)
    assert capi.validate(q, lx, ly, y)[0] == capi.ST_ROW_MISMATCH
