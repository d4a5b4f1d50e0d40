"""GPU tests of the analysis exports: best (Viterbi) alignment and node posteriors, through the C ABI, against the
CPU oracle (which is itself pinned to brute-force path enumeration in tests/test_oracle.py)."""
import numpy as np
import pytest
import torch

from compactwarprnntloss_b200 import capi
from tests.helpers import ragged_case

pytestmark = pytest.mark.gpu


def _rescore(g, off, T, U, moves):
    """Log-probability of a move sequence from gathered log-probs [STU,2], or None when it is not a valid path."""
    t = u = 0
    total = 0.0
    for k in moves:
        if t >= T or u > U or (k == 1 and u >= U):
            return None
        total += g[off + t * (U + 1) + u, int(k)]
        t, u = (t, u + 1) if k else (t + 1, u)
    return total if (t, u) == (T, U) else None


@pytest.mark.parametrize("shape", [(6, (1, 30), (0, 12), 9), (3, (40, 90), (30, 70), 16), (2, (20, 40), (500, 600), 8),
                                   (40, (1, 6), (0, 4), 5)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_best_alignment_against_oracle(oracle, shape, dtype):
    from tests.gpu_helpers import run_engine
    N, Tr, Ur, V = shape
    case = ragged_case(7 * N + V, N, Tr, Ur, V=V, sigma=1.5)
    out = run_engine(case, dtype=dtype, want_grad=False, keep=True)
    lx, ly = case["lx"], case["ly"]
    stride = int((lx + ly).max()) + 3
    moves, scores = capi.export_alignment(out["p"], out["lx"], out["ly"], out["ws"], stride)
    moves, scores = moves.cpu().numpy(), scores.double().cpu().numpy()
    g = oracle.gather(oracle.log_softmax(torch.as_tensor(case["x"]).to(dtype).double().numpy()), lx, ly, case["y"], 0)
    want_moves, want_scores = oracle.viterbi(g, lx, ly)
    off, _ = oracle.offsets(lx, ly)
    np.testing.assert_allclose(scores, want_scores, rtol=1e-5, atol=1e-5)
    same = 0
    for n in range(N):
        T, U = int(lx[n]), int(ly[n])
        mv = moves[n]
        assert np.all(mv[T + U:] == -1) and mv[T + U - 1] == 0 and int(mv[:T + U].sum()) == U
        got = _rescore(g, off[n], T, U, mv[:T + U])
        # a valid path whose probability is the best one's (a near-tie may be walked back the other way)
        assert got is not None and abs(got - want_scores[n]) <= 1e-5 * max(1.0, abs(want_scores[n]))
        same += int(np.array_equal(mv[:T + U], want_moves[n, :T + U]))
    assert same >= N - 1
    # the best path cannot be more probable than all paths together
    assert np.all(scores <= -out["costs"] + 1e-4 * np.abs(out["costs"]))


def test_alignment_after_a_costs_only_forward_and_argument_errors(oracle):
    from tests.gpu_helpers import run_engine
    case = ragged_case(3, 4, (5, 20), (1, 9), V=12)
    full = run_engine(case, want_grad=False, keep=True)
    only = run_engine(case, costs_only=True, keep=True)
    stride = int((case["lx"] + case["ly"]).max())
    a, sa = capi.export_alignment(full["p"], full["lx"], full["ly"], full["ws"], stride)
    b, sb = capi.export_alignment(only["p"], only["lx"], only["ly"], only["ws"], stride)
    assert torch.equal(a, b) and torch.equal(sa, sb)
    with pytest.raises(capi.CwrnntError):  # posteriors need alpha, which a costs-only forward does not keep
        capi.export_posteriors(only["p"], only["lx"], only["ly"], only["ws"], 20, 10)
    L = capi.lib()
    import ctypes
    rc = L.cwrnnt_export_alignment(ctypes.byref(full["p"]), full["lx"].data_ptr(), full["ly"].data_ptr(),
                                   full["ws"].data_ptr(), full["ws"].data_ptr(), 1, stride, a.data_ptr(),
                                   sa.data_ptr(), None)
    assert rc == 2  # scratch too small: refused before any launch


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_node_posteriors_against_oracle(oracle, dtype):
    from tests.gpu_helpers import run_engine
    case = ragged_case(19, 5, (2, 60), (0, 25), V=20, sigma=1.5)
    out = run_engine(case, dtype=dtype, want_grad=False, keep=True)
    lx, ly = case["lx"], case["ly"]
    Tm, Up = int(lx.max()) + 1, int(ly.max()) + 2
    post = capi.export_posteriors(out["p"], out["lx"], out["ly"], out["ws"], Tm, Up).double().cpu().numpy()
    g = oracle.gather(oracle.log_softmax(torch.as_tensor(case["x"]).to(dtype).double().numpy()), lx, ly, case["y"], 0)
    want = oracle.posteriors(g, lx, ly)
    off, _ = oracle.offsets(lx, ly)
    for n in range(5):
        T, m = int(lx[n]), int(ly[n]) + 1
        got = post[n, :T, :m]
        assert np.abs(got - want[off[n]:off[n] + T * m].reshape(T, m)).max() <= 1e-5
        assert np.all(post[n, T:] == 0) and np.all(post[n, :, m:] == 0)
        for d in range(T + m - 1):  # every alignment crosses each anti-diagonal exactly once
            s = sum(got[t, d - t] for t in range(T) if 0 <= d - t < m)
            assert abs(s - 1) <= 2e-5


def test_python_level_analysis(oracle):
    """`compactwarprnntloss_b200.analyse`: one call from compact logits to costs, best path, posteriors and padded
    alpha / beta; the emission frames derived from the path agree with the oracle's path."""
    from compactwarprnntloss_b200 import analyse
    case = ragged_case(29, 4, (5, 40), (1, 12), V=16, sigma=1.5)
    dev = "cuda:0"
    x = torch.as_tensor(case["x"]).to(dev)
    lx, ly = torch.as_tensor(case["lx"]).to(dev), torch.as_tensor(case["ly"]).to(dev)
    y = torch.as_tensor(case["y"]).to(dev)
    res = analyse(x, lx, y, ly, 0, fused_log_softmax=True, want_alpha_beta=True)
    g = oracle.gather(oracle.log_softmax(case["x"]), case["lx"], case["ly"], case["y"], 0)
    want_moves, want_scores = oracle.viterbi(g, case["lx"], case["ly"])
    fw = oracle.forward(g, case["lx"], case["ly"], want_ab=True)
    np.testing.assert_allclose(res.costs.cpu().numpy(), fw["costs"], rtol=1e-5)
    np.testing.assert_allclose(res.path_log_prob.cpu().numpy(), want_scores, rtol=1e-5, atol=1e-5)
    Tm, Up = int(case["lx"].max()), int(case["ly"].max()) + 1
    assert res.posteriors.shape == (4, Tm, Up) and res.alphas.shape == (4, Tm, Up)
    for n in range(4):
        T, U = int(case["lx"][n]), int(case["ly"][n])
        mv = want_moves[n, :T + U]
        want_frames = np.cumsum(mv == 0)[mv == 1]
        got_frames = res.emission_frames(n).cpu().numpy()
        assert got_frames.shape == (U,) and np.all(np.diff(got_frames) >= 0) and np.all(got_frames < T)
        if np.array_equal(res.moves[n, :T + U].cpu().numpy(), mv):
            assert np.array_equal(got_frames, want_frames)
        o = fw["offset"][n]
        np.testing.assert_allclose(res.alphas[n, :T, :U + 1].cpu().numpy(),
                                   fw["alpha"][o:o + T * (U + 1)].reshape(T, U + 1), rtol=1e-5, atol=1e-5)
        assert abs(float(res.posteriors[n, 0, 0]) - 1) < 1e-5 and abs(float(res.posteriors[n, T - 1, U]) - 1) < 1e-5
    with pytest.raises(ValueError):
        analyse(x[:-1], lx, y, ly, 0, fused_log_softmax=True)
