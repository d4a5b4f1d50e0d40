"""Pins the CPU checker (oracle/) before anything is compared against it.

Independent anchors: brute-force path enumeration, torchaudio's CPU rnnt_loss, central finite differences, and the
float32 "as the reference computes it" flavour against the double one.
"""
import numpy as np
import pytest
import torch

from tests.helpers import ragged_case


def _padded_from_compact(x, lx, ly, V):
    N, Tm, Um = len(lx), int(lx.max()), int(ly.max())
    out = np.zeros((N, Tm, Um + 1, V), dtype=x.dtype)
    at = 0
    for n in range(N):
        T, m = int(lx[n]), int(ly[n]) + 1
        out[n, :T, :m] = x[at:at + T * m].reshape(T, m, V)
        at += T * m
    return out


@pytest.mark.parametrize("T,U", [(1, 0), (1, 3), (4, 0), (2, 2), (4, 3), (5, 4), (3, 6)])
def test_costs_match_brute_force(oracle, T, U):
    c = ragged_case(100 + 10 * T + U, 1, (T, T), (U, U), V=5)
    lp = oracle.log_softmax(c["x"])
    g = oracle.gather(lp, c["lx"], c["ly"], c["y"], 0)
    fw = oracle.forward(g, c["lx"], c["ly"], want_ab=True)
    gb = g[:, 0].reshape(T, U + 1)
    gl = g[:, 1].reshape(T, U + 1)
    want = oracle.brute_force_cost(gb.tolist(), gl.tolist())
    assert abs(fw["costs"][0] - want) < 1e-10
    assert fw["mismatch"][0] == 0
    # alpha end == beta start
    a_end = fw["alpha"][-1] + g[-1, 0]
    assert abs(a_end - fw["beta"][0]) < 1e-10
    assert abs(oracle.costs_only(g, c["lx"], c["ly"])[0] - want) < 1e-10


def test_pair_gradients_are_derivatives(oracle):
    """grads[STU,2] returned by the forward are d cost / d gathered log-prob (central differences)."""
    c = ragged_case(7, 3, (2, 5), (0, 4), V=6)
    lp = oracle.log_softmax(c["x"])
    g = oracle.gather(lp, c["lx"], c["ly"], c["y"], 0)
    fw = oracle.forward(g, c["lx"], c["ly"])
    off = fw["offset"]
    eps = 1e-6
    for n in range(3):
        T, m = int(c["lx"][n]), int(c["ly"][n]) + 1
        for i in range(T * m):
            for col in range(2):
                if col == 1 and i % m == m - 1:
                    continue  # no label move out of the last column
                r = off[n] + i
                gp, gm = g.copy(), g.copy()
                gp[r, col] += eps
                gm[r, col] -= eps
                d = (oracle.costs_only(gp, c["lx"], c["ly"])[n] - oracle.costs_only(gm, c["lx"], c["ly"])[n]) / (2 * eps)
                assert abs(d - fw["grads"][r, col]) < 1e-7, (n, i, col)


def test_blank_gradient_zero_on_last_frame_off_corner(oracle):
    c = ragged_case(11, 2, (3, 4), (2, 3), V=4)
    g = oracle.gather(oracle.log_softmax(c["x"]), c["lx"], c["ly"], c["y"], 0)
    fw = oracle.forward(g, c["lx"], c["ly"])
    for n in range(2):
        T, m = int(c["lx"][n]), int(c["ly"][n]) + 1
        last = fw["grads"][fw["offset"][n] + (T - 1) * m: fw["offset"][n] + T * m]
        assert np.all(last[:-1, 0] == 0.0) and last[-1, 0] < 0
        assert last[-1, 1] == 0.0


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_fused_matches_torchaudio_cpu(oracle, seed):
    import torchaudio.functional as AF
    c = ragged_case(seed, 4, (3, 12), (1, 7), V=9, sigma=1.5)
    costs, dense = oracle.fused(c["x"], c["lx"], c["ly"], c["y"], 0)
    xp = torch.tensor(_padded_from_compact(c["x"], c["lx"], c["ly"], 9), requires_grad=True)
    loss = AF.rnnt_loss(xp, torch.tensor(c["y"]), torch.tensor(c["lx"]), torch.tensor(c["ly"]), blank=0,
                        reduction="none", fused_log_softmax=True)
    loss.sum().backward()
    np.testing.assert_allclose(costs, loss.detach().numpy(), rtol=2e-6, atol=2e-5)
    gp = _padded_from_compact(dense, c["lx"], c["ly"], 9)
    assert np.abs(gp - xp.grad.numpy()).max() < 5e-6


def test_fused_gradient_matches_autograd_through_log_softmax(oracle):
    """dense = chain rule of the reference's sparse gradient through torch.log_softmax, in double."""
    c = ragged_case(5, 3, (2, 9), (0, 5), V=7, sigma=2.0)
    w = np.array([0.3, -1.2, 2.0])
    costs, dense = oracle.fused(c["x"], c["lx"], c["ly"], c["y"], 0, weights=w)
    x = torch.tensor(c["x"], dtype=torch.float64, requires_grad=True)
    lp = torch.log_softmax(x, -1)
    g = oracle.gather(lp.detach().numpy(), c["lx"], c["ly"], c["y"], 0)
    fw = oracle.forward(g, c["lx"], c["ly"])
    sparse = oracle.backward(fw["grads"], w, c["lx"], c["ly"], c["y"], 0, 7, accumulate_equal=True)
    lp.backward(torch.tensor(sparse))
    np.testing.assert_allclose(costs, fw["costs"], rtol=0, atol=1e-11)
    assert np.abs(dense - x.grad.numpy()).max() < 1e-12
    # every dense row sums to zero (softmax Jacobian annihilates constants)
    assert np.abs(dense.sum(-1)).max() < 1e-12


def test_backward_scatter_assign_vs_accumulate(oracle):
    """The reference scatter assigns: a label equal to blank overwrites the blank term (gather kernel :70-73)."""
    c = ragged_case(3, 2, (2, 4), (1, 3), V=4, allow_blank_label=True)
    c["y"][:, 0] = 0  # force label == blank at u = 0
    g = oracle.gather(oracle.log_softmax(c["x"]), c["lx"], c["ly"], c["y"], 0)
    fw = oracle.forward(g, c["lx"], c["ly"])
    w = np.ones(2)
    ref = oracle.backward(fw["grads"], w, c["lx"], c["ly"], c["y"], 0, 4, accumulate_equal=False)
    acc = oracle.backward(fw["grads"], w, c["lx"], c["ly"], c["y"], 0, 4, accumulate_equal=True)
    r0 = fw["offset"][0]
    assert ref[r0, 0] == fw["grads"][r0, 1]
    assert acc[r0, 0] == fw["grads"][r0, 0] + fw["grads"][r0, 1]


def test_ref32_flavour_close_to_double(oracle):
    c = ragged_case(9, 5, (1, 70), (0, 40), V=3)  # the reference's own test uses V = 3
    g = oracle.gather(oracle.log_softmax(c["x"]), c["lx"], c["ly"], c["y"], 0)
    f64 = oracle.forward(g, c["lx"], c["ly"], want_ab=True)
    f32 = oracle.forward_ref32(g.astype(np.float32), c["lx"], c["ly"], want_ab=True)
    np.testing.assert_allclose(f32["costs"], f64["costs"], rtol=2e-5)
    assert np.abs(f32["grads"] - f64["grads"]).max() < 2e-3
    np.testing.assert_allclose(f32["alpha"], f64["alpha"], rtol=1e-4, atol=1e-3)


def test_offsets_and_empty_labels(oracle):
    lx = np.array([3, 1, 2], np.int32)
    ly = np.array([0, 0, 0], np.int32)  # U = 0 everywhere: the reference cannot launch this (Up-1 = 0 grid)
    off, rows = oracle.offsets(lx, ly)
    assert off.tolist() == [0, 3, 4] and rows == 6
    x = np.random.default_rng(0).standard_normal((6, 5))
    costs, dense = oracle.fused(x, lx, ly, np.zeros((3, 0), np.int32), 2)
    lp = oracle.log_softmax(x)
    assert abs(costs[0] + lp[0:3, 2].sum()) < 1e-12
    assert abs(costs[1] + lp[3, 2]) < 1e-12


def test_property_random_tiny_lattices_match_brute_force(oracle):
    """Property test over ragged shapes (hypothesis): double flavour == path enumeration, float flavour close."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=40, deadline=None)
    @given(T=st.integers(1, 5), U=st.integers(0, 4), V=st.integers(2, 6), seed=st.integers(0, 10 ** 6),
           blank=st.integers(0, 1))
    def run(T, U, V, seed, blank):
        c = ragged_case(seed, 1, (T, T), (U, U), V=V, blank=blank, allow_blank_label=True)
        lp = oracle.log_softmax(c["x"])
        g = oracle.gather(lp, c["lx"], c["ly"], c["y"], blank)
        fw = oracle.forward(g, c["lx"], c["ly"])
        want = oracle.brute_force_cost(g[:, 0].reshape(T, U + 1).tolist(), g[:, 1].reshape(T, U + 1).tolist())
        assert abs(fw["costs"][0] - want) < 1e-9
        f32 = oracle.forward_ref32(g.astype(np.float32), c["lx"], c["ly"])
        assert abs(f32["costs"][0] - want) < 1e-4 * max(1.0, abs(want))
        costs, dense = oracle.fused(c["x"], c["lx"], c["ly"], c["y"], blank)
        assert abs(costs[0] - want) < 1e-9 and np.abs(dense.sum(-1)).max() < 1e-12

    run()


@pytest.mark.parametrize("T,U", [(1, 0), (1, 3), (4, 0), (2, 2), (4, 3), (5, 4), (3, 6)])
def test_best_path_matches_enumeration(oracle, T, U):
    """The max-product recursion and its walk back against the most probable of all enumerated monotone paths."""
    c = ragged_case(300 + 10 * T + U, 1, (T, T), (U, U), V=5)
    g = oracle.gather(oracle.log_softmax(c["x"]), c["lx"], c["ly"], c["y"], 0)
    moves, scores = oracle.viterbi(g, c["lx"], c["ly"])
    want, want_moves = oracle.brute_force_best_path(g[:, 0].reshape(T, U + 1).tolist(),
                                                    g[:, 1].reshape(T, U + 1).tolist())
    assert abs(scores[0] - want) < 1e-12
    assert moves.shape == (1, T + U) and moves[0].tolist() == want_moves      # random reals: no ties
    assert moves[0, -1] == 0 and int(moves[0].sum()) == U
    # the best path is one of the summed paths: its probability cannot exceed the total
    assert scores[0] <= -oracle.costs_only(g, c["lx"], c["ly"])[0] + 1e-12


def test_best_paths_of_a_ragged_batch_are_padded_and_consistent(oracle):
    c = ragged_case(41, 6, (1, 30), (0, 12), V=9)
    g = oracle.gather(oracle.log_softmax(c["x"]), c["lx"], c["ly"], c["y"], 0)
    moves, scores = oracle.viterbi(g, c["lx"], c["ly"])
    off, _ = oracle.offsets(c["lx"], c["ly"])
    for n in range(6):
        T, U = int(c["lx"][n]), int(c["ly"][n])
        mv = moves[n]
        assert np.all(mv[T + U:] == -1) and set(mv[:T + U].tolist()) <= {0, 1}
        assert int(mv[:T + U].sum()) == U
        # re-score the path from the gathered log-probs
        t = u = 0
        total = 0.0
        for k in mv[:T + U]:
            r = off[n] + t * (U + 1) + u
            total += g[r, int(k)]
            t, u = (t, u + 1) if k else (t + 1, u)
        assert (t, u) == (T, U) and abs(total - scores[n]) < 1e-10


def test_node_posteriors_sum_to_one_on_every_diagonal(oracle):
    """Every alignment crosses each anti-diagonal t+u = d exactly once, so the node posteriors of a diagonal add up to
    one; the corner cells have posterior one."""
    c = ragged_case(43, 4, (2, 25), (0, 10), V=7)
    g = oracle.gather(oracle.log_softmax(c["x"]), c["lx"], c["ly"], c["y"], 0)
    post = oracle.posteriors(g, c["lx"], c["ly"])
    off, _ = oracle.offsets(c["lx"], c["ly"])
    for n in range(4):
        T, m = int(c["lx"][n]), int(c["ly"][n]) + 1
        p = post[off[n]:off[n] + T * m].reshape(T, m)
        assert abs(p[0, 0] - 1) < 1e-12 and abs(p[-1, -1] - 1) < 1e-12
        for d in range(T + m - 1):
            s = sum(p[t, d - t] for t in range(T) if 0 <= d - t < m)
            assert abs(s - 1) < 1e-10
