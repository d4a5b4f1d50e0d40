"""GPU parity: the CUDA engine, called through the C ABI, against the CPU oracle on the same seeded inputs.

Tolerances (float32 logits): |dloss|/loss <= 1e-5 and max|dgrad| <= 1e-5, the bounds stated for this engine against the
reference. Half-precision logits: costs are computed in float32 from the exactly-upcast inputs, so the same 1e-5
relative bound holds against the oracle on the upcast inputs; gradients are rounded to the storage type on the way out,
so they are allowed half an ulp of the storage type relative to the largest gradient (2^-8 for bfloat16, 2^-11 for
float16) on top of 1e-5.
"""
import numpy as np
import pytest
import torch

from tests.helpers import ragged_case

pytestmark = pytest.mark.gpu

LOSS_RTOL = 1e-5
GRAD_ATOL = 1e-5


def _upcast(case, dtype):
    c = dict(case)
    c["x"] = torch.as_tensor(case["x"]).to(dtype).double().numpy()
    return c


def _check_fused(oracle, case, dtype=torch.float32, **kw):
    from tests.gpu_helpers import run_engine
    got = run_engine(case, dtype=dtype, fused=True, **kw)
    up = _upcast(case, dtype)
    w = kw.get("grad_costs")
    B = len(case["lx"])
    weights = np.ones(B)
    if w is not None:
        weights = np.broadcast_to(np.asarray(w, dtype=np.float64), (B,)).copy()
    scale = np.ones(B)
    if kw.get("average_frames"):
        scale = 1.0 / case["lx"].astype(np.float64)
    den = kw.get("mean_denominator") or B
    if kw.get("reduce") == "mean":
        weights = weights / den
    costs, dense = oracle.fused(up["x"], case["lx"], case["ly"], case["y"], case["blank"], weights=weights * scale)
    costs = costs * scale
    assert got["status"][0] == 0, got["status"]
    np.testing.assert_allclose(got["costs"], costs, rtol=LOSS_RTOL, atol=1e-6)
    if kw.get("reduce") == "mean":
        assert abs(got["loss"] - costs.sum() / den) <= LOSS_RTOL * abs(costs.sum() / den) + 1e-6
    if kw.get("reduce") == "sum":
        assert abs(got["loss"] - costs.sum()) <= LOSS_RTOL * abs(costs.sum()) + 1e-6
    atol = GRAD_ATOL
    if dtype == torch.bfloat16:
        atol += 2.0 ** -8 * np.abs(dense).max()
    if dtype == torch.float16:
        atol += 2.0 ** -11 * np.abs(dense).max()
    err = np.abs(got["grad"] - dense).max()
    assert err <= atol, (err, atol)
    return got, costs, dense


@pytest.mark.parametrize("V", [3, 5, 8, 32, 64, 100, 128, 257, 512, 1024, 2048, 4100, 8192])
def test_fused_float32_vocab_sizes(oracle, V):
    case = ragged_case(V, 5, (1, 23), (0, 9), V=V, sigma=2.0)
    _check_fused(oracle, case, grad_costs=np.linspace(0.5, 1.5, 5))


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float64])
@pytest.mark.parametrize("V", [6, 64, 128, 1024, 4096, 8200])
def test_fused_other_dtypes(oracle, dtype, V):
    case = ragged_case(1000 + V, 4, (2, 17), (0, 8), V=V, sigma=1.5)
    _check_fused(oracle, case, dtype=dtype)


@pytest.mark.parametrize("reduce,avg", [("mean", False), ("sum", False), ("mean", True), (None, True)])
def test_reductions_and_average_frames(oracle, reduce, avg):
    case = ragged_case(77, 6, (3, 30), (1, 12), V=64)
    _check_fused(oracle, case, reduce=reduce, average_frames=avg, grad_costs=1.7 if reduce else None)
    _check_fused(oracle, case, reduce=reduce, average_frames=avg, mean_denominator=24 if reduce == "mean" else 0)


def test_edge_shapes(oracle):
    # U = 0 for every sequence (the reference cannot launch this: zero-sized grid), T = 1, single cell, blank != 0,
    # a label equal to blank
    c = ragged_case(5, 4, (1, 9), (0, 0), V=16)
    _check_fused(oracle, c)
    c = ragged_case(6, 3, (1, 1), (0, 7), V=16)
    _check_fused(oracle, c)
    c = ragged_case(7, 1, (1, 1), (0, 0), V=4)
    _check_fused(oracle, c)
    c = ragged_case(8, 4, (2, 11), (1, 6), V=24, blank=23)
    _check_fused(oracle, c)
    c = ragged_case(9, 4, (2, 11), (1, 6), V=12, blank=3, allow_blank_label=True)
    c["y"][:, 0] = 3
    _check_fused(oracle, c)


@pytest.mark.parametrize("T,U", [(40, 31), (33, 32), (5, 200), (300, 70), (12, 511), (30, 700), (64, 1030), (20, 2100)])
def test_wide_and_long_lattices(oracle, T, U):
    """Column counts that cross warp seams (32), the split-role kernel's limit (512 columns), the one-column-per-thread
    limit (1024 -> 4 columns per thread) and 2048 (8 per thread)."""
    case = ragged_case(T * 7 + U, 2, (T - 3, T), (U - 2, U), V=8, sigma=1.0)
    _check_fused(oracle, case)


@pytest.mark.parametrize("T", [1, 2, 3, 4, 5, 8, 13, 16, 17, 31, 64])
@pytest.mark.parametrize("U", [161, 255, 256, 330, 511])
def test_wide_lattices_round_boundaries(oracle, T, U):
    """Launches wider than 160 columns run the wavefront in rounds of four steps over a 16-slot operand ring and 8
    result rows. The number of diagonals T+U takes every residue of 4 and 16 here, with fewer frames than one round, one
    frame, and a narrow sequence (one warp) beside the wide one in the same launch."""
    rng = np.random.default_rng(T * 1000 + U)
    lx = np.array([T, max(1, T - 1), T], dtype=np.int32)
    ly = np.array([U, 7, U - 33], dtype=np.int32)
    V = 6
    y = rng.integers(1, V, size=(3, U)).astype(np.int32)
    rows = int((lx.astype(np.int64) * (ly + 1)).sum())
    case = dict(x=rng.standard_normal((rows, V)).astype(np.float32), lx=lx, ly=ly, y=y, blank=0, V=V)
    _check_fused(oracle, case)


def test_long_form_sequence_against_oracle(oracle):
    """One sequence of the long-form workload's size (T=1200, U=300, V=512: 1900 diagonals, 301 columns = 10 compute
    and 10 helper warps in the wavefront kernel)."""
    case = ragged_case(4, 1, (1200, 1200), (300, 300), V=512, sigma=1.0)
    _check_fused(oracle, case, reduce="mean")


def test_empty_batch_and_tiny_batches_launch_nothing_harmful():
    from compactwarprnntloss_b200 import capi
    dev = torch.device("cuda:0")
    x = torch.zeros(0, 8, device=dev)
    lx = torch.zeros(0, dtype=torch.int32, device=dev)
    y = torch.zeros(0, 0, dtype=torch.int32, device=dev)
    p = capi.make_problem(x, lx, y, 0, capi.FUSED_LOG_SOFTMAX)
    ws = capi.alloc_workspace(p, dev)
    costs = torch.zeros(1, device=dev)
    capi.forward(p, x, lx, lx, y, ws, costs)           # B = 0: accepted, nothing to do
    capi.backward(p, x, lx, lx, y, ws, None, 0, x)
    torch.cuda.synchronize()


def test_many_sequences_order_and_cursor(oracle):
    case = ragged_case(31, 300, (1, 12), (0, 6), V=8)
    _check_fused(oracle, case, reduce="mean")
    # more sequences than the longest-first sort handles (4096): identity order, 9000 wavefront CTAs
    case = ragged_case(32, 4500, (1, 4), (0, 3), V=4)
    _check_fused(oracle, case, reduce="sum")


def test_thousands_of_tiny_lattices_repeatedly(oracle):
    """One- to sixteen-cell lattices, thousands of short-lived wavefront CTAs per launch: the schedule in which a helper
    warp can get ahead of its compute warp. The first operands of a direction must be taken out of the staging ring
    before the helper's first refill (a race here showed as a wrong beta(0,0) in a few of 4500 sequences per launch)."""
    from compactwarprnntloss_b200 import capi
    B = 4500
    case = ragged_case(32, B, (1, 4), (0, 3), V=4)
    want, _ = oracle.fused(case["x"], case["lx"], case["ly"], case["y"], 0, want_grad=False)
    dev = torch.device("cuda:0")
    x = torch.as_tensor(case["x"]).to(dev)
    lx, ly = torch.as_tensor(case["lx"]).to(dev), torch.as_tensor(case["ly"]).to(dev)
    y = torch.as_tensor(case["y"]).to(dev).contiguous()
    p = capi.make_problem(x, lx, y, 0, capi.FUSED_LOG_SOFTMAX)
    for rep in range(10):
        ws = capi.alloc_workspace(p, dev)
        if rep % 2:
            ws.fill_(0xFF)  # NaN patterns wherever nothing is written
        costs = torch.empty(B, device=dev)
        capi.forward(p, x, lx, ly, y, ws, costs, None)
        assert capi.read_status(ws)[0] == 0, rep
        np.testing.assert_allclose(costs.cpu().numpy(), want, rtol=LOSS_RTOL, atol=1e-6, err_msg=f"launch {rep}")


def test_costs_only_matches_full(oracle):
    from tests.gpu_helpers import run_engine
    case = ragged_case(12, 7, (2, 40), (0, 25), V=48)
    full = run_engine(case, want_grad=False)
    only = run_engine(case, costs_only=True)
    np.testing.assert_allclose(only["costs"], full["costs"], rtol=1e-7)
    costs, _ = oracle.fused(case["x"], case["lx"], case["ly"], case["y"], 0, want_grad=False)
    np.testing.assert_allclose(only["costs"], costs, rtol=LOSS_RTOL)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.float64])
def test_wide_lattices_costs_only_and_other_dtypes(oracle, dtype):
    """The wide-lattice wavefront (rounds for float-type inputs, the per-diagonal barrier for double) with 16-bit and
    double inputs, and with beta-only CTAs (costs without gradients): 200 to 340 columns beside a narrow sequence."""
    from tests.gpu_helpers import run_engine
    case = ragged_case(91, 4, (9, 60), (200, 339), V=16)
    case["ly"][1] = 5
    rows = int((case["lx"].astype(np.int64) * (case["ly"] + 1)).sum())
    case["x"] = np.random.default_rng(5).standard_normal((rows, 16)).astype(np.float32)
    _check_fused(oracle, case, dtype=dtype)
    up = _upcast(case, dtype)
    only = run_engine(case, dtype=dtype, costs_only=True)
    costs, _ = oracle.fused(up["x"], case["lx"], case["ly"], case["y"], 0, want_grad=False)
    np.testing.assert_allclose(only["costs"], costs, rtol=LOSS_RTOL, atol=1e-6)


def test_recursion_alone_on_a_gathered_workspace(oracle):
    """cwrnnt_recursion re-runs the alpha/beta wavefront and the cost step on the state a forward left behind: costs
    and loss come out bit-identical, with and without the alpha direction, and a backward may still follow."""
    from compactwarprnntloss_b200 import capi
    from tests.gpu_helpers import run_engine
    case = ragged_case(14, 9, (3, 70), (0, 40), V=24)
    out = run_engine(case, reduce="mean", keep=True)
    p, ws = out["p"], out["ws"]
    costs = torch.full((p.B,), float("nan"), device="cuda:0")
    loss = torch.full((), float("nan"), device="cuda:0")
    capi.recursion(p, out["lx"], out["ly"], ws, costs, loss)
    assert np.array_equal(costs.double().cpu().numpy(), out["costs"]) and float(loss) == out["loss"]
    gx = torch.empty_like(out["x"])
    capi.backward(p, out["x"], out["lx"], out["ly"], out["y"], ws, None, 0, gx)
    assert np.array_equal(gx.double().cpu().numpy(), out["grad"])
    q = capi.make_problem(out["x"], out["lx"], out["y"], 0, capi.FUSED_LOG_SOFTMAX | capi.COSTS_ONLY)
    costs.fill_(float("nan"))
    capi.recursion(q, out["lx"], out["ly"], ws, costs, None)       # beta only
    np.testing.assert_allclose(costs.double().cpu().numpy(), out["costs"], rtol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_log_prob_mode_is_reference_contract(oracle, dtype):
    """x = log-probs: costs, sparse dense-shaped gradient, pair gradients and padded alpha/beta as the reference."""
    from compactwarprnntloss_b200 import capi
    from tests.gpu_helpers import run_engine
    case = ragged_case(21, 5, (2, 21), (1, 9), V=10, sigma=1.3)
    lp = oracle.log_softmax(case["x"])
    c2 = dict(case, x=lp)
    gc = np.array([1.0, 0.5, -2.0, 3.0, 0.25])
    got = run_engine(c2, dtype=dtype, fused=False, grad_costs=gc, keep=True)
    g = oracle.gather(torch.as_tensor(lp).to(dtype).double().numpy(), case["lx"], case["ly"], case["y"], 0)
    fw = oracle.forward(g, case["lx"], case["ly"], want_ab=True)
    np.testing.assert_allclose(got["costs"], fw["costs"], rtol=LOSS_RTOL)
    dense = oracle.backward(fw["grads"], gc, case["lx"], case["ly"], case["y"], 0, 10, accumulate_equal=True)
    assert np.abs(got["grad"] - dense).max() <= 3 * GRAD_ATOL  # |g_n| up to 3
    # pair gradients [STU,2]
    ct = capi.cost_dtype(dtype)
    pg = torch.empty(lp.shape[0], 2, dtype=ct, device="cuda:0")
    capi.pair_grads(got["p"], got["x"], got["lx"], got["ly"], got["y"], got["ws"], pg)
    assert np.abs(pg.double().cpu().numpy() - fw["grads"]).max() <= GRAD_ATOL
    # padded alphas / betas [N, Tmax, Umax+1]
    Tm, Up = int(case["lx"].max()), int(case["ly"].max()) + 1
    al = torch.full((5, Tm, Up), 7.0, dtype=ct, device="cuda:0")
    be = torch.full((5, Tm, Up), 7.0, dtype=ct, device="cuda:0")
    capi.export_alpha_beta(got["p"], got["lx"], got["ly"], got["ws"], Tm, Up, al, be)
    al, be = al.double().cpu().numpy(), be.double().cpu().numpy()
    for n in range(5):
        T, m = int(case["lx"][n]), int(case["ly"][n]) + 1
        o = fw["offset"][n]
        np.testing.assert_allclose(al[n, :T, :m], fw["alpha"][o:o + T * m].reshape(T, m), rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(be[n, :T, :m], fw["beta"][o:o + T * m].reshape(T, m), rtol=1e-5, atol=1e-5)
        assert np.all(al[n, T:] == 0) and np.all(al[n, :, m:] == 0) and np.all(be[n, T:] == 0)
    # reference-shaped backward from saved pair gradients
    dn = torch.full((lp.shape[0], 10), 9.0, dtype=ct, device="cuda:0")
    capi.scatter_backward(got["p"], pg, torch.as_tensor(gc).to(ct).cuda(), got["lx"], got["ly"], got["y"], dn)
    assert np.abs(dn.double().cpu().numpy() - dense).max() <= 3 * GRAD_ATOL


def test_status_words_flag_bad_inputs(oracle):
    from compactwarprnntloss_b200 import capi
    from tests.gpu_helpers import run_engine
    case = ragged_case(41, 3, (2, 6), (1, 4), V=8)
    bad = dict(case, lx=case["lx"].copy())
    bad["lx"][1] += 1  # rows no longer add up
    out = run_engine(bad, want_grad=False)
    assert out["status"][0] & capi.ST_ROW_MISMATCH and np.all(np.isnan(out["costs"]))
    bad = dict(case, lx=case["lx"].copy())
    bad["lx"][2] = 0
    out = run_engine(bad, want_grad=False)
    assert out["status"][0] & capi.ST_BAD_LENGTH and out["status"][1] == 2
    bad = dict(case, y=case["y"].copy())
    bad["y"][0, 0] = 99
    out = run_engine(bad, want_grad=False)
    assert out["status"][0] == capi.ST_BAD_LABEL and np.all(np.isfinite(out["costs"]))
    # argument errors never reach the device
    x = torch.zeros(4, 8, device="cuda:0")
    lx = torch.tensor([2], dtype=torch.int32, device="cuda:0")
    y = torch.zeros(1, 1, dtype=torch.int32, device="cuda:0")
    p = capi.make_problem(x, lx, y, blank=8, flags=0)
    assert capi.lib().cwrnnt_workspace_bytes(p) < 0
    p = capi.make_problem(x, lx, y, blank=0, flags=0, max_u=capi.MAX_COLUMNS)
    p.y_stride = capi.MAX_COLUMNS
    with pytest.raises(capi.CwrnntError):
        capi.forward(p, x, lx, lx, y, torch.empty(1 << 20, dtype=torch.uint8, device="cuda:0"),
                     torch.empty(1, device="cuda:0"))


def test_backward_is_repeatable_and_linear(oracle):
    """The saved state is never modified (the reference scales it in place): two backwards agree, and scale linearly."""
    from tests.gpu_helpers import run_engine
    from compactwarprnntloss_b200 import capi
    case = ragged_case(51, 4, (3, 20), (1, 9), V=64)
    out = run_engine(case, keep=True)
    g1 = torch.empty_like(out["x"])
    g2 = torch.empty_like(out["x"])
    two = torch.tensor([2.0], device="cuda:0")
    capi.backward(out["p"], out["x"], out["lx"], out["ly"], out["y"], out["ws"], None, 0, g1)
    capi.backward(out["p"], out["x"], out["lx"], out["ly"], out["y"], out["ws"], two, 0, g2)
    assert torch.equal(g1.cpu(), torch.as_tensor(out["grad"]).float())
    assert torch.allclose(g2, 2 * g1, rtol=1e-6, atol=1e-9)
    # rows of the logit gradient sum to zero
    assert g1.double().sum(-1).abs().max().item() < 1e-5


@pytest.mark.parametrize("cfg", [1, 2, 3, 4, 5])
def test_benchmark_shapes_properties(oracle, cfg):
    """The five benchmark workloads exactly as `synth` generates them (1: tiny; 2: Conformer V=1024 fp32; 3: V=4096
    bf16, reduction sum; 4: long-form, one 1000+ frame sequence; 5: ragged fp16): the leading sequences of each - as
    many as the oracle finishes in seconds - against the oracle, plus the zero row sum of the logit gradient."""
    from compactwarprnntloss_b200 import synth
    from tests.gpu_helpers import run_engine
    lx, ly, y = synth.lengths_and_labels(cfg)
    B = {1: 4, 2: 6, 3: 2, 4: 1, 5: 48}[cfg]
    wl = synth.WORKLOADS[cfg]
    ids = list(range(B))
    x = synth.compact_logits(cfg, lx, ly, ids)
    case = dict(x=x.numpy() if x.dtype == torch.float32 else x, lx=lx[:B].numpy(), ly=ly[:B].numpy(),
                y=y[:B].numpy(), blank=0, V=x.shape[1])
    dtype = wl.dtype
    got = run_engine(case, dtype=dtype, reduce=wl.reduction)
    xd = x.double().numpy()
    w = np.full(B, 1.0 / B if wl.reduction == "mean" else 1.0)
    costs, dense = oracle.fused(xd, case["lx"], case["ly"], case["y"], 0, weights=w)
    assert got["status"][0] == 0
    np.testing.assert_allclose(got["costs"], costs, rtol=LOSS_RTOL)
    want_loss = costs.mean() if wl.reduction == "mean" else costs.sum()
    assert abs(got["loss"] - want_loss) <= LOSS_RTOL * abs(want_loss)
    half_ulp = {torch.float32: 0.0, torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8}[dtype]
    assert np.abs(got["grad"] - dense).max() <= GRAD_ATOL + half_ulp * np.abs(dense).max()
    row_sum = {torch.float32: 1e-4, torch.float16: 2e-2, torch.bfloat16: 5e-2}[dtype]
    assert np.abs(got["grad"].sum(-1)).max() < row_sum


def test_reference_test_generator_shape(oracle):
    """The shape the reference's own test draws (test/test.py:10-25): fewer than 20 sequences, up to 511 frames, up to
    512 labels, V = 3, the longest sequence reaching the padded sizes. Here with 12 sequences, T up to 300 and U up to
    512, so that the 513-column lattice takes the single-role wavefront kernel while the 3-element rows take the
    scalar (unaligned vocabulary) streaming kernels - the two paths no benchmark workload touches together."""
    rng = np.random.default_rng(0)
    N, T, U, V = 12, 300, 512, 3
    lx = rng.integers(T // 2, T + 1, size=N).astype(np.int32)
    ly = rng.integers(U // 2, U + 1, size=N).astype(np.int32)
    lx += T - lx.max()
    ly += U - ly.max()
    y = rng.integers(1, V, size=(N, U)).astype(np.int32)
    rows = int((lx.astype(np.int64) * (ly + 1)).sum())
    case = dict(x=rng.standard_normal((rows, V)).astype(np.float32), lx=lx, ly=ly, y=y, blank=0, V=V)
    _check_fused(oracle, case, reduce="mean")
    # and as the reference is called: log-probabilities in, sparse gradient out
    from tests.gpu_helpers import run_engine
    lp = oracle.log_softmax(case["x"])
    got = run_engine(dict(case, x=lp), fused=False)
    g = oracle.gather(lp, lx, ly, y, 0)
    fw = oracle.forward(g, lx, ly)
    np.testing.assert_allclose(got["costs"], fw["costs"], rtol=LOSS_RTOL)
    dense = oracle.backward(fw["grads"], np.ones(N), lx, ly, y, 0, V, accumulate_equal=True)
    assert np.abs(got["grad"] - dense).max() <= GRAD_ATOL


def test_forward_backward_guard(oracle):
    """The reference's only consistency check (cwarp_cuda_rnnt_kernel.cu:350-366): alpha's and beta's log-likelihood of
    a sequence more than 1e-3 apart (relative) -> their mean is the cost's log-likelihood and the status word gets
    CWRNNT_ST_FWD_BWD_GAP. Driven through cwrnnt_fill_costs, which runs the same device function as the wavefront
    kernel's epilogue, on hand-made log-likelihoods."""
    from compactwarprnntloss_b200 import capi
    dev = torch.device("cuda:0")
    lx = torch.tensor([10, 20, 30, 40], dtype=torch.int32, device=dev)
    la = torch.tensor([-100.0, -100.0, -50.0, -7.0], dtype=torch.float64, device=dev)
    lb = torch.tensor([-100.05, -100.2, -50.0, -7.0000001], dtype=torch.float64, device=dev)
    p = capi.Problem(0, 4, 4, 0, 0, 0, capi.F32, 0, 0)
    costs = torch.zeros(4, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    capi.fill_costs(p, lx, la, lb, costs, status)
    # |a-b|/|max| = 5e-4 (kept: beta), 2e-3 (mean), 0, 1.4e-8
    np.testing.assert_allclose(costs.cpu().numpy(), [100.05, 100.1, 50.0, 7.0000001], rtol=2e-7)
    assert int(status[0]) == capi.ST_FWD_BWD_GAP
    status.zero_()
    q = capi.Problem(0, 4, 2, 0, 0, 0, capi.F64, capi.AVERAGE_FRAMES, 0)
    c64 = torch.zeros(2, dtype=torch.float64, device=dev)
    capi.fill_costs(q, lx[2:], la[2:], lb[2:], c64, status)
    np.testing.assert_allclose(c64.cpu().numpy(), [50.0 / 30, 7.0000001 / 40], rtol=1e-12)
    assert int(status[0]) == 0
    capi.fill_costs(q, lx[:2], None, lb[:2], c64, status)           # no alpha: no guard (costs-only path)
    np.testing.assert_allclose(c64.cpu().numpy(), [100.05 / 10, 100.2 / 20], rtol=1e-12)
    assert int(status[0]) == 0
    # a real forward on a consistent lattice never raises the bit
    from tests.gpu_helpers import run_engine
    out = run_engine(ragged_case(3, 6, (5, 60), (1, 20), V=32), want_grad=False)
    assert not out["status"][0] & capi.ST_FWD_BWD_GAP


def test_sharded_forward_fills_global_cost_vector(oracle):
    """Two shards of one batch, run one after the other on one GPU: each fills its own slots of the cost vector and
    zeroes the rest, so the sum of the two vectors (what the all-reduce computes) is every cost plus the mean loss."""
    from compactwarprnntloss_b200 import capi, sharding
    case = ragged_case(71, 7, (3, 25), (1, 9), V=32)
    costs64, _ = oracle.fused(case["x"], case["lx"], case["ly"], case["y"], 0, want_grad=False)
    plan = sharding.plan_shards(case["lx"], case["ly"], 2)
    off = np.concatenate([[0], np.cumsum(case["lx"].astype(np.int64) * (case["ly"] + 1))])
    total = torch.zeros(8, device="cuda:0")
    for ids in plan:
        rows = np.concatenate([np.arange(off[i], off[i + 1]) for i in ids])
        x = torch.as_tensor(case["x"][rows]).cuda().contiguous()
        lx = torch.as_tensor(case["lx"][ids]).cuda()
        ly = torch.as_tensor(case["ly"][ids]).cuda()
        y = torch.as_tensor(case["y"][ids]).cuda().contiguous()
        p = capi.make_problem(x, lx, y, 0, capi.FUSED_LOG_SOFTMAX | capi.REDUCE_MEAN, mean_denominator=7)
        ws = capi.alloc_workspace(p, x.device)
        costs = torch.empty(len(ids), device="cuda:0")
        loss = torch.empty((), device="cuda:0")
        vec = torch.full((8,), float("nan"), device="cuda:0")
        capi.forward_sharded(p, x, lx, ly, y, ws, costs, loss, torch.tensor(ids, dtype=torch.int32, device="cuda:0"),
                             7, vec)
        v = vec.cpu().numpy()
        others = [i for i in range(7) if i not in ids]
        assert np.all(v[others] == 0.0)
        np.testing.assert_allclose(v[ids], costs.cpu().numpy(), rtol=0)
        assert abs(v[7] - float(loss)) == 0.0
        total += vec
    np.testing.assert_allclose(total[:7].cpu().numpy(), costs64, rtol=LOSS_RTOL)
    assert abs(float(total[7]) - costs64.mean()) <= LOSS_RTOL * costs64.mean()


def test_host_pipeline_matches_device_path(oracle):
    from compactwarprnntloss_b200 import capi
    from tests.gpu_helpers import run_engine
    case = ragged_case(61, 9, (5, 40), (1, 12), V=128, sigma=2.0)
    dev = run_engine(case, reduce="mean", grad_costs=0.5)
    x = torch.as_tensor(case["x"]).pin_memory()
    gx = torch.empty_like(x).pin_memory()
    pipe = capi.HostPipeline(0)
    costs, loss, st = pipe.run(x, torch.as_tensor(case["lx"]), torch.as_tensor(case["ly"]), torch.as_tensor(case["y"]),
                               flags=capi.FUSED_LOG_SOFTMAX | capi.REDUCE_MEAN, grad_costs=torch.tensor([0.5]),
                               grad_x=gx, chunk_rows=600)  # forces several chunks
    pipe.close()
    assert st[0] == 0
    np.testing.assert_allclose(costs.numpy(), dev["costs"], rtol=1e-6)
    assert abs(float(loss) - dev["loss"]) < 1e-5 * abs(dev["loss"])
    assert np.abs(gx.numpy() - dev["grad"]).max() < 1e-7


def test_more_than_2_31_elements_bf16(oracle):
    """V=4096 bfloat16, 2.2 G elements (the reference's 32-bit accessors reject such a tensor): row offsets and element
    indices are 64-bit. The first and the last sequence (whose rows lie beyond element 2^31) are checked against the
    oracle; the rest through the zero row-sum property of the logit gradient."""
    from compactwarprnntloss_b200 import capi
    dev = torch.device("cuda:0")
    V, B = 4096, 12
    rng = np.random.default_rng(5)
    lx = rng.integers(300, 501, size=B).astype(np.int32)
    ly = rng.integers(100, 151, size=B).astype(np.int32)
    rows = int((lx.astype(np.int64) * (ly + 1)).sum())
    while rows * V <= 2 ** 31 + 2 ** 27:
        lx = lx + 20
        rows = int((lx.astype(np.int64) * (ly + 1)).sum())
    y = rng.integers(1, V, size=(B, int(ly.max()))).astype(np.int32)
    g = torch.Generator(device=dev).manual_seed(7)
    x = (torch.randn(rows, V, device=dev, generator=g) * 3.0).to(torch.bfloat16)
    lxd, lyd, yd = torch.tensor(lx, device=dev), torch.tensor(ly, device=dev), torch.tensor(y, device=dev)
    p = capi.make_problem(x, lxd, yd, 0, capi.FUSED_LOG_SOFTMAX | capi.REDUCE_SUM)
    ws = capi.alloc_workspace(p, dev)
    costs = torch.empty(B, device=dev)
    loss = torch.empty((), device=dev)
    gx = torch.empty_like(x)
    capi.forward(p, x, lxd, lyd, yd, ws, costs, loss)
    capi.backward(p, x, lxd, lyd, yd, ws, None, 0, gx)
    assert capi.read_status(ws)[0] == 0
    off = np.concatenate([[0], np.cumsum(lx.astype(np.int64) * (ly + 1))])
    assert off[-1] * V > 2 ** 31
    for n in (0, B - 1):
        xs = x[off[n]:off[n + 1]].double().cpu().numpy()
        c64, d64 = oracle.fused(xs, lx[n:n + 1], ly[n:n + 1], y[n:n + 1], 0)
        assert abs(float(costs[n]) - c64[0]) <= LOSS_RTOL * c64[0]
        got = gx[off[n]:off[n + 1]].double().cpu().numpy()
        assert np.abs(got - d64).max() <= GRAD_ATOL + 2.0 ** -8 * np.abs(d64).max()
    assert abs(float(loss) - float(costs.double().sum())) <= 1e-5 * float(loss)
    # every row of the logit gradient sums to ~0 (bf16 rounding of 4096 terms), sampled across the whole tensor
    idx = torch.linspace(0, rows - 1, 4096, device=dev).long()
    assert gx[idx].double().sum(-1).abs().max().item() < 0.05
