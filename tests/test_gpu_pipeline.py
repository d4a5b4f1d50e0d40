"""GPU tests of the pipelined single-call step (cwrnnt_loss_grad): sequence groups, side streams, device-side group
bounds. The pipelined call runs the same kernels on the same data as cwrnnt_forward + cwrnnt_backward, only cut into
groups and overlapped, so every result must be BIT-identical to that pair's, for any number of groups."""
import numpy as np
import pytest
import torch

from compactwarprnntloss_b200 import capi
from tests.helpers import ragged_case

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.fixture(scope="module")
def pipe():
    p = capi.Pipe(DEV)
    yield p
    p.close()


def _setup(case, dtype=torch.float32, flags=capi.FUSED_LOG_SOFTMAX | capi.REDUCE_MEAN, mean_denominator=0):
    x = torch.as_tensor(case["x"]).to(dtype).to(DEV).contiguous()
    lx = torch.as_tensor(case["lx"], dtype=torch.int32).to(DEV)
    ly = torch.as_tensor(case["ly"], dtype=torch.int32).to(DEV)
    y = torch.as_tensor(case["y"], dtype=torch.int32).to(DEV).contiguous()
    p = capi.make_problem(x, lx, y, case["blank"], flags, mean_denominator)
    return p, x, lx, ly, (y if y.numel() else None)


def _two_calls(p, x, lx, ly, y, gc=None, stride=0):
    ct = capi.cost_dtype(x.dtype)
    ws = capi.alloc_workspace(p, DEV)
    costs = torch.full((p.B,), float("nan"), dtype=ct, device=DEV)
    loss = torch.full((), float("nan"), dtype=ct, device=DEV)
    gx = torch.full_like(x, float("nan"))
    capi.forward(p, x, lx, ly, y, ws, costs, loss)
    capi.backward(p, x, lx, ly, y, ws, gc, stride, gx)
    torch.cuda.synchronize()
    return costs, loss, gx


def _one_call(pipe, p, x, lx, ly, y, groups, gc=None, stride=0, **shard):
    ct = capi.cost_dtype(x.dtype)
    ws = capi.alloc_workspace(p, DEV)
    costs = torch.full((p.B,), float("nan"), dtype=ct, device=DEV)
    loss = torch.full((), float("nan"), dtype=ct, device=DEV)
    gx = torch.full_like(x, float("nan"))
    capi.loss_grad(p, x, lx, ly, y, ws, costs, loss, gc, stride, gx, pipe=pipe, groups=groups, **shard)
    torch.cuda.synchronize()
    assert capi.read_status(ws)[0] == 0
    return costs, loss, gx, ws


def _same(a, b):
    assert torch.equal(a, b), float((a.double() - b.double()).abs().max())


@pytest.mark.parametrize("groups", [0, 1, 2, 3, 4, 8])  # 0 = the library's choice (1 for a problem this small)
def test_groups_are_bit_identical_to_forward_backward(pipe, groups):
    # 40 sequences, ~60k rows: ranges of 2048-row multiples, several sequences per group
    case = ragged_case(11, 40, (20, 90), (3, 40), V=256, sigma=2.0)
    args = _setup(case)
    c0, l0, g0 = _two_calls(*args)
    c1, l1, g1, _ = _one_call(pipe, *args, groups=groups)
    _same(c0, c1)
    _same(l0, l1)
    _same(g0, g1)


def test_sequences_longer_than_a_range_and_empty_groups(pipe):
    # 3 sequences of very different size cut into 8 ranges: one sequence spans several ranges (its group is the
    # range of its last row, the groups before that stay empty) and the gradient grid of its group is too small for
    # it, so the CTAs loop
    rng = np.random.default_rng(5)
    lx = np.array([400, 30, 90], np.int32)
    ly = np.array([60, 5, 20], np.int32)
    y = rng.integers(1, 64, size=(3, 60)).astype(np.int32)
    rows = int((lx.astype(np.int64) * (ly + 1)).sum())
    case = dict(x=rng.standard_normal((rows, 64)).astype(np.float32), lx=lx, ly=ly, y=y, blank=0, V=64)
    args = _setup(case)
    c0, l0, g0 = _two_calls(*args)
    for groups in (2, 8):
        c1, l1, g1, _ = _one_call(pipe, *args, groups=groups)
        _same(c0, c1)
        _same(l0, l1)
        _same(g0, g1)


def test_traced_pipe_reports_a_timeline(pipe):
    """A pipe created with tracing reports, per sequence group of the last step, when its range was gathered, its
    wavefront done and its gradient done; results are the same as through an untraced pipe."""
    case = ragged_case(12, 30, (20, 70), (3, 130), V=64, sigma=2.0)
    args = _setup(case)
    c0, l0, g0 = _two_calls(*args)
    traced = capi.Pipe(DEV, traced=True)
    c1, l1, g1, _ = _one_call(traced, *args, groups=3)
    _same(c0, c1)
    _same(g0, g1)
    tl = traced.timeline()
    assert len(tl) == 3 and all(0 < a <= b <= c for a, b, c in tl)
    _one_call(traced, *args, groups=1)
    assert traced.timeline() == []       # an ungrouped step stays on the caller's stream: nothing to report
    traced.close()
    with pytest.raises(capi.CwrnntError):
        pipe.timeline()  # an untraced pipe has no timestamps


@pytest.mark.parametrize("shape", [(6, (30, 90), (5, 40)), (12, (10, 40), (100, 300))])
def test_adaptive_gradient_schedule_is_bit_identical_and_capturable(pipe, shape):
    """Batches of at most 8 sequences, or with lattices wider than 256 columns, queue each group's gradient behind the
    group's wavefront on that wavefront's own stream (at the lowest launch priority) instead of in group order. Same
    results bit for bit, and the whole step - priority attribute included - can be captured and replayed."""
    B, Tr, Ur = shape
    case = ragged_case(77 + B, B, Tr, Ur, V=64, sigma=1.5)
    args = _setup(case)
    p, x, lx, ly, y = args
    assert p.B <= 8 or p.max_u + 1 > 256
    c0, l0, g0 = _two_calls(*args)
    for groups in (2, 3, 4):
        c1, l1, g1, _ = _one_call(pipe, *args, groups=groups)
        _same(c0, c1)
        _same(l0, l1)
        _same(g0, g1)
    ws = capi.alloc_workspace(p, DEV)
    costs, loss, gx = torch.empty(p.B, device=DEV), torch.empty((), device=DEV), torch.empty_like(x)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            capi.loss_grad(p, x, lx, ly, y, ws, costs, loss, None, 0, gx, pipe=pipe, groups=3)
    torch.cuda.synchronize()
    for _ in range(2):
        costs.fill_(float("nan"))
        gx.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        _same(c0, costs)
        _same(l0, loss)
        _same(g0, gx)


def test_single_sequence(pipe):
    case = ragged_case(2, 1, (150, 150), (40, 40), V=128)
    args = _setup(case)
    c0, l0, g0 = _two_calls(*args)
    c1, l1, g1, _ = _one_call(pipe, *args, groups=4)
    _same(c0, c1)
    _same(g0, g1)


@pytest.mark.parametrize("dtype,flags", [
    (torch.float16, capi.FUSED_LOG_SOFTMAX | capi.REDUCE_SUM),
    (torch.bfloat16, capi.FUSED_LOG_SOFTMAX | capi.REDUCE_MEAN | capi.AVERAGE_FRAMES),
    (torch.float64, capi.FUSED_LOG_SOFTMAX),
    (torch.float32, capi.REDUCE_MEAN),  # log-probability contract: sparse gradient
    (torch.float32, capi.FUSED_LOG_SOFTMAX),
])
def test_dtypes_modes_and_per_sequence_upstream_gradients(pipe, oracle, dtype, flags):
    case = ragged_case(21, 24, (30, 80), (5, 30), V=200 if dtype != torch.float32 else 203, sigma=1.5)
    if not flags & capi.FUSED_LOG_SOFTMAX:
        case["x"] = oracle.log_softmax(case["x"]).astype(np.float32)
    args = _setup(case, dtype=dtype, flags=flags)
    ct = capi.cost_dtype(dtype)
    gc = torch.linspace(0.5, 2.0, args[0].B, dtype=ct, device=DEV)
    c0, l0, g0 = _two_calls(*args, gc=gc, stride=1)
    c1, l1, g1, _ = _one_call(pipe, *args, groups=3, gc=gc, stride=1)
    _same(c0, c1)
    _same(g0, g1)
    if flags & (capi.REDUCE_MEAN | capi.REDUCE_SUM):
        _same(l0, l1)


def test_without_a_pipe_and_repeated_calls(pipe):
    case = ragged_case(4, 16, (20, 60), (4, 25), V=512)
    args = _setup(case)
    c0, l0, g0 = _two_calls(*args)
    c1, l1, g1, _ = _one_call(None, *args, groups=4)  # no side streams: the same work in sequence
    _same(c0, c1)
    _same(g0, g1)
    for _ in range(3):  # the pipe's streams and events are reused call after call
        c2, l2, g2, ws = _one_call(pipe, *args, groups=4)
        _same(c0, c2)
        _same(l0, l2)
        _same(g0, g2)
    # the workspace is left as cwrnnt_forward leaves it: a plain backward may follow
    p, x, lx, ly, y = args
    gx = torch.empty_like(x)
    capi.backward(p, x, lx, ly, y, ws, None, 0, gx)
    _same(g0, gx)


def test_sharded_cost_vector(pipe):
    case = ragged_case(8, 12, (20, 70), (3, 30), V=256)
    n_global = 20
    args = _setup(case, mean_denominator=n_global)
    p, x, lx, ly, y = args
    ids = torch.tensor([19, 0, 3, 5, 7, 9, 11, 13, 15, 17, 2, 4], dtype=torch.int32, device=DEV)
    vec0 = torch.full((n_global + 1,), float("nan"), device=DEV)
    ws = capi.alloc_workspace(p, DEV)
    costs = torch.empty(p.B, device=DEV)
    loss = torch.empty((), device=DEV)
    capi.forward_sharded(p, x, lx, ly, y, ws, costs, loss, ids, n_global, vec0)
    vec1 = torch.full((n_global + 1,), float("nan"), device=DEV)
    c1, l1, g1, _ = _one_call(pipe, *args, groups=4, global_ids=ids, n_global=n_global, cost_vector=vec1)
    torch.cuda.synchronize()
    _same(vec0, vec1)
    _same(costs, c1)


def test_argument_errors(pipe):
    case = ragged_case(1, 4, (10, 20), (2, 8), V=64)
    p, x, lx, ly, y = _setup(case)
    ws = capi.alloc_workspace(p, DEV)
    costs, loss, gx = torch.empty(p.B, device=DEV), torch.empty((), device=DEV), torch.empty_like(x)
    with pytest.raises(capi.CwrnntError):
        capi.loss_grad(p, x, lx, ly, y, ws, costs, loss, None, 0, gx, pipe=pipe, groups=9)
    q, *_ = _setup(case, flags=capi.FUSED_LOG_SOFTMAX | capi.COSTS_ONLY)
    with pytest.raises(capi.CwrnntError):
        capi.loss_grad(q, x, lx, ly, y, ws, costs, loss, None, 0, gx, pipe=pipe)
    with pytest.raises(capi.CwrnntError):  # a cost vector shorter than the batch
        capi.loss_grad(p, x, lx, ly, y, ws, costs, loss, None, 0, gx, pipe=pipe, n_global=2,
                       cost_vector=torch.empty(3, device=DEV))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.float64])
def test_scale_grad(dtype):
    g = torch.randn(37, 101, device=DEV).to(dtype)  # odd sizes: vector body and scalar tail
    p = capi.Problem(37, 101, 0, 0, 0, 0, capi.dtype_code(dtype), 0, 0)
    ct = capi.cost_dtype(dtype)
    ref = g.clone()
    capi.scale_grad(p, g, torch.ones(1, dtype=ct, device=DEV))
    _same(g, ref)
    capi.scale_grad(p, g, torch.full((1,), 0.25, dtype=ct, device=DEV))
    _same(g, (ref.to(ct) * 0.25).to(dtype))
    view = g.view(-1)[1:1 + 36 * 101].view(36, 101)  # base not 16-byte aligned
    q = capi.Problem(36, 101, 0, 0, 0, 0, capi.dtype_code(dtype), 0, 0)
    want = (view.to(ct) * 3.0).to(dtype)
    capi.scale_grad(q, view, torch.full((1,), 3.0, dtype=ct, device=DEV))
    _same(view, want)


@pytest.mark.parametrize("fused", [True, False])
def test_autograd_eager_gradient_equals_deferred(oracle, fused):
    import cwarp_rnnt
    case = ragged_case(17, 10, (15, 60), (2, 20), V=96, sigma=1.5)
    xin = case["x"] if fused else oracle.log_softmax(case["x"]).astype(np.float32)
    lx = torch.as_tensor(case["lx"]).to(DEV)
    ly = torch.as_tensor(case["ly"]).to(DEV)
    y = torch.as_tensor(case["y"]).to(DEV).contiguous()

    def run(eager, upstream, twice=False):
        x = torch.as_tensor(xin).to(DEV).requires_grad_(True)
        loss = cwarp_rnnt.transducer_loss(x, lx, y, ly, 0, "mean", fused_log_softmax=fused, eager_grad=eager)
        (loss * upstream).backward(retain_graph=twice)
        if twice:
            first = x.grad.clone()
            x.grad = None
            (loss * upstream).backward()  # the stored gradient was handed over: recomputed from the workspace
            if upstream == 1.0:
                _same(first, x.grad)
            else:
                torch.testing.assert_close(x.grad, first, rtol=2e-6, atol=1e-8)
        return loss.detach(), x.grad

    for upstream in (1.0, 128.0):
        l0, g0 = run(False, upstream)
        l1, g1 = run(True, upstream)
        _same(l0, l1)
        if upstream == 1.0:
            _same(g0, g1)
        else:  # scaled after the fact instead of inside the gradient kernel: one more rounding
            torch.testing.assert_close(g1, g0, rtol=2e-6, atol=1e-8)
    run(True, 1.0, twice=True)
    run(True, 3.0, twice=True)


def test_pipelined_step_captured_in_a_cuda_graph(pipe, oracle):
    """Fork and join are event waits, so the whole pipelined step - side streams included - is captured into one CUDA
    graph. Group membership is worked out on the device, so the graph can be replayed on other lengths as long as the
    row and sequence counts stay: here the same sequences in another order, with new logits."""
    case = ragged_case(41, 12, (10, 60), (2, 25), V=128, sigma=1.5)
    p, x, lx, ly, y = _setup(case)
    B = p.B
    ws = capi.alloc_workspace(p, DEV)
    costs, loss, gx = torch.empty(B, device=DEV), torch.empty((), device=DEV), torch.empty_like(x)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        capi.loss_grad(p, x, lx, ly, y, ws, costs, loss, None, 0, gx, pipe=pipe, groups=3)  # first use: not captured
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            capi.loss_grad(p, x, lx, ly, y, ws, costs, loss, None, 0, gx, pipe=pipe, groups=3)
    torch.cuda.synchronize()
    rng = np.random.default_rng(3)
    for trial in range(2):
        perm = rng.permutation(B)
        lx2, ly2, y2 = case["lx"][perm], case["ly"][perm], case["y"][perm]
        fresh = (rng.standard_normal(case["x"].shape) * 1.5).astype(np.float32)
        x.copy_(torch.as_tensor(fresh))
        lx.copy_(torch.as_tensor(lx2))
        ly.copy_(torch.as_tensor(ly2))
        y.copy_(torch.as_tensor(y2))
        graph.replay()
        torch.cuda.synchronize()
        assert capi.read_status(ws)[0] == 0
        c64, d64 = oracle.fused(fresh, lx2, ly2, y2, 0, weights=np.full(B, 1.0 / B))
        np.testing.assert_allclose(costs.cpu().numpy(), c64, rtol=1e-5)
        assert abs(float(loss) - c64.mean()) <= 1e-5 * c64.mean()
        assert np.abs(gx.cpu().numpy() - d64).max() <= 1e-5


def test_costs_are_ready_before_the_gradient_pass(pipe):
    """cwrnnt_pipe_wait_costs: a second stream that waits for the costs-ready event sees the final costs, loss and
    cost vector (the place where a sharded caller starts its all-reduce), and the gradient still comes out right."""
    case = ragged_case(23, 20, (20, 80), (3, 30), V=512)
    args = _setup(case)
    p, x, lx, ly, y = args
    c0, l0, g0 = _two_calls(*args)
    ws = capi.alloc_workspace(p, DEV)
    costs = torch.full((p.B,), float("nan"), device=DEV)
    loss = torch.full((), float("nan"), device=DEV)
    vec = torch.full((p.B + 1,), float("nan"), device=DEV)
    gx = torch.empty_like(x)
    other = torch.cuda.Stream()
    for groups in (1, 4):
        capi.loss_grad(p, x, lx, ly, y, ws, costs, loss, None, 0, gx, pipe=pipe, groups=groups, n_global=p.B,
                       cost_vector=vec)
        with torch.cuda.stream(other):
            pipe.wait_costs(other)
            seen_costs, seen_loss, seen_vec = costs.clone(), loss.clone(), vec.clone()
        other.synchronize()
        _same(seen_costs, c0)
        _same(seen_loss, l0)
        _same(seen_vec[:-1], c0)
        torch.cuda.synchronize()
        _same(gx, g0)


def test_random_shapes_against_the_two_call_path(pipe):
    """Forty seeded random problems - batch sizes from 1 to 70, vocabularies that hit every row shape of the streaming
    kernels (vector-aligned and not), all four element types, every group count - must reproduce cwrnnt_forward +
    cwrnnt_backward bit for bit."""
    rng = np.random.default_rng(2025)
    dtypes = [torch.float32, torch.float16, torch.bfloat16, torch.float64]
    vocab = [3, 8, 24, 64, 100, 128, 256, 520, 1024, 2048, 4104]
    for trial in range(40):
        B = int(rng.integers(1, 71))
        V = int(vocab[rng.integers(len(vocab))])
        t_hi = int(rng.integers(1, 60 if V <= 1024 else 12))
        u_hi = int(rng.integers(0, 30 if V <= 1024 else 8))
        case = ragged_case(1000 + trial, B, (1, t_hi), (0, u_hi), V=V)
        dtype = dtypes[trial % 4]
        flags = capi.FUSED_LOG_SOFTMAX | (capi.REDUCE_MEAN if trial % 3 else capi.REDUCE_SUM)
        args = _setup(case, dtype=dtype, flags=flags)
        c0, l0, g0 = _two_calls(*args)
        groups = int(rng.integers(0, 9))
        c1, l1, g1, _ = _one_call(pipe, *args, groups=groups)
        assert torch.equal(c0, c1) and torch.equal(l0, l1) and torch.equal(g0, g1), (trial, B, V, dtype, groups)


def test_many_tiny_sequences_in_groups(pipe):
    """4500 sequences (beyond the longest-first sort, 9000 wavefront CTAs per launch, four launches sharing one
    completion ticket)."""
    case = ragged_case(32, 4500, (1, 4), (0, 3), V=8)
    args = _setup(case)
    c0, l0, g0 = _two_calls(*args)
    for groups in (4, 8):
        c1, l1, g1, _ = _one_call(pipe, *args, groups=groups)
        _same(c0, c1)
        _same(l0, l1)
        _same(g0, g1)


def test_invalid_lengths_stop_every_group(pipe):
    """A row count that disagrees with the lengths is fatal: no group's kernels do their work, the costs, the loss,
    the cost vector and every element of the gradient are NaN, the status says why, and the pipe is usable again
    afterwards."""
    case = ragged_case(6, 30, (10, 40), (2, 12), V=64)
    p, x, lx, ly, y = _setup(case)
    lx_bad = lx.clone()
    lx_bad[3] += 1
    ws = capi.alloc_workspace(p, DEV)
    costs = torch.zeros(p.B, device=DEV)
    loss = torch.zeros((), device=DEV)
    gx = torch.full_like(x, 5.0)
    vec = torch.zeros(p.B + 3, device=DEV)
    for groups in (4, 1):
        gx.fill_(5.0)
        capi.loss_grad(p, x, lx_bad, ly, y, ws, costs, loss, None, 0, gx, pipe=pipe, groups=groups, n_global=p.B + 2,
                       cost_vector=vec)
        torch.cuda.synchronize()
        st = capi.read_status(ws)
        assert st[0] & capi.ST_ROW_MISMATCH
        assert bool(torch.isnan(costs).all()) and bool(torch.isnan(loss)) and bool(torch.isnan(vec).all())
        assert bool(torch.isnan(gx).all())
    gx.fill_(5.0)
    capi.forward(p, x, lx_bad, ly, y, ws, costs, loss)
    capi.backward(p, x, lx_bad, ly, y, ws, None, 0, gx)
    assert bool(torch.isnan(loss)) and bool(torch.isnan(gx).all())
    c0, l0, g0 = _two_calls(p, x, lx, ly, y)
    c1, l1, g1, _ = _one_call(pipe, p, x, lx, ly, y, groups=4)
    _same(c0, c1)
    _same(g0, g1)


def test_graphed_step_bucket(oracle):
    """GraphedStep: one graph per (rows, sequences, label width) bucket, replayed on batches whose lengths differ."""
    from compactwarprnntloss_b200 import GraphedStep
    case = ragged_case(51, 10, (5, 50), (1, 20), V=96, sigma=1.5)
    B, n_rows = 10, case["x"].shape[0]
    bucket = GraphedStep(n_rows, 96, B, int(case["ly"].max()) + 3, dtype=torch.float32, device=DEV, groups=3)
    rng = np.random.default_rng(7)
    for trial in range(3):
        perm = rng.permutation(B)
        lx, ly, y = case["lx"][perm], case["ly"][perm], case["y"][perm]
        x = (rng.standard_normal(case["x"].shape) * 1.5).astype(np.float32)
        loss, costs, grad = bucket.step(torch.as_tensor(x).to(DEV), torch.as_tensor(lx).to(DEV),
                                        torch.as_tensor(ly).to(DEV), torch.as_tensor(y).to(DEV))
        torch.cuda.synchronize()
        assert bucket.status()[0] == 0
        c64, d64 = oracle.fused(x, lx, ly, y, 0, weights=np.full(B, 1.0 / B))
        np.testing.assert_allclose(costs.cpu().numpy(), c64, rtol=1e-5)
        assert abs(float(loss) - c64.mean()) <= 1e-5 * c64.mean()
        assert np.abs(grad.cpu().numpy() - d64).max() <= 1e-5
