"""`cwrnnt_costs_static`: the costs-only forward that takes no workspace and allocates nothing.

It exists for hosts that cannot call cudaMalloc (a plug-in whose framework owns all device memory, a binding without
a device allocator, a loop that cannot afford an allocation's synchronisation); its scratch is a fixed array inside the
library. The checks: through the C ABI, two calls in a row on different batches (the second one smaller, so that it
runs over the first call's leftovers in the shared array) give the same costs and loss as `cwrnnt_forward` with a
caller workspace, within the tolerance of the other GPU tests; free device memory does not move across a call; a batch
above the stated capacity is refused before anything is launched.

Collected last on purpose (file name), so a run that stops at the first failure has already covered everything else.
"""
import ctypes

import numpy as np
import pytest
import torch

from tests.helpers import ragged_case

pytestmark = pytest.mark.gpu
LOSS_RTOL = 1e-5


def _device_inputs(case):
    dev = torch.device("cuda:0")
    return (torch.as_tensor(case["x"]).to(dev).contiguous(), torch.as_tensor(case["lx"]).to(dev),
            torch.as_tensor(case["ly"]).to(dev), torch.as_tensor(case["y"]).to(dev).contiguous())


def _both_ways(case, flags):
    from compactwarprnntloss_b200 import capi
    x, lx, ly, y = _device_inputs(case)
    p = capi.make_problem(x, lx, y, case["blank"], flags | capi.COSTS_ONLY)
    ws = capi.alloc_workspace(p, x.device)
    want_c = torch.empty(p.B, device=x.device)
    want_l = torch.zeros((), device=x.device)
    capi.forward(p, x, lx, ly, y, ws, want_c, want_l)
    got_c = torch.full((p.B,), float("nan"), device=x.device)
    got_l = torch.full((), float("nan"), device=x.device)
    p2 = capi.make_problem(x, lx, y, case["blank"], flags)  # COSTS_ONLY is implied by the entry point
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    capi.costs_static(p2, x, lx, ly, y, got_c, got_l)
    torch.cuda.synchronize()
    free_after = torch.cuda.mem_get_info()[0]
    return want_c.cpu().numpy(), float(want_l), got_c.cpu().numpy(), float(got_l), free_before, free_after


def test_static_scratch_entry_point_matches_workspace_entry_point(oracle):
    from compactwarprnntloss_b200 import capi
    flags = capi.FUSED_LOG_SOFTMAX | capi.REDUCE_MEAN
    big = ragged_case(901, 9, (10, 60), (2, 25), V=64, sigma=2.0)
    small = ragged_case(902, 3, (2, 12), (0, 6), V=64, sigma=1.0)
    first = _both_ways(big, flags)          # first call on this device also resolves the scratch address
    second = _both_ways(small, flags)       # runs over the leftovers of the first call
    third = _both_ways(big, flags)
    for case, (want_c, want_l, got_c, got_l, _, _) in ((big, first), (small, second), (big, third)):
        assert np.all(np.isfinite(got_c))
        np.testing.assert_allclose(got_c, want_c, rtol=LOSS_RTOL, atol=1e-6)
        assert abs(got_l - want_l) <= LOSS_RTOL * abs(want_l) + 1e-6
        costs, _ = oracle.fused(case["x"], case["lx"], case["ly"], case["y"], case["blank"], want_grad=False)
        np.testing.assert_allclose(got_c, costs, rtol=LOSS_RTOL, atol=1e-6)
    # nothing was allocated by the second and third calls (the first may have loaded the kernels' module)
    assert second[4] == second[5] and third[4] == third[5]


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from compactwarprnntloss_b200 import capi
    L = capi.lib()
    dev = torch.device("cuda:0")
    one = torch.zeros(1, dtype=torch.int32, device=dev)
    x = torch.zeros(8, 4, device=dev)
    y = torch.zeros(1, 1, dtype=torch.int32, device=dev)
    costs = torch.zeros(1, device=dev)
    p = capi.make_problem(x, one, y, 0, capi.FUSED_LOG_SOFTMAX)
    p.n_rows = capi.STATIC_MAX_ROWS + 1     # descriptor only: refused before any pointer is touched
    vp = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    rc = L.cwrnnt_costs_static(ctypes.byref(p), vp(x), vp(one), vp(one), vp(y), vp(costs), None, None)
    assert rc == capi.ERR_CAPACITY
    assert str(capi.STATIC_MAX_ROWS) in L.cwrnnt_last_error().decode()
    p.n_rows, p.B = 8, capi.STATIC_MAX_SEQUENCES + 1
    assert L.cwrnnt_costs_static(ctypes.byref(p), vp(x), vp(one), vp(one), vp(y), vp(costs), None, None) == capi.ERR_CAPACITY
    with pytest.raises(capi.CwrnntError, match="at most"):
        capi.costs_static(p, x, one, one, y, costs)


def test_static_scratch_entry_point_at_its_stated_capacity(oracle):
    """Exactly CWRNNT_STATIC_MAX_ROWS rows, and exactly CWRNNT_STATIC_MAX_SEQUENCES sequences: the carve of the
    built-in array leaves a few KB of slack there, so the largest accepted problems are run for real against the
    workspace entry point."""
    from compactwarprnntloss_b200 import capi
    rng = np.random.default_rng(77)
    V = 8
    # (a) the row limit with few, larger sequences: 128 lattices of 64 x 16 = 131072 rows
    lx = np.full(128, 64, np.int32)
    ly = np.full(128, 15, np.int32)
    assert int((lx.astype(np.int64) * (ly + 1)).sum()) == capi.STATIC_MAX_ROWS
    y = rng.integers(1, V, size=(128, 15)).astype(np.int32)
    big_rows = dict(x=rng.standard_normal((capi.STATIC_MAX_ROWS, V)).astype(np.float32), lx=lx, ly=ly, y=y, blank=0, V=V)
    # (b) the sequence limit: 1024 sequences of 128 rows -> also the row limit
    lx = np.full(1024, 32, np.int32)
    ly = np.full(1024, 3, np.int32)
    y = rng.integers(1, V, size=(1024, 3)).astype(np.int32)
    many = dict(x=rng.standard_normal((capi.STATIC_MAX_ROWS, V)).astype(np.float32), lx=lx, ly=ly, y=y, blank=0, V=V)
    for case in (big_rows, many, big_rows):
        want_c, want_l, got_c, got_l, _, _ = _both_ways(case, capi.FUSED_LOG_SOFTMAX | capi.REDUCE_SUM)
        assert np.all(np.isfinite(got_c))
        np.testing.assert_allclose(got_c, want_c, rtol=LOSS_RTOL, atol=1e-6)
        assert abs(got_l - want_l) <= LOSS_RTOL * abs(want_l)
        assert capi.static_status(torch.device("cuda:0"))[0] == 0
    costs, _ = oracle.fused(many["x"], many["lx"], many["ly"], many["y"], 0, want_grad=False)
    np.testing.assert_allclose(_both_ways(many, capi.FUSED_LOG_SOFTMAX)[2], costs, rtol=LOSS_RTOL, atol=1e-6)


def test_static_scratch_entry_point_reports_its_status_words():
    """The scratch is private, so the status of a call is read through cwrnnt_static_status: a clamped label and
    lengths that do not add up must be visible there, not only as NaN costs."""
    from compactwarprnntloss_b200 import capi
    dev = torch.device("cuda:0")
    case = ragged_case(903, 5, (3, 12), (1, 6), V=16)
    x, lx, ly, y = _device_inputs(case)
    p = capi.make_problem(x, lx, y, 0, capi.FUSED_LOG_SOFTMAX)
    costs = torch.empty(p.B, device=dev)
    capi.costs_static(p, x, lx, ly, y, costs)
    assert capi.static_status(dev)[0] == 0
    bad_y = y.clone()
    bad_y[0, 0] = 16
    capi.costs_static(p, x, lx, ly, bad_y, costs)
    assert capi.static_status(dev)[0] == capi.ST_BAD_LABEL and bool(torch.isfinite(costs).all())
    bad_lx = lx.clone()
    bad_lx[2] += 1
    capi.costs_static(p, x, bad_lx, ly, y, costs)
    st = capi.static_status(dev)
    assert st[0] & capi.ST_ROW_MISMATCH and bool(torch.isnan(costs).all())
    capi.costs_static(p, x, lx, ly, y, costs)       # and the next good call starts from a clean header
    assert capi.static_status(dev)[0] == 0 and bool(torch.isfinite(costs).all())
