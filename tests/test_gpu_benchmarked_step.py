"""The exact step `bench.py` times, at its size, against the CPU oracle.

`bench.py` calls `cwrnnt_loss_grad` with `groups = 0` on the whole Conformer-shape batch (32 sequences, 314 340 lattice
nodes, 1.29 GB of float32 logits): at that size the library cuts the step into sequence groups on its own, the group
bounds are worked out on the device and the streaming grids are sized per row range - code that smaller problems only
reach when a test forces a group count. Here that very call, and the Python entry point `transducer_loss(...,
fused_log_softmax=True)` + `backward()` that sits on top of it, are held to the double-precision oracle on all 32
sequences: costs and loss to 1e-5 relative, every gradient element to 1e-5 absolute.
"""
import numpy as np
import pytest
import torch

from compactwarprnntloss_b200 import capi, synth

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


@pytest.fixture(scope="module")
def conformer_batch(oracle):
    lx, ly, y = synth.lengths_and_labels(2)
    x = synth.compact_logits(2, lx, ly)
    B = len(lx)
    costs, dense = oracle.fused(x.double().numpy(), lx.numpy(), ly.numpy(), y.numpy(), 0, weights=np.full(B, 1.0 / B))
    return dict(x=x, lx=lx, ly=ly, y=y, costs=costs, dense=torch.from_numpy(dense))


def _max_abs_diff(gx, dense64):
    worst = 0.0
    for a in range(0, gx.shape[0], 65536):  # in slices: the double copy of the whole gradient is 2.6 GB
        worst = max(worst, float((gx[a:a + 65536].double().cpu() - dense64[a:a + 65536]).abs().max()))
    return worst


def test_full_conformer_batch_through_the_c_abi_call_bench_times(conformer_batch):
    c = conformer_batch
    x = c["x"].to(DEV)
    lx, ly, y = c["lx"].to(DEV), c["ly"].to(DEV), c["y"].to(DEV).contiguous()
    p = capi.make_problem(x, lx, y, 0, capi.FUSED_LOG_SOFTMAX | capi.REDUCE_MEAN)
    assert capi.pipeline_groups(p, 0) > 1, "the benchmarked size must take the grouped pipeline without being told to"
    ws = capi.alloc_workspace(p, DEV)
    costs = torch.full((p.B,), float("nan"), device=DEV)
    loss = torch.full((), float("nan"), device=DEV)
    gx = torch.full_like(x, float("nan"))
    one = torch.ones(1, device=DEV)
    pipe = capi.Pipe(DEV)
    for _ in range(2):  # the second call runs on the pipe's already-used streams and events, as every timed step does
        capi.loss_grad(p, x, lx, ly, y, ws, costs, loss, one, 0, gx, pipe=pipe, groups=0)
    torch.cuda.synchronize()
    pipe.close()
    assert capi.read_status(ws)[0] == 0
    np.testing.assert_allclose(costs.cpu().numpy(), c["costs"], rtol=1e-5)
    assert abs(float(loss) - c["costs"].mean()) <= 1e-5 * c["costs"].mean()
    assert _max_abs_diff(gx, c["dense"]) <= 1e-5


@pytest.mark.parametrize("check", [True, False])
def test_full_conformer_batch_through_transducer_loss(conformer_batch, check):
    import cwarp_rnnt
    c = conformer_batch
    x = c["x"].to(DEV).requires_grad_(True)
    lx, ly, y = c["lx"].to(DEV), c["ly"].to(DEV), c["y"].to(DEV).contiguous()
    loss = cwarp_rnnt.transducer_loss(x, lx, y, ly, 0, "mean", fused_log_softmax=True, check=check)
    loss.backward()
    torch.cuda.synchronize()
    assert abs(float(loss) - c["costs"].mean()) <= 1e-5 * c["costs"].mean()
    assert _max_abs_diff(x.grad, c["dense"]) <= 1e-5
    per_seq = cwarp_rnnt.transducer_loss(x.detach(), lx, y, ly, 0, "none", fused_log_softmax=True, check=check)
    np.testing.assert_allclose(per_seq.cpu().numpy(), c["costs"], rtol=1e-5)


def test_invalid_batch_is_loud_without_the_check():
    """check=False never synchronises, so nothing can be raised; a batch whose lengths do not add up to the row count
    must then show in every result - NaN costs, NaN loss, NaN gradient - not as a zero loss and an unwritten gradient."""
    import cwarp_rnnt
    from tests.helpers import ragged_case
    case = ragged_case(6, 30, (10, 40), (2, 12), V=64)
    x = torch.as_tensor(case["x"]).to(DEV).requires_grad_(True)
    lx = torch.as_tensor(case["lx"]).to(DEV)
    ly = torch.as_tensor(case["ly"]).to(DEV)
    y = torch.as_tensor(case["y"]).to(DEV).contiguous()
    lx[3] += 1
    for eager in (True, False):
        x.grad = None
        loss = cwarp_rnnt.transducer_loss(x, lx, y, ly, 0, "mean", fused_log_softmax=True, check=False,
                                          eager_grad=eager)
        loss.backward()
        assert bool(torch.isnan(loss)) and bool(torch.isnan(x.grad).all()), eager
    costs = cwarp_rnnt.transducer_loss(x.detach(), lx, y, ly, 0, "none", fused_log_softmax=True, check=False)
    assert bool(torch.isnan(costs).all())
    with pytest.raises(ValueError, match="rows"):   # and with the check it raises, after the kernels were queued
        cwarp_rnnt.transducer_loss(x, lx, y, ly, 0, "mean", fused_log_softmax=True)
    lx[3] -= 1
    y[0, 0] = 64
    with pytest.raises(ValueError, match="label"):
        cwarp_rnnt.transducer_loss(x, lx, y, ly, 0, "mean", fused_log_softmax=True)


def test_validate_async_fills_pinned_words_behind_the_stream():
    from tests.helpers import ragged_case
    case = ragged_case(5, 40, (1, 40), (0, 17), V=33)
    x = torch.as_tensor(case["x"]).to(DEV)
    lx, ly = torch.as_tensor(case["lx"]).to(DEV), torch.as_tensor(case["ly"]).to(DEV)
    y = torch.as_tensor(case["y"]).to(DEV).contiguous()
    p = capi.make_problem(x, lx, y, 0, capi.FUSED_LOG_SOFTMAX)
    words = torch.full((4,), 123, dtype=torch.int32).pin_memory()
    scratch = torch.empty(4, dtype=torch.int32, device=DEV)
    capi.validate_async(p, lx, ly, y, words, scratch)
    done = torch.cuda.Event()
    done.record()
    done.synchronize()
    assert words.tolist() == [0, -1, int(case["lx"].max()), int(case["ly"].max())]
    assert words.tolist() == capi.validate(p, lx, ly, y)
