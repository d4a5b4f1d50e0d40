"""Two ranks on two GPUs over NCCL: every rank runs its shard of one batch through the pipelined single-call step
(`cwrnnt_loss_grad` with a global cost vector), one all-reduce is the whole exchange, and every rank ends with all
costs and the global loss, checked against the CPU oracle; each rank's gradient is checked on its own rows. Skipped
on a box with fewer than two GPUs (the CPU ranks of test_sharding.py cover the host side there)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

B_GLOBAL = 10


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _case():
    from tests.helpers import ragged_case
    return ragged_case(2024, B_GLOBAL, (5, 60), (0, 200), V=24, sigma=1.5)


def _shard_rows(case, ids):
    """Compact rows of the listed sequences, in that order."""
    lx, ly = case["lx"].astype(np.int64), case["ly"].astype(np.int64)
    off = np.concatenate([[0], np.cumsum(lx * (ly + 1))])
    return np.concatenate([case["x"][off[i]:off[i + 1]] for i in ids], axis=0)


def _rank_main(rank, world, port, ret):
    import torch.distributed as dist
    from compactwarprnntloss_b200 import capi, sharding
    from oracle import oracle as orc
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dev = torch.device(f"cuda:{rank}")
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        case = _case()
        plan = sharding.plan_shards(case["lx"].tolist(), case["ly"].tolist(), world)
        sharding.validate_plan(plan, B_GLOBAL)
        ids = plan[rank]
        x = torch.from_numpy(_shard_rows(case, ids)).to(dev)
        lx = torch.from_numpy(case["lx"][ids]).to(dev)
        ly = torch.from_numpy(case["ly"][ids]).to(dev)
        y = torch.from_numpy(case["y"][ids]).contiguous().to(dev)
        flags = capi.FUSED_LOG_SOFTMAX | capi.REDUCE_MEAN
        p = capi.make_problem(x, lx, y, 0, flags, mean_denominator=B_GLOBAL)
        ws = capi.alloc_workspace(p, dev)
        costs = torch.empty(p.B, device=dev)
        loss = torch.zeros((), device=dev)
        gx = torch.empty_like(x)
        vec = torch.empty(B_GLOBAL + 1, device=dev)
        ids_dev = torch.tensor(ids, dtype=torch.int32, device=dev)
        pipe = capi.Pipe(dev)
        for _ in range(2):  # a second call on the same workspace and pipe gives the same answer
            capi.loss_grad(p, x, lx, ly, y, ws, costs, loss, None, 0, gx, pipe=pipe, groups=2, global_ids=ids_dev,
                           n_global=B_GLOBAL, cost_vector=vec)
            dist.all_reduce(vec, op=dist.ReduceOp.SUM)
        torch.cuda.synchronize()
        pipe.close()
        assert capi.read_status(ws)[0] == 0

        want_costs, _ = orc.fused(case["x"].astype(np.float64), case["lx"], case["ly"], case["y"], 0, want_grad=False)
        got = vec.double().cpu().numpy()
        np.testing.assert_allclose(got[:B_GLOBAL], want_costs, rtol=1e-5, atol=1e-6)
        assert abs(got[B_GLOBAL] - want_costs.mean()) <= 1e-5 * abs(want_costs.mean())
        # this rank's gradient of the global mean, against the oracle on its own sequences
        sub = dict(x=_shard_rows(case, ids).astype(np.float64), lx=case["lx"][ids], ly=case["ly"][ids],
                   y=case["y"][ids])
        _, dense = orc.fused(sub["x"], sub["lx"], sub["ly"], sub["y"], 0,
                             weights=np.full(len(ids), 1.0 / B_GLOBAL))
        assert np.abs(gx.double().cpu().numpy() - dense).max() <= 2e-6
        ret[rank] = True
    finally:
        dist.destroy_process_group()


def test_two_ranks_two_gpus_costs_loss_and_gradients():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(world))
