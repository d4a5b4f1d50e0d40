"""Host-side sharding logic and the cost-vector exchange among CPU ranks (gloo, world_size 2 and 3)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from compactwarprnntloss_b200 import sharding, synth


def test_plan_is_balanced_deterministic_and_complete():
    lx, ly, _ = synth.lengths_and_labels(5)
    for world in (1, 2, 4, 8):
        plan = sharding.plan_shards(lx.tolist(), ly.tolist(), world)
        sharding.validate_plan(plan, len(lx))
        assert plan == sharding.plan_shards(lx.tolist(), ly.tolist(), world)
        # longest critical path (T+U) first, so its wavefront starts first
        chain = (lx + ly).tolist()
        longest = sharding.plan_shards(lx.tolist(), ly.tolist(), world, order="longest_first")
        assert all(all(chain[a] >= chain[b] for a, b in zip(ids, ids[1:])) for ids in longest)
        # default: the same, except that a shard of at most 8 sequences is led by its shortest one
        for ids, ref in zip(plan, longest):
            assert ids == ([ref[-1]] + ref[:-1] if 1 < len(ref) <= 8 else ref)
        asc = sharding.plan_shards(lx.tolist(), ly.tolist(), world, order="ascending")
        assert [sorted(ids) for ids in plan] == asc and all(ids == sorted(ids) for ids in asc)
        assert sharding.shard_imbalance(lx, ly, plan) < 1.05
    lx4, ly4, _ = synth.lengths_and_labels(4)
    few = sharding.plan_shards(lx4.tolist(), ly4.tolist(), 1)[0]
    chain4 = (lx4 + ly4).tolist()
    assert chain4[few[0]] == min(chain4) and chain4[few[1]] == max(chain4)
    lx2, ly2, _ = synth.lengths_and_labels(2, B=64)
    assert sharding.shard_imbalance(lx2, ly2, sharding.plan_shards(lx2, ly2, 8)) < 1.05


def test_plan_rejects_bad_input_and_bad_plans():
    with pytest.raises(ValueError):
        sharding.plan_shards([1, 2], [1], 2)
    with pytest.raises(ValueError):
        sharding.plan_shards([1], [1], 0)
    with pytest.raises(ValueError):
        sharding.plan_shards([1], [1], 1, order="random")
    with pytest.raises(ValueError):
        sharding.validate_plan([[0, 1], [1, 2]], 3)   # sequence 1 twice: ranks disagree on the plan
    with pytest.raises(ValueError):
        sharding.validate_plan([[0], [2]], 3)         # sequence 1 lost
    assert sharding.plan_shards([], [], 3) == [[], [], []]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lx, ly, _ = synth.lengths_and_labels(1, B=11)
        plan = sharding.plan_shards(lx.tolist(), ly.tolist(), world)
        ids = plan[rank]
        true_costs = torch.arange(11, dtype=torch.float32) * 1.5 + 2.0
        local = true_costs[ids]
        costs, loss = sharding.exchange_costs(local, ids, 11, local_loss=local.sum() / 11)
        ok = torch.allclose(costs, true_costs) and abs(float(loss) - float(true_costs.mean())) < 1e-5
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_cost_exchange_among_cpu_ranks(world):
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, ret)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert all(ret.get(r) for r in range(world))


def _straggler_main(rank, world, port, ret):
    """Rank 1 never joins the collective: rank 0 must get an error from the bounded wait, not hang."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        ret[1] = "left"
        os._exit(0)  # leaves between steps, nothing in flight
    try:
        sharding.exchange_costs(torch.ones(1), [0], 2, local_loss=torch.tensor(1.0))
        ret[0] = "no error"
    except Exception as e:  # noqa: BLE001
        ret[0] = "error: " + type(e).__name__


def test_missing_rank_surfaces_as_error_not_hang():
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_straggler_main, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
    for p in procs:
        if p.is_alive():
            p.kill()
    assert ret.get(1) == "left"
    assert str(ret.get(0, "")).startswith("error"), ret.get(0)


def test_sequences_keep_their_data_wherever_they_land():
    """Per-sequence seeding: a sequence's logits do not depend on which rank or chunk generates it."""
    lx, ly, _ = synth.lengths_and_labels(1)
    full = synth.compact_logits(1, lx, ly)
    part = synth.compact_logits(1, lx, ly, ids=[2])
    off = int((lx[:2].long() * (ly[:2].long() + 1)).sum())
    rows = int(lx[2]) * (int(ly[2]) + 1)
    assert torch.equal(full[off:off + rows], part)
    assert synth.lattice_nodes(lx, ly) == full.shape[0]
