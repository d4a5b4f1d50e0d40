"""Sequence sharding across the GPUs of one box, and the one small collective a sharded step needs.

Sequences are independent (a lattice is never split), so the path shards by assigning whole sequences to ranks,
balanced by lattice size; logits and gradients never cross GPUs. The only exchange is the per-sequence cost vector and
the loss: one all-reduce(sum) over a zero-initialised [B_global + 1] vector in which every rank fills the slots of its
own sequences and adds its partial loss to the last slot (equivalent to an all-gather of costs plus a loss reduction,
in a single ~1 KB message). Gradient weights use the global batch size, known up front, so the backward pass needs no
collective at all.
"""
from typing import List, Optional, Sequence, Tuple

import torch


def plan_shards(lx: Sequence[int], ly: Sequence[int], world: int, order: str = "pipeline") -> List[List[int]]:
    """Longest-processing-time-first assignment of sequences to ``world`` ranks.

    Weight of a sequence = its lattice size T*(U+1) (streaming cost is proportional to it for a fixed V); ties are
    broken by the wavefront critical path T+U, then by index, so every rank computes the same plan. Returns the global
    sequence ids of each rank in the order the rank should lay its rows out in memory:

    ``order="longest_first"``  descending T+U, ties by index. The pipelined step cuts a rank's rows into
        groups in memory order and starts the alpha/beta wavefront of a group as soon as its rows are gathered; a
        wavefront is a chain of T+U dependent steps, so the longest chains must start first to finish underneath the
        streaming passes instead of after them. It is the sharding layer that decides a shard's row order, so this
        costs nothing.
    ``order="pipeline"`` (default)  longest_first, except that a shard of at most 8 sequences (the size below which
        the pipelined step gives every sequence a group of its own) is led by its SHORTEST sequence. The gradient pass
        can begin only when some wavefront is done; with a handful of long lattices the first one gathered is the
        first one done, so the shortest goes first and the gradient pass follows the gather pass without a gap
        (measured on 4 x [1250 x 300] x 512: 1.49 ms per step against 1.56), while the longest, gathered right after
        it, still has both passes to hide under. With many sequences per group a group is as slow as its longest
        chain, and a lead of short ones buys nothing (ragged 256-sequence batch: 0.71 ms against 0.68 with one short
        sequence in front; 0.69-0.77 ms against 0.66 with a leading block of short sequences holding 5-27 % of the rows).
    ``order="ascending"``  ascending global index (each rank's compact rows stay in global order).
    """
    if order not in ("longest_first", "pipeline", "ascending"):
        raise ValueError("order must be 'longest_first', 'pipeline' or 'ascending'")
    if world < 1:
        raise ValueError("world must be >= 1")
    lx = [int(v) for v in lx]
    ly = [int(v) for v in ly]
    if len(lx) != len(ly):
        raise ValueError("lx and ly differ in length")
    by_size = sorted(range(len(lx)), key=lambda i: (-(lx[i] * (ly[i] + 1)), -(lx[i] + ly[i]), i))
    load = [0] * world
    out: List[List[int]] = [[] for _ in range(world)]
    for i in by_size:
        r = min(range(world), key=lambda k: (load[k], k))
        out[r].append(i)
        load[r] += lx[i] * (ly[i] + 1)
    if order == "ascending":
        return [sorted(ids) for ids in out]
    shards = [sorted(ids, key=lambda i: (-(lx[i] + ly[i]), i)) for ids in out]
    if order == "pipeline":
        for r, ids in enumerate(shards):
            if 1 < len(ids) <= 8:
                shards[r] = [ids[-1]] + ids[:-1]
    return shards


def shard_imbalance(lx: Sequence[int], ly: Sequence[int], plan: List[List[int]]) -> float:
    """max rank load / mean rank load (1.0 = perfectly balanced)."""
    loads = [sum(int(lx[i]) * (int(ly[i]) + 1) for i in ids) for ids in plan]
    mean = sum(loads) / max(len(loads), 1)
    return max(loads) / mean if mean > 0 else 1.0


def validate_plan(plan: List[List[int]], B: int) -> None:
    """Every sequence exactly once; raises ValueError otherwise (a rank with a stale or foreign plan)."""
    seen = sorted(i for ids in plan for i in ids)
    if seen != list(range(B)):
        raise ValueError(f"shard plan does not cover sequences 0..{B - 1} exactly once")


def exchange_costs(local_costs: torch.Tensor, ids: Sequence[int], B_global: int,
                   local_loss: Optional[torch.Tensor] = None, group=None,
                   out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """All ranks end with every sequence's cost and the summed loss. One all-reduce of B_global + 1 numbers.

    ``local_costs[k]`` is the cost of global sequence ``ids[k]``; ``local_loss`` is this rank's partial loss (already
    divided by the global denominator for a mean). ``out`` may provide a reusable [B_global + 1] buffer.
    """
    import torch.distributed as dist
    if len(ids) != local_costs.numel():
        raise ValueError("ids and local_costs differ in length")
    vec = out if out is not None else torch.empty(B_global + 1, dtype=local_costs.dtype, device=local_costs.device)
    vec.zero_()
    if len(ids):
        idx = torch.as_tensor(list(ids), dtype=torch.long, device=local_costs.device)
        vec.index_copy_(0, idx, local_costs)
    if local_loss is not None:
        vec[B_global] = local_loss
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(vec, op=dist.ReduceOp.SUM, group=group)
    return vec[:B_global], vec[B_global]
