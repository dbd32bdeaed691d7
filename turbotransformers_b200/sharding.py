"""Request sharding across GPUs of one node.

The transformer-layer path has no cross-request operation (layer norm and softmax are per row, weights are read
only), so it scales by giving each GPU its own requests and a replica of the weights; no collective touches the data
path. The only multi-GPU logic is therefore on the host: who gets which request, and how per-rank timings combine.

`balanced_shards` assigns variable-length requests so that every rank gets about the same attention + GEMM work
(cost ~ L^2 * 4H + L * 24H^2 per layer); `contiguous_shards` is the fixed-length split (batch 256 -> 128/64/32 per GPU).
"""
from typing import List, Sequence


def request_cost(length: int, hidden: int = 768) -> float:
    """Relative FLOPs of one encoder layer for a sequence of this length."""
    return 24.0 * hidden * hidden * length + 4.0 * hidden * length * length


def contiguous_shards(n_requests: int, world: int) -> List[List[int]]:
    """Rank r gets requests [r*ceil(n/world), ...): the split the benchmark's fixed-length configurations use."""
    per = (n_requests + world - 1) // world
    return [list(range(r * per, min(n_requests, (r + 1) * per))) for r in range(world)]


def balanced_shards(lengths: Sequence[int], world: int, hidden: int = 768) -> List[List[int]]:
    """Longest-processing-time greedy: requests sorted by cost, each given to the least-loaded rank.
    Every request index appears exactly once; within a rank the indices are returned in ascending order."""
    order = sorted(range(len(lengths)), key=lambda i: (-request_cost(lengths[i], hidden), i))
    load = [0.0] * world
    shards: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda k: (load[k], k))
        shards[r].append(i)
        load[r] += request_cost(lengths[i], hidden)
    return [sorted(s) for s in shards]


def imbalance(lengths: Sequence[int], shards: List[List[int]], hidden: int = 768) -> float:
    """max rank load / mean rank load (1.0 = perfect)."""
    loads = [sum(request_cost(lengths[i], hidden) for i in s) for s in shards]
    mean = sum(loads) / len(loads)
    return max(loads) / mean if mean > 0 else 1.0


def job_throughput(units_per_rank: Sequence[float], ms_per_rank: Sequence[float]) -> float:
    """Whole-job units per second: all ranks' units over the slowest rank's time."""
    return sum(units_per_rank) / (max(ms_per_rank) / 1e3)


def reduce_max_ms(ms: float, device=None) -> float:
    """Max over ranks of a duration (identity without an initialised process group)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(ms)
    t = torch.tensor([ms], dtype=torch.float64, device=device if device is not None else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_rows(local_rows, shards: List[List[int]], rank: int):
    """All-gathers per-request result rows (a [n_local, H] CPU tensor ordered like shards[rank]) into request order.
    Used by multi-GPU serving loops to hand results back in the order requests came in."""
    import torch
    import torch.distributed as dist
    world = len(shards)
    if world == 1 or not dist.is_initialized():
        return local_rows
    parts = [None] * world
    dist.all_gather_object(parts, local_rows)
    n = sum(len(s) for s in shards)
    out = torch.empty((n,) + tuple(local_rows.shape[1:]), dtype=local_rows.dtype)
    for r, s in enumerate(shards):
        for j, i in enumerate(s):
            out[i] = parts[r][j]
    return out
