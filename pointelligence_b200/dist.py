"""Data parallelism over ragged batches of scenes.

A batch of point clouds shards by whole scenes: edges never cross samples
(the sample id is part of every cell key), so each rank builds its own
geometry and the only exchange is the sum of parameter gradients -- one
bucketed all-reduce per step over ``torch.distributed`` (NCCL on GPUs, gloo in
the CPU tests).
"""
from __future__ import annotations

from typing import Iterable, List, Sequence

import torch
import torch.distributed as dist


def partition_scenes(sizes: Sequence[int], world_size: int, exponent: float = 1.0) -> List[List[int]]:
    """Longest-processing-time greedy assignment of scenes to ranks.

    ``sizes[s]`` is the point count of scene ``s``; cost is ``size ** exponent``.
    Returns, per rank, the ascending list of scene ids it owns.  Deterministic.
    """
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    order = sorted(range(len(sizes)), key=lambda s: (-float(sizes[s]) ** exponent, s))
    load = [0.0] * world_size
    owned: List[List[int]] = [[] for _ in range(world_size)]
    for s in order:
        r = min(range(world_size), key=lambda q: (load[q], q))
        owned[r].append(s)
        load[r] += float(sizes[s]) ** exponent
    return [sorted(o) for o in owned]


def allreduce_gradients(params: Iterable[torch.nn.Parameter], group=None, average: bool = True,
                        bucket_bytes: int = 32 << 20, async_op: bool = False):
    """Sum (or average) ``.grad`` of every parameter over the process group.

    Gradients are packed into fp32 buckets of about ``bucket_bytes`` so that a
    few large collectives replace one launch per tensor; parameters without a
    gradient contribute zeros so every rank issues the same collectives.
    Returns the list of work handles when ``async_op`` (call ``finish()`` on the
    returned object), else None.
    """
    params = [p for p in params if p.requires_grad]
    if not params or not dist.is_available() or not dist.is_initialized():
        return None
    world = dist.get_world_size(group)
    if world == 1:
        return None
    buckets, cur, cur_bytes = [], [], 0
    for p in params:
        n = p.numel() * 4
        if cur and cur_bytes + n > bucket_bytes:
            buckets.append(cur)
            cur, cur_bytes = [], 0
        cur.append(p)
        cur_bytes += n
    if cur:
        buckets.append(cur)
    pending = []
    for bucket in buckets:
        dev = bucket[0].device
        flat = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1).float()
                          for p in bucket]).to(dev)
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=True)
        pending.append((work, flat, bucket))

    class _Pending:
        def finish(self_inner):
            for work, flat, bucket in pending:
                work.wait()
                if average:
                    flat.div_(world)
                off = 0
                for p in bucket:
                    n = p.numel()
                    g = flat[off:off + n].view_as(p).to(p.dtype)
                    if p.grad is None:
                        p.grad = g.clone()
                    else:
                        p.grad.copy_(g)
                    off += n

    handle = _Pending()
    if async_op:
        return handle
    handle.finish()
    return None
