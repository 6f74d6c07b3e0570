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


class OverlappedGradientReducer:
    """Gradient all-reduce that runs beside the backward pass.

    Parameters are packed, in reverse registration order (the order in which a backward pass
    finishes them), into fp32 buckets of about ``bucket_bytes``.  A hook on every parameter copies
    its finished gradient into the bucket; when a bucket is complete its all-reduce starts at once
    on the communication stream while the backward pass goes on producing the next one.  Buckets
    start strictly in bucket order, so that every rank issues the same sequence of collectives
    whatever order its autograd graph finishes in.  ``finish()`` -- call it after ``backward()`` --
    starts what has not started (parameters that got no gradient count as zeros), waits, and
    writes the summed (or averaged) gradients back into ``.grad``.

    With one rank, or without an initialised process group, the hooks do nothing.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], group=None, average: bool = True,
                 bucket_bytes: int = 32 << 20):
        self.params = [p for p in params if p.requires_grad]
        self.group, self.average = group, average
        self.active = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.world = dist.get_world_size(group) if self.active else 1
        self.buckets: List[dict] = []
        self._slot = {}
        cur, cur_bytes = [], 0
        for p in reversed(self.params):
            n = p.numel() * 4
            if cur and cur_bytes + n > bucket_bytes:
                self._close(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += n
        if cur:
            self._close(cur)
        self._handles = [p.register_post_accumulate_grad_hook(self._on_grad) for p in self.params] if self.active else []
        self._next = 0
        self.enabled = True     # False: the hooks ignore a backward pass (e.g. an instrumented step)

    def _close(self, plist):
        flat = torch.zeros(sum(p.numel() for p in plist), dtype=torch.float32, device=plist[0].device)
        index, off = len(self.buckets), 0
        for p in plist:
            self._slot[p] = (index, off)
            off += p.numel()
        self.buckets.append({"params": plist, "flat": flat, "missing": len(plist), "filled": set(), "work": None})

    def _on_grad(self, p):
        if not self.enabled:
            return
        index, off = self._slot[p]
        b = self.buckets[index]
        if p in b["filled"]:        # a second backward before finish(): .grad already accumulated, copy again
            b["flat"][off:off + p.numel()].copy_(p.grad.reshape(-1))
            return
        b["flat"][off:off + p.numel()].copy_(p.grad.reshape(-1))
        b["filled"].add(p)
        b["missing"] -= 1
        self._launch_ready()

    def _launch_ready(self):
        while self._next < len(self.buckets) and self.buckets[self._next]["missing"] == 0:
            b = self.buckets[self._next]
            b["work"] = dist.all_reduce(b["flat"], op=dist.ReduceOp.SUM, group=self.group, async_op=True)
            self._next += 1

    def finish(self):
        """Complete the step: every bucket reduced, ``.grad`` of every parameter replaced by the sum
        (or mean) over the ranks.  Resets the reducer for the next backward pass."""
        if not self.active:
            return
        for b in self.buckets:
            if b["missing"]:                       # parameters without a gradient this step: zeros
                for p in b["params"]:
                    if p not in b["filled"]:
                        index, off = self._slot[p]
                        b["flat"][off:off + p.numel()].zero_()
                b["missing"] = 0
        self._launch_ready()
        for b in self.buckets:
            b["work"].wait()
            if self.average:
                b["flat"].div_(self.world)
            off = 0
            for p in b["params"]:
                g = b["flat"][off:off + p.numel()].view_as(p)
                if p.grad is None:
                    p.grad = g.to(p.dtype).clone()
                else:
                    p.grad.copy_(g)
                off += p.numel()
            b["missing"], b["filled"], b["work"] = len(b["params"]), set(), None
        self._next = 0

    def remove(self):
        for h in self._handles:
            h.remove()
        self._handles = []
