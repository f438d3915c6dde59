"""Data-parallel gradient reduction for the generic (autograd) training path.

The reference leaves gradients as DTensor ``Partial`` values and lets ``optimizer.step()`` all-reduce each of
them lazily, about three times per parameter per step (trainer.py:645-646 and the probe described for
``torch.optim.Adam``). Here the reduction is explicit: once per step, all gradients of the same dtype are
packed into flat buckets and averaged with one asynchronous all-reduce per bucket.
"""

from __future__ import annotations

from typing import Iterable

import torch
import torch.distributed as dist


@torch.no_grad()
def reduce_gradients(params: Iterable[torch.nn.Parameter], group, bucket_bytes: int = 256 << 20, average: bool = True) -> None:
    """Average (or sum) ``.grad`` of every parameter over ``group`` in place."""
    if group is None or dist.get_world_size(group) == 1:
        return
    world = dist.get_world_size(group)
    grads = [p.grad for p in params if p.grad is not None]
    buckets: list[list[torch.Tensor]] = []
    cur: list[torch.Tensor] = []
    cur_bytes, cur_dtype = 0, None
    for g in grads:
        nbytes = g.numel() * g.element_size()
        if cur and (g.dtype != cur_dtype or cur_bytes + nbytes > bucket_bytes):
            buckets.append(cur)
            cur, cur_bytes = [], 0
        cur.append(g)
        cur_bytes += nbytes
        cur_dtype = g.dtype
    if cur:
        buckets.append(cur)
    pending = []
    for bucket in buckets:
        flat = torch.cat([g.reshape(-1) for g in bucket])
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=True)
        pending.append((work, flat, bucket))
    for work, flat, bucket in pending:
        work.wait()
        if average:
            flat.div_(world)
        off = 0
        for g in bucket:
            n = g.numel()
            g.copy_(flat[off : off + n].view_as(g))
            off += n
