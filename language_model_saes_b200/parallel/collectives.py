"""Autograd-aware collectives over mesh dimensions, and the cross-shard top-k.

Models hold local shards and call these explicitly:

* ``all_reduce_sum(x, group)``: forward sums over the group; backward passes the gradient through (each
  rank's partial contributes linearly to the sum, so d out / d partial = identity). This is what the
  reference obtains implicitly from ``DTensor.redistribute(Partial -> Replicate)`` after the decoder matmul
  (models/sae.py:374-375 there).
* ``distributed_topk(x_local, k, group)``: per-row (or whole-batch) top-k over a feature axis that is
  sharded across ``group``. The reference finds the threshold with an up-to-50-step bisection, three
  all-reduces and several host syncs per step (utils/distributed/ops.py:158-266). Here every rank
  contributes its k local maxima, one all-gather makes the tp*k candidates visible everywhere, and the
  global k-th value is read off: one collective, no host sync, exact.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


class _AllReduceSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, group):
        out = x.contiguous().clone()
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        return grad, None


class _IdentityFwdAllReduceBwd(torch.autograd.Function):
    """Forward identity on a tensor replicated in ``group``; backward sums the gradients of the ranks
    (each rank used the replicated value in its own shard of the computation)."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, grad):
        g = grad.contiguous().clone()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


class _AllReduceSumBoth(torch.autograd.Function):
    """Sum over the group in forward AND backward: for a value that every rank then uses in its own, different
    part of the computation (e.g. the head-summed crosscoder pre-activations), so that the gradients of the
    ranks have to be added up as well."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, group):
        ctx.group = group
        out = x.contiguous().clone()
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        g = grad.contiguous().clone()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


def all_reduce_sum_both(x: torch.Tensor, group) -> torch.Tensor:
    if group is None or dist.get_world_size(group) == 1:
        return x
    return _AllReduceSumBoth.apply(x, group)


def all_reduce_sum(x: torch.Tensor, group) -> torch.Tensor:
    if group is None or dist.get_world_size(group) == 1:
        return x
    return _AllReduceSum.apply(x, group)


def copy_to_group(x: torch.Tensor, group) -> torch.Tensor:
    if group is None or dist.get_world_size(group) == 1:
        return x
    return _IdentityFwdAllReduceBwd.apply(x, group)


def all_gather_cat(x: torch.Tensor, group, dim: int = 0) -> torch.Tensor:
    """Non-differentiable all-gather + concatenate along ``dim``."""
    if group is None or dist.get_world_size(group) == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=dim)


@torch.no_grad()
def distributed_threshold(score: torch.Tensor, k: int, group) -> torch.Tensor:
    """k-th largest value per leading index of ``score`` [..., n_local] over the union of all shards.

    Returns a tensor shaped like ``score[..., :1]``; entries ``>=`` it are the global top-k (ties keep more
    than k, as the reference's threshold formulation does).
    """
    n_local = score.shape[-1]
    tp = dist.get_world_size(group) if group is not None else 1
    k_local = min(k, n_local)
    local_top = torch.topk(score, k_local, dim=-1).values
    if k_local < k:
        pad = score.new_full((*score.shape[:-1], k - k_local), float("-inf"))
        local_top = torch.cat([local_top, pad], dim=-1)
    cands = all_gather_cat(local_top, group, dim=-1) if tp > 1 else local_top
    kk = min(k, cands.shape[-1])
    return torch.topk(cands, kk, dim=-1).values[..., -1:]


def distributed_topk(
    x: torch.Tensor, k: int, group, dim: int | tuple[int, ...] = -1, *, positive_only: bool = True
) -> torch.Tensor:
    """Mask-multiply top-k with straight-through gradient where the LAST listed dim is sharded over ``group``.

    ``dim`` may name several dimensions (e.g. ``(-2, -1)`` = batch-level top-k); they are flattened for the
    selection. Only positive entries can be selected when ``positive_only`` (the reference's bisection starts
    at zero, so non-positive values never pass).
    """
    dims = (dim,) if isinstance(dim, int) else tuple(dim)
    dims = tuple(d % x.ndim for d in dims)
    keep = tuple(d for d in range(x.ndim) if d not in dims)
    perm = keep + dims
    xp = x.permute(perm)
    lead = xp.shape[: len(keep)]
    flat = xp.reshape(*lead, -1)
    with torch.no_grad():
        score = flat.float()
        if positive_only:
            score = torch.where(score > 0, score, torch.zeros_like(score))
        thr = distributed_threshold(score, k, group)
        mask = score >= thr
        if positive_only:
            mask &= score > 0
    out = (flat * mask.to(flat.dtype)).reshape(xp.shape)
    inv = [0] * len(perm)
    for i, p in enumerate(perm):
        inv[p] = i
    return out.permute(inv)
