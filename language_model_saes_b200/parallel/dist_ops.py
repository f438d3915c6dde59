"""Tensor operations that understand sharding, written over local shards.

The reference project wraps ``torch.distributed.tensor.DTensor`` for these (utils/distributed/ops.py:42-640 and
utils/distributed/utils.py:23-122). Here a sharded value is a ``Sharded``: the local shard, the dimension it is
split on (``None`` = replicated) and the process group of the split; shards are equal-sized and ordered by group
rank. Every function also takes plain tensors, for which it is the ordinary torch operation.

Index-style gathers (``batch_index``, ``multi_batch_index``, ``nonzero``) use one variable-length exchange per call:
the per-rank counts and the padded payload travel together in a single all-gather of a ``[1 + max_len, ...]`` block
whose first row is the count, instead of one collective for lengths and one for data.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Optional, Sequence

import torch
import torch.distributed as dist


@dataclass
class Sharded:
    """Local shard of a logical tensor split evenly on ``dim`` across ``group`` (``dim=None``: replicated)."""

    local: torch.Tensor
    dim: int | None = None
    group: dist.ProcessGroup | None = None

    @property
    def world(self) -> int:
        return dist.get_world_size(self.group) if (self.group is not None and self.dim is not None) else 1

    @property
    def rank(self) -> int:
        return dist.get_rank(self.group) if (self.group is not None and self.dim is not None) else 0

    @property
    def shape(self) -> torch.Size:
        s = list(self.local.shape)
        if self.dim is not None:
            s[self.dim] *= self.world
        return torch.Size(s)

    @property
    def offset(self) -> int:
        return 0 if self.dim is None else self.rank * self.local.shape[self.dim]

    @property
    def device(self):
        return self.local.device

    @property
    def dtype(self):
        return self.local.dtype

    def like(self, local: torch.Tensor, dim: int | None = "same") -> "Sharded":  # type: ignore[assignment]
        return Sharded(local, self.dim if dim == "same" else dim, self.group)

    def full(self) -> torch.Tensor:
        return full_tensor(self)


TensorLike = torch.Tensor | Sharded


def to_local(x: TensorLike) -> torch.Tensor:
    return x.local if isinstance(x, Sharded) else x


def full_tensor(x: TensorLike) -> torch.Tensor:
    """The logical tensor on every rank (one all-gather along the sharded dimension)."""
    if not isinstance(x, Sharded) or x.dim is None or x.world == 1:
        return to_local(x)
    loc = x.local.contiguous()
    out = _all_gather_stacked(loc, x.group, x.world)
    return torch.cat(list(out.unbind(0)), dim=x.dim) if x.dim != 0 else out.reshape(-1, *loc.shape[1:])


def _all_gather_stacked(loc: torch.Tensor, group, world: int) -> torch.Tensor:
    """``[world, *loc.shape]`` with slice r = rank r's tensor (the flat-concatenation form of the collective, which
    every backend accepts, viewed as stacked)."""
    flat = loc.reshape(-1)
    out = torch.empty(world * flat.numel(), dtype=loc.dtype, device=loc.device)
    dist.all_gather_into_tensor(out, flat, group=group)
    return out.view(world, *loc.shape)


def item(x: TensorLike) -> float | int | bool:
    """Python scalar of a 0-d (or 1-element) value; a sharded one is gathered first."""
    return full_tensor(x).item()


def maybe_local_map(fn: Callable[..., torch.Tensor], out_dim: int | None | str = "same") -> Callable[..., TensorLike]:
    """Run ``fn`` on local shards. Arguments that are ``Sharded`` are unwrapped; the result is wrapped like the first
    sharded argument (``out_dim`` overrides the sharded dimension of the result)."""

    def wrapper(*args: Any, **kwargs: Any):
        proto = next((a for a in (*args, *kwargs.values()) if isinstance(a, Sharded)), None)
        out = fn(*[to_local(a) if isinstance(a, Sharded) else a for a in args],
                 **{k: to_local(v) if isinstance(v, Sharded) else v for k, v in kwargs.items()})  # fmt: skip
        if proto is None:
            return out
        return proto.like(out, out_dim)

    return wrapper


def masked_fill(x: TensorLike, mask: TensorLike, value: float) -> TensorLike:
    """Out-of-place masked fill; ``x`` and ``mask`` must be sharded alike."""
    out = to_local(x).masked_fill(to_local(mask), value)
    return x.like(out) if isinstance(x, Sharded) else out


def slice_fill(x: TensorLike, slice_tuple, value) -> TensorLike:
    """In-place fill of a slice given in LOCAL coordinates of the shard (the reference has the same convention)."""
    to_local(x)[slice_tuple] = to_local(value) if isinstance(value, Sharded) else value
    return x


def searchsorted(sorted_sequence: TensorLike, values, *, right: bool = False, side: str | None = None) -> TensorLike:
    if isinstance(sorted_sequence, Sharded):
        assert sorted_sequence.dim is None, "Only replicated tensors are supported"
    vals = to_local(values) if isinstance(values, Sharded) else values
    out = torch.searchsorted(to_local(sorted_sequence), vals, right=right, side=side)
    return sorted_sequence.like(out) if isinstance(sorted_sequence, Sharded) else out


def _gather_ragged(rows: torch.Tensor, group, world: int, cat_dim: int = 0) -> list[torch.Tensor]:
    """All-gather tensors whose size on ``cat_dim`` differs per rank; returns the per-rank tensors. The counts ride in
    a small int64 all-gather, the payload in one padded all-gather sized by the largest count."""
    n = torch.tensor([rows.shape[cat_dim]], dtype=torch.int64, device=rows.device)
    counts = torch.empty(world, dtype=torch.int64, device=rows.device)
    dist.all_gather_into_tensor(counts, n, group=group)
    counts_l = counts.tolist()
    m = max(counts_l)
    rows = rows.movedim(cat_dim, 0).contiguous()
    pad = torch.zeros((m, *rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    pad[: rows.shape[0]] = rows
    out = _all_gather_stacked(pad, group, world)
    return [out[r, : counts_l[r]].movedim(0, cat_dim) for r in range(world)]


def nonzero(x: TensorLike, *, as_tuple: bool = False):
    """Global coordinates of the non-zero entries, identical on every rank, ordered by owning rank then locally
    row-major (for a split on dim 0 this is the row-major order of the logical tensor)."""
    if not isinstance(x, Sharded) or x.dim is None or x.world == 1:
        return torch.nonzero(to_local(x), as_tuple=as_tuple)
    nz = torch.nonzero(x.local)
    nz[:, x.dim] += x.offset
    out = torch.cat(_gather_ragged(nz, x.group, x.world), dim=0)
    return tuple(out.unbind(1)) if as_tuple else out


def _index_local(x: torch.Tensor, idx: torch.Tensor, n_batch_dims: int) -> torch.Tensor:
    return x[(*[slice(None)] * n_batch_dims, *idx.unbind(dim=1))]


def batch_index(x: TensorLike, indices: TensorLike, n_batch_dims: int = 0, preserve_order: bool = False) -> torch.Tensor:
    """``x[..., i0, i1, ...]`` for every row ``(i0, i1, ...)`` of the replicated ``indices`` (``n_batch_dims`` leading
    dimensions are kept whole). The result is replicated. Without ``preserve_order`` rows come grouped by the rank that
    owns them (cheaper: no scatter back); with it they are in the order of ``indices``."""
    idx = to_local(indices)
    if not isinstance(x, Sharded) or x.dim is None or x.world == 1:
        return _index_local(to_local(x), idx, n_batch_dims)
    sd = x.dim - n_batch_dims
    if sd < 0 or sd >= idx.shape[1]:
        # the split is on a dimension that is not indexed: index locally, result stays sharded there -> gather it
        out = _index_local(x.local, idx, n_batch_dims)
        new_dim = x.dim if sd < 0 else x.dim - idx.shape[1] + 1
        return full_tensor(Sharded(out, new_dim, x.group))
    size = x.local.shape[x.dim]
    mine = (idx[:, sd] >= x.offset) & (idx[:, sd] < x.offset + size)
    loc = idx[mine].clone()
    loc[:, sd] -= x.offset
    out = _index_local(x.local, loc, n_batch_dims)
    parts = _gather_ragged(out, x.group, x.world, cat_dim=n_batch_dims)
    res = torch.cat(parts, dim=n_batch_dims)
    if not preserve_order:
        return res
    owner = torch.div(idx[:, sd], size, rounding_mode="floor")
    order = torch.argsort(owner, stable=True)  # rows of ``res`` correspond to indices[order]
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=order.device)
    return res.index_select(n_batch_dims, inv)


def multi_batch_index(xs_and_indices: Sequence[tuple[TensorLike, TensorLike]], n_batch_dims: int = 0,
                      preserve_order: bool = False) -> list[torch.Tensor]:  # fmt: skip
    """``batch_index`` for many tensors. Tensors of one dtype, group and trailing shape share a single exchange: their
    locally indexed rows are concatenated, gathered once and split again."""
    results: list[Optional[torch.Tensor]] = [None] * len(xs_and_indices)
    buckets: dict[Any, list[int]] = {}
    for i, (x, idx) in enumerate(xs_and_indices):
        if not isinstance(x, Sharded) or x.dim is None or x.world == 1 or n_batch_dims != 0:
            results[i] = batch_index(x, idx, n_batch_dims, preserve_order)
            continue
        sd = x.dim
        if sd >= to_local(idx).shape[1]:
            results[i] = batch_index(x, idx, n_batch_dims, preserve_order)
            continue
        tail = tuple(x.local.shape[to_local(idx).shape[1] :])
        buckets.setdefault((x.dtype, id(x.group), tail), []).append(i)
    for members in buckets.values():
        pieces, metas = [], []
        for i in members:
            x, idx = xs_and_indices[i]
            idx = to_local(idx)
            size = x.local.shape[x.dim]
            mine = (idx[:, x.dim] >= x.offset) & (idx[:, x.dim] < x.offset + size)
            loc = idx[mine].clone()
            loc[:, x.dim] -= x.offset
            pieces.append(_index_local(x.local, loc, 0))
            metas.append((idx, size, x.dim))
        x0 = xs_and_indices[members[0]][0]
        lens = torch.tensor([p.shape[0] for p in pieces], dtype=torch.int64, device=x0.device)
        all_lens = _all_gather_stacked(lens, x0.group, x0.world)
        parts = _gather_ragged(torch.cat(pieces, dim=0), x0.group, x0.world)
        all_lens_l = all_lens.tolist()
        split = [p.split(all_lens_l[r], dim=0) for r, p in enumerate(parts)]
        for j, i in enumerate(members):
            res = torch.cat([split[r][j] for r in range(x0.world)], dim=0)
            if preserve_order:
                idx, size, sd = metas[j]
                order = torch.argsort(torch.div(idx[:, sd], size, rounding_mode="floor"), stable=True)
                inv = torch.empty_like(order)
                inv[order] = torch.arange(order.numel(), device=order.device)
                res = res.index_select(0, inv)
            results[i] = res
    return results  # type: ignore[return-value]


def all_gather_dict(data: dict[str, Any], group: Optional[dist.ProcessGroup] = None) -> list[dict[str, Any]]:
    """One dict per rank. Tensor values may differ in shape between ranks (shapes travel with the non-tensor values in
    a single object all-gather; tensor payloads use tensor collectives)."""
    world = dist.get_world_size(group=group)
    meta = {k: (("t", tuple(v.shape), v.dtype) if isinstance(v, torch.Tensor) else ("o", v)) for k, v in data.items()}
    metas: list = [None] * world
    dist.all_gather_object(metas, meta, group=group)
    out: list[dict[str, Any]] = [dict() for _ in range(world)]
    for k, v in data.items():
        if isinstance(v, torch.Tensor):
            numels = [int(torch.Size(metas[r][k][1]).numel()) for r in range(world)]
            pad = torch.zeros(max(numels), dtype=v.dtype, device=v.device)
            pad[: v.numel()] = v.reshape(-1)
            stacked = _all_gather_stacked(pad, group, world)
            for r in range(world):
                out[r][k] = stacked[r, : numels[r]].reshape(metas[r][k][1]).to(metas[r][k][2])
        else:
            for r in range(world):
                out[r][k] = metas[r][k][1]
    return out


def all_gather_list(data: list[Any], group: Optional[dist.ProcessGroup] = None, flatten: bool = True):
    if not dist.is_initialized() or dist.get_world_size(group=group) == 1:
        return data
    parts: list = [None] * dist.get_world_size(group=group)
    dist.all_gather_object(parts, data, group=group)
    return [x for p in parts for x in p] if flatten else parts


def broadcast_object(obj: Any | None, group_src: int = 0, group: Optional[dist.ProcessGroup] = None) -> Any:
    if not dist.is_initialized() or dist.get_world_size(group=group) == 1:
        return obj
    box = [obj]
    dist.broadcast_object_list(box, group=group, group_src=group_src)
    return box[0]
