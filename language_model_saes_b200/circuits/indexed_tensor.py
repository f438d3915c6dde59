"""Tensors whose axes are labelled by graph nodes.

A node is ``(key, index tuple)``: ``key`` names a tensor of the computation (a hook point, ``"logits"``, ...), the
index tuple selects one element of it. ``NodeDimension`` is an ordered list of nodes and labels one tensor axis;
``NodeIndexedTensor`` / ``Vector`` / ``Matrix`` carry data plus one ``NodeDimension`` per axis. Same API and semantics
as circuits/indexed_tensor.py of the reference project (:37-861).

Storage differs: instead of one ``Node`` object per key with a dense inverse-lookup table spanning the whole index
range of that key (which for ``(position, feature)`` indices of a large dictionary is ``positions x d_sae`` entries),
a dimension is two flat device tensors, ``key_ids [n]`` and ``indices [n, D]`` (index tuples right-padded with zeros
to the widest rank ``D``), and lookups go through ONE sorted int64 code per node (mixed radix over key id and index
columns) with ``torch.searchsorted``. Memory is O(n) whatever the index ranges are, and every operation is a handful of
vectorised kernels without a per-key Python loop.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Generic, Iterator, Self, Sequence, TypeVar

import torch
from torch import Tensor

from ..core.pytree import PyTree
from ..utils.timer import timer

Number = int | float | bool


@dataclass
class NodeInfo(PyTree):
    """Some elements of one tensor of the graph: ``indices [n_elements, d_index]``."""

    key: Any
    indices: Tensor

    @property
    def is_identity(self) -> bool:
        """True when the indices enumerate a whole grid ``0..max`` in row-major order."""
        idx = self.indices
        if idx.numel() == 0:
            return False
        extent = (idx.max(dim=0).values + 1).tolist()
        n = 1
        for e in extent:
            n *= int(e)
        if n != idx.shape[0]:
            return False
        grid = torch.stack(torch.meshgrid(*[torch.arange(int(e), device=idx.device) for e in extent], indexing="ij"), dim=-1)
        return bool(torch.equal(idx, grid.reshape(-1, idx.shape[1])))

    def __len__(self) -> int:
        return self.indices.shape[0]

    def __eq__(self, other: object) -> bool:
        return isinstance(other, NodeInfo) and self.key == other.key and torch.equal(self.indices, other.indices)

    def __getitem__(self, index: slice) -> Self:
        return type(self)(self.key, self.indices[index])

    def split(self, batch_size: int) -> tuple[Self, Self]:
        return self[:batch_size], self[batch_size:]

    def unbind(self) -> list[Self]:
        return [self[i : i + 1] for i in range(len(self))]

    def __iter__(self) -> Iterator[Self]:
        return iter(self.unbind())


class _Lookup:
    """Sorted codes of a dimension's nodes. A node's code is ``((key_id * r_0 + i_0) * r_1 + i_1) ...`` with the
    radices ``r_c = 1 + max index in column c``; anything outside those ranges cannot be a member."""

    def __init__(self, key_ids: Tensor, indices: Tensor):
        self.radix = (indices.max(dim=0).values + 1).clamp(min=1) if indices.numel() else torch.ones(indices.shape[1], dtype=torch.long, device=indices.device)
        span = 1
        for r in self.radix.tolist():
            span *= int(r)
        n_keys = int(key_ids.max()) + 1 if key_ids.numel() else 1
        self.exact = span * n_keys < 2**62
        codes = self.encode(key_ids, indices)[0]
        self.sorted_codes, self.order = torch.sort(codes, stable=True)

    def encode(self, key_ids: Tensor, indices: Tensor) -> tuple[Tensor, Tensor]:
        """(codes, in_range). With ranges too wide for 62 bits the code is a mixing hash and membership is confirmed by
        comparing the rows afterwards."""
        in_range = ((indices >= 0) & (indices < self.radix)).all(dim=1) & (key_ids >= 0)
        if self.exact:
            code = key_ids.clamp(min=0)
            for c in range(indices.shape[1]):
                code = code * self.radix[c] + indices[:, c].clamp(min=0, max=int(self.radix[c]) - 1)
            return code, in_range
        code = key_ids.clamp(min=0) * 0x9E3779B1
        for c in range(indices.shape[1]):
            code = (code ^ (code >> 29)) * 0x5851F42D + indices[:, c]
        return code & 0x3FFFFFFFFFFFFFFF, in_range


@dataclass
class NodeDimension(PyTree):
    """Ordered list of nodes; position in the list = offset along the labelled axis."""

    keys: list[Any]
    """Distinct keys in order of first appearance."""
    key_ids: Tensor
    """``[n]`` int64, position of each node's key in ``keys``."""
    indices: Tensor
    """``[n, D]`` int64 index tuples, zero-padded on the right to the widest rank."""
    ranks: list[int]
    """Length of the index tuple of each key."""
    device_mesh: Any = field(default=None, repr=False, compare=False)
    _lookup: Any = field(default=None, repr=False, compare=False)
    _n2o_cache: dict = field(default_factory=dict, repr=False, compare=False)

    # ---- construction ------------------------------------------------------------------------
    @classmethod
    def empty(cls, device: torch.device | str, device_mesh=None) -> Self:
        z = torch.empty(0, dtype=torch.long, device=device)
        return cls([], z, z.reshape(0, 1), [], device_mesh)

    @classmethod
    def from_node_infos(cls, node_infos: Sequence[NodeInfo], device: torch.device | str | None = None, device_mesh=None) -> Self:
        if len(node_infos) == 0:
            if device is None:
                raise ValueError("Cannot build NodeDimension from empty `node_infos` without an explicit device.")
            return cls.empty(device, device_mesh)
        device = device if device is not None else node_infos[0].indices.device
        keys: list[Any] = []
        ranks: list[int] = []
        pos: dict[Any, int] = {}
        for ni in node_infos:
            if ni.key not in pos:
                pos[ni.key] = len(keys)
                keys.append(ni.key)
                ranks.append(ni.indices.shape[1])
            else:
                assert ranks[pos[ni.key]] == ni.indices.shape[1], f"index rank of key {ni.key!r} changed"
        width = max(ranks)
        key_ids = torch.cat([torch.full((len(ni),), pos[ni.key], dtype=torch.long, device=device) for ni in node_infos])
        indices = torch.cat([torch.nn.functional.pad(ni.indices.to(device=device, dtype=torch.long), (0, width - ni.indices.shape[1])) for ni in node_infos])
        return cls(keys, key_ids, indices, ranks, device_mesh)

    @property
    def device(self):
        return self.indices.device

    def _with(self, key_ids: Tensor, indices: Tensor) -> Self:
        """Same key table, other nodes; unused keys are dropped so that ``keys`` lists only keys that occur."""
        used = torch.unique(key_ids).tolist() if key_ids.numel() else []
        if len(used) == len(self.keys):
            return type(self)(list(self.keys), key_ids, indices, list(self.ranks), self.device_mesh)
        # keep first-appearance order of the remaining nodes
        first = {}
        for k in key_ids.tolist() if key_ids.numel() < 4096 else self._first_order(key_ids):
            first.setdefault(k, len(first))
        remap = torch.full((len(self.keys),), -1, dtype=torch.long, device=key_ids.device)
        for old, new in first.items():
            remap[old] = new
        keys = [self.keys[o] for o in first]
        ranks = [self.ranks[o] for o in first]
        width = max(ranks) if ranks else 1
        return type(self)(keys, remap[key_ids], indices[:, :width], ranks, self.device_mesh)

    @staticmethod
    def _first_order(key_ids: Tensor) -> list[int]:
        uniq, inv = torch.unique(key_ids, return_inverse=True)
        first_pos = torch.full((uniq.numel(),), key_ids.numel(), dtype=torch.long, device=key_ids.device)
        first_pos.scatter_reduce_(0, inv, torch.arange(key_ids.numel(), device=key_ids.device), reduce="amin")
        return uniq[torch.argsort(first_pos)].tolist()

    # ---- views -------------------------------------------------------------------------------
    def __len__(self) -> int:
        return self.key_ids.shape[0]

    def __hash__(self) -> int:
        return hash((tuple(map(str, self.keys)), self.key_ids.data_ptr(), self.indices.data_ptr(), len(self)))

    def __eq__(self, other: object) -> bool:
        return (isinstance(other, NodeDimension) and len(self) == len(other)
                and [self.keys[i] for i in self.key_ids.tolist()] == [other.keys[i] for i in other.key_ids.tolist()]
                and torch.equal(self._padded(max(self.indices.shape[1], other.indices.shape[1])),
                                other._padded(max(self.indices.shape[1], other.indices.shape[1]))))  # fmt: skip

    def _padded(self, width: int) -> Tensor:
        return torch.nn.functional.pad(self.indices, (0, width - self.indices.shape[1]))

    @property
    def node_infos(self) -> list[NodeInfo]:
        """Maximal runs of consecutive nodes with the same key, in order."""
        if len(self) == 0:
            return []
        change = torch.ones(len(self), dtype=torch.bool, device=self.device)
        change[1:] = self.key_ids[1:] != self.key_ids[:-1]
        starts = change.nonzero().squeeze(-1).tolist() + [len(self)]
        ids = self.key_ids[starts[:-1]].tolist()
        return [NodeInfo(self.keys[k], self.indices[a:b, : self.ranks[k]]) for k, a, b in zip(ids, starts[:-1], starts[1:])]

    @property
    def node_mappings(self) -> dict[Any, NodeInfo]:
        """Per key, all its index tuples (in order of appearance)."""
        return {key: NodeInfo(key, self.indices[self.key_ids == i, : self.ranks[i]]) for i, key in enumerate(self.keys)}

    def offsets_of_key(self, key: Any) -> Tensor:
        return (self.key_ids == self.keys.index(key)).nonzero().squeeze(-1) if key in self.keys else torch.empty(0, dtype=torch.long, device=self.device)

    def __iter__(self) -> Iterator[NodeInfo]:
        ids = self.key_ids.tolist()
        for i, k in enumerate(ids):
            yield NodeInfo(self.keys[k], self.indices[i : i + 1, : self.ranks[k]])

    # ---- algebra -----------------------------------------------------------------------------
    def _translate(self, other: "NodeDimension") -> Tensor:
        """``other``'s key ids expressed in this dimension's key table (-1 for keys this dimension lacks)."""
        table = torch.tensor([self.keys.index(k) if k in self.keys else -1 for k in other.keys] or [-1], dtype=torch.long, device=self.device)
        return table[other.key_ids.to(self.device)] if len(other) else torch.empty(0, dtype=torch.long, device=self.device)

    def __add__(self, other: "NodeDimension") -> "NodeDimension":
        if len(other) == 0:
            return self
        if len(self) == 0:
            return other
        keys, ranks = list(self.keys), list(self.ranks)
        table = []
        for k, r in zip(other.keys, other.ranks):
            if k in keys:
                assert ranks[keys.index(k)] == r, f"index rank of key {k!r} differs"
                table.append(keys.index(k))
            else:
                table.append(len(keys))
                keys.append(k)
                ranks.append(r)
        width = max(ranks)
        ids = torch.cat([self.key_ids, torch.tensor(table, dtype=torch.long, device=self.device)[other.key_ids.to(self.device)]])
        idx = torch.cat([self._padded(width), other._padded(width).to(self.device)])
        return type(self)(keys, ids, idx, ranks, self.device_mesh)

    def __sub__(self, other: "NodeDimension") -> "NodeDimension":
        """Nodes of ``self`` that are not in ``other`` (order kept)."""
        if len(other) == 0 or len(self) == 0:
            return self
        return self.offsets_to_nodes((other.nodes_to_offsets(self) == -1).nonzero().squeeze(-1))

    @timer.time("nodes_to_offsets")
    def nodes_to_offsets(self, dimension: "NodeDimension") -> Tensor:
        """For every node of ``dimension`` its offset in ``self``, or -1 when ``self`` does not contain it."""
        ck = hash(dimension)
        hit = self._n2o_cache.get(ck)
        if hit is not None and hit.shape[0] == len(dimension):
            return hit
        out = torch.full((len(dimension),), -1, dtype=torch.long, device=self.device)
        if len(self) and len(dimension):
            if self._lookup is None:
                self._lookup = _Lookup(self.key_ids, self.indices)
            lk: _Lookup = self._lookup
            width = self.indices.shape[1]
            q_idx = dimension.indices.to(self.device)
            extra_zero = (q_idx[:, width:] == 0).all(dim=1) if q_idx.shape[1] > width else None
            q_idx = torch.nn.functional.pad(q_idx[:, :width], (0, max(0, width - q_idx.shape[1])))
            q_ids = self._translate(dimension)
            codes, ok = lk.encode(q_ids, q_idx)
            if extra_zero is not None:
                ok = ok & extra_zero
            pos = torch.searchsorted(lk.sorted_codes, codes).clamp(max=len(self) - 1)
            cand = lk.order[pos]
            ok = ok & (lk.sorted_codes[pos] == codes)
            if not lk.exact:
                ok = ok & (self.key_ids[cand] == q_ids) & (self.indices[cand] == q_idx).all(dim=1)
            out = torch.where(ok, cand, out)
        self._n2o_cache[ck] = out
        return out

    @timer.time("offsets_to_nodes")
    def offsets_to_nodes(self, offsets: Tensor) -> "NodeDimension":
        """The nodes at ``offsets``, in that order."""
        if offsets.numel() == 0:
            return type(self).empty(self.device, self.device_mesh)
        offsets = offsets.to(self.device)
        return self._with(self.key_ids[offsets], self.indices[offsets])

    def filter(self, predicate: Callable[[NodeInfo], bool]) -> Self:
        """Keep the keys whose whole group (``NodeInfo`` of all its indices) satisfies ``predicate``."""
        keep = [i for i, (key, ni) in enumerate(self.node_mappings.items()) if predicate(ni)]
        return self._keep_keys(keep)

    @timer.time("filter_keys")
    def filter_keys(self, predicate: Callable[[Any], bool]) -> Self:
        return self._keep_keys([i for i, k in enumerate(self.keys) if predicate(k)])

    def _keep_keys(self, keep: list[int]) -> Self:
        if not keep:
            return type(self).empty(self.device, self.device_mesh)
        mask = torch.isin(self.key_ids, torch.tensor(keep, dtype=torch.long, device=self.device))
        # grouped by key like the reference (which rebuilds from per-key groups)
        order = torch.argsort(self.key_ids[mask], stable=True)
        return self._with(self.key_ids[mask][order], self.indices[mask][order])

    @timer.time("unique")
    def unique(self) -> Self:
        """Distinct nodes, grouped by key (in key-table order) and sorted by index inside a key."""
        if len(self) == 0:
            return self
        rows = torch.unique(torch.cat([self.key_ids[:, None], self.indices], dim=1), dim=0)
        return self._with(rows[:, 0].contiguous(), rows[:, 1:].contiguous())

    def to(self, device: torch.device | str) -> Self:
        return type(self)(list(self.keys), self.key_ids.to(device), self.indices.to(device), list(self.ranks), None)

    def full_tensor(self) -> Self:
        return type(self)(list(self.keys), self.key_ids, self.indices, list(self.ranks), None)

    # ---- serialisation: {key: {"indices": [m, d], "offsets": [m]}} ------------------------------
    def __unstructure__(self) -> dict[str, Any]:
        out = {}
        for i, key in enumerate(self.keys):
            sel = (self.key_ids == i).nonzero().squeeze(-1)
            out[key] = {"key": key, "indices": self.indices[sel, : self.ranks[i]], "offsets": sel}
        return out

    @classmethod
    def __structure__(cls, data: dict[str, Any]) -> Self:
        if not data:
            return cls.empty("cpu")
        keys = list(data.keys())
        ranks = [int(data[k]["indices"].shape[1]) for k in keys]
        n = sum(int(data[k]["offsets"].numel()) for k in keys)
        dev = data[keys[0]]["indices"].device
        key_ids = torch.empty(n, dtype=torch.long, device=dev)
        indices = torch.zeros(n, max(ranks), dtype=torch.long, device=dev)
        for i, k in enumerate(keys):
            off = data[k]["offsets"].long()
            key_ids[off] = i
            indices[off, : ranks[i]] = data[k]["indices"].long()
        return cls(keys, key_ids, indices, ranks)


def _as_dimension(d, device) -> NodeDimension:
    return d if isinstance(d, NodeDimension) else NodeDimension.from_node_infos(d, device=device)


@dataclass
class NodeIndexedTensor(PyTree):
    """A tensor with one ``NodeDimension`` per axis."""

    n_dims: int
    data: Tensor
    dimensions: tuple[NodeDimension, ...]

    @classmethod
    def from_data(cls, data: Tensor, dimensions: tuple[Sequence[NodeInfo] | NodeDimension, ...]) -> Self:
        dims = tuple(_as_dimension(d, data.device) for d in dimensions)
        assert all(len(d) == data.shape[i] for i, d in enumerate(dims)), "Data length must match dimension length"
        return cls(data.ndim, data, dims)

    @classmethod
    def from_dimensions(cls, dimensions: tuple[Sequence[NodeInfo] | NodeDimension, ...], device: torch.device | str = "cpu",
                        dtype: torch.dtype = torch.float32, device_mesh=None) -> Self:  # fmt: skip
        dims = tuple(_as_dimension(d, device) for d in dimensions)
        return cls.from_data(torch.zeros([len(d) for d in dims], dtype=dtype, device=device), dims)

    @timer.time("extend")
    def extend(self, dimension: NodeDimension, dim: int, data: Tensor | None = None):
        """Append nodes (and their data, zeros by default) along axis ``dim``."""
        shape = tuple(len(dimension) if i == dim else s for i, s in enumerate(self.data.shape))
        if data is None:
            data = torch.zeros(shape, dtype=self.data.dtype, device=self.data.device)
        assert tuple(data.shape) == shape, f"Data shape mismatches expected shape: {tuple(data.shape)} != {shape}"
        self.data = torch.cat([self.data, data], dim=dim)
        self.dimensions = tuple(d + dimension if i == dim else d for i, d in enumerate(self.dimensions))

    def _selectors(self, key) -> tuple[NodeDimension | None, ...]:
        key = key if isinstance(key, tuple) else (key,)
        if len(key) != self.n_dims:
            raise ValueError(f"Expected {self.n_dims} dimension selectors, got {len(key)}")
        return key

    @timer.time("__getitem__")
    @torch.no_grad()
    def __getitem__(self, key: tuple[NodeDimension | None, ...] | NodeDimension | None) -> Self:
        """One selector per axis: a ``NodeDimension`` picks those nodes (in its order), ``None`` keeps the axis."""
        key = self._selectors(key)
        data = self.data
        for dim, sel in enumerate(key):
            if sel is not None:
                data = data.index_select(dim, self.dimensions[dim].nodes_to_offsets(sel))
        return type(self).from_data(data, tuple(sel if sel is not None else self.dimensions[i] for i, sel in enumerate(key)))

    @timer.time("__setitem__")
    @torch.no_grad()
    def __setitem__(self, key, value: "NodeIndexedTensor | Tensor | Number"):
        key = self._selectors(key)
        value = value.data if isinstance(value, NodeIndexedTensor) else value
        indexers = []
        for dim, sel in enumerate(key):
            off = self.dimensions[dim].nodes_to_offsets(sel) if sel is not None else torch.arange(self.data.shape[dim], device=self.data.device)
            shape = [1] * self.n_dims
            shape[dim] = off.shape[0]
            indexers.append(off.view(*shape))
        self.data[tuple(indexers)] = value
        return self

    def __add__(self, other: Self) -> Self:
        return type(self).from_data(self.data + other.data, self.dimensions)

    def map(self, function: Callable[[Tensor], Tensor]) -> Self:
        return type(self).from_data(function(self.data), self.dimensions)

    def clone(self) -> Self:
        return type(self).from_data(self.data.clone(), self.dimensions)

    def __and__(self, other: Self) -> Self:
        return type(self).from_data(self.data & other.data, self.dimensions)

    def __invert__(self) -> Self:
        return type(self).from_data(~self.data, self.dimensions)

    @timer.time("nonzero")
    def nonzero(self) -> tuple[Tensor, tuple[NodeDimension, ...]]:
        """Values of the non-zero entries and, per axis, the nodes they sit at."""
        idx = self.data.nonzero(as_tuple=True)
        return self.data[idx], tuple(self.dimensions[i].offsets_to_nodes(idx[i]) for i in range(self.n_dims))


class NodeIndexedVector(NodeIndexedTensor):
    def add_nodes(self, node_infos: NodeDimension, data: Tensor | None = None):
        self.extend(node_infos, 0, data)

    def topk(self, k: int, ignore_dimension: NodeDimension | None = None):
        data = self.data
        if ignore_dimension is not None and len(ignore_dimension) > 0:
            off = self.dimensions[0].nodes_to_offsets(ignore_dimension)
            data = data.clone()
            data[off[off >= 0]] = float("-inf")
        values, idx = torch.topk(data, k=k, dim=0)
        return values, self.dimensions[0].offsets_to_nodes(idx)

    def matmul(self, other: "NodeIndexedMatrix | NodeIndexedVector", _check_node_matching: bool = False):
        if _check_node_matching:
            assert self.dimensions[0] == other.dimensions[0], "contracted node dimensions differ"
        data = self.data @ other.data
        if isinstance(other, NodeIndexedMatrix):
            return NodeIndexedVector.from_data(data, (other.dimensions[1],))
        if isinstance(other, NodeIndexedVector):
            return data.item()
        raise ValueError(f"Invalid type as right operand in NodeIndexedVector.matmul: {type(other)}. Expected NodeIndexedMatrix or NodeIndexedVector.")

    def __matmul__(self, other):
        return self.matmul(other)


class NodeIndexedMatrix(NodeIndexedTensor):
    """Rows = targets, columns = sources."""

    def add_targets(self, node_infos: NodeDimension, data: Tensor | None = None):
        self.extend(node_infos, 0, data)

    def add_sources(self, node_infos: NodeDimension, data: Tensor | None = None):
        self.extend(node_infos, 1, data)

    def matmul(self, other: "NodeIndexedVector | NodeIndexedMatrix", _check_node_matching: bool = False):
        if _check_node_matching:
            assert self.dimensions[1] == other.dimensions[0], "contracted node dimensions differ"
        data = self.data @ other.data
        if isinstance(other, NodeIndexedMatrix):
            return NodeIndexedMatrix.from_data(data, (self.dimensions[0], other.dimensions[1]))
        if isinstance(other, NodeIndexedVector):
            return NodeIndexedVector.from_data(data, (self.dimensions[0],))
        raise ValueError(f"Invalid type as right operand in NodeIndexedMatrix.matmul: {type(other)}")

    def __matmul__(self, other):
        return self.matmul(other)

    def flat_topk(self, k: int) -> "NodeIndexed[Tensor]":
        """Top ``k`` entries of the whole matrix: values plus the (row node, column node) of each."""
        k = min(k, self.data.numel())
        if k == 0:
            e = torch.empty(0, dtype=torch.long, device=self.data.device)
            return NodeIndexed(self.data.reshape(-1)[:0], (self.dimensions[0].offsets_to_nodes(e), self.dimensions[1].offsets_to_nodes(e)))
        values, flat = torch.topk(self.data.reshape(-1), k)
        n_cols = self.data.shape[1]
        return NodeIndexed(values, (self.dimensions[0].offsets_to_nodes(flat // n_cols), self.dimensions[1].offsets_to_nodes(flat % n_cols)))

    def any(self, dim: int) -> NodeIndexedVector:
        return NodeIndexedVector.from_data(self.data.any(dim), (self.dimensions[1 - dim],))

    @timer.time("masked_fill_dim_")
    def masked_fill_dim_(self, dim: int, mask: NodeIndexedVector, value: Number) -> Self:
        """Fill whole rows (``dim=0``) / columns (``dim=1``) at the nodes where ``mask`` is true."""
        off = self.dimensions[dim].nodes_to_offsets(mask.dimensions[0])[mask.data]
        off = off[off >= 0]
        if off.numel() > 0:
            if dim == 0:
                self.data[off, :] = value
            else:
                self.data[:, off] = value
        return self

    @timer.time("masked_fill_")
    def masked_fill_(self, mask: "NodeIndexedMatrix", value: Number) -> Self:
        self.data.masked_fill_(mask.data, value)
        return self


V = TypeVar("V")


@dataclass
class NodeIndexed(Generic[V], PyTree):
    """Any indexable ``value`` whose entries are labelled by one node per dimension (e.g. edge lists: one source and
    one target node per entry)."""

    value: V
    dimensions: tuple[NodeDimension, ...]

    def __len__(self) -> int:
        return len(self.dimensions[0])

    def __iter__(self):
        nodes = [list(d) for d in self.dimensions]
        for i in range(len(self)):
            yield (self.value[i], *(n[i] for n in nodes))  # type: ignore[index]

    def __getitem__(self, index: "tuple[NodeDimension, int] | NodeDimension") -> Self:
        """Select the entries labelled (along dimension ``which``, default 0) by the nodes of ``indexer``."""
        indexer, which = index if isinstance(index, tuple) else (index, 0)
        off = self.dimensions[which].nodes_to_offsets(indexer)
        dims = tuple(indexer if i == which else d.offsets_to_nodes(off) for i, d in enumerate(self.dimensions))
        return type(self)(self.value[off], dims)  # type: ignore[index]
