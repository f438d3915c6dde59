"""Named device meshes, dimension maps and rank helpers.

Design: one process per GPU; every parameter is a plain *local shard* tensor and every collective is
explicit. ``torch.distributed.device_mesh.DeviceMesh`` (NCCL on GPUs, gloo on CPU) supplies rendezvous
and the per-dimension process groups; it is the ``device_mesh`` object the public API accepts, as in the
reference project. ``DimMap`` keeps the reference's interface (utils/distributed/dimmap.py:11-186 there):
a mapping mesh-dimension-name -> tensor dimension from which placements, local slices and DTensor
conversions derive; here ``local_slices`` / ``shard`` / ``gather`` are the primary operations and the DTensor
conversions exist for checkpoint compatibility.

Mesh dimension names used by the framework: ``data`` (batch), ``model`` (dictionary/feature axis),
``head`` (crosscoder heads), ``sweep`` (independent runs sharing a stream).
"""

from __future__ import annotations

import functools
import operator
from typing import Any, Callable, Sequence

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import DeviceMesh, init_device_mesh

__all__ = [
    "DimMap",
    "DeviceMesh",
    "build_mesh",
    "mesh_dim_size",
    "mesh_local_rank",
    "mesh_group",
    "mesh_rank",
    "is_primary_rank",
    "get_process_group",
]


def build_mesh(device_type: str, shape: Sequence[int], names: Sequence[str]) -> DeviceMesh:
    """``init_device_mesh`` with named dimensions; initialises the default process group when needed."""
    return init_device_mesh(device_type, tuple(shape), mesh_dim_names=tuple(names))


def _has_dim(mesh: DeviceMesh | None, name: str) -> bool:
    return mesh is not None and mesh.mesh_dim_names is not None and name in mesh.mesh_dim_names


def mesh_dim_size(mesh: DeviceMesh | None, name: str) -> int:
    """Size of a named mesh dimension; 1 when there is no mesh or no such dimension."""
    if not _has_dim(mesh, name):
        return 1
    return mesh.size(mesh.mesh_dim_names.index(name))  # type: ignore[union-attr]


def mesh_local_rank(mesh: DeviceMesh | None, name: str) -> int:
    """This process's coordinate along a named mesh dimension; 0 when absent."""
    if not _has_dim(mesh, name):
        return 0
    return mesh.get_local_rank(name)  # type: ignore[union-attr]


mesh_dim_rank = mesh_local_rank


def mesh_group(mesh: DeviceMesh | None, name: str) -> dist.ProcessGroup | None:
    if not _has_dim(mesh, name):
        return None
    return mesh.get_group(name)  # type: ignore[union-attr]


def mesh_rank(mesh: DeviceMesh | None) -> int:
    """Linear rank inside the mesh (row-major over its dimensions); 0 without a mesh."""
    if mesh is None:
        return 0
    coord = mesh.get_coordinate()
    if coord is None:
        return -1
    sizes = [mesh.size(i) for i in range(mesh.ndim)]
    r = 0
    for c, s in zip(coord, sizes):
        r = r * s + c
    return r


def is_primary_rank(mesh: DeviceMesh | None, dim_name: str = "sweep") -> bool:
    """True on the process whose coordinates are all zero, ignoring the ``dim_name`` coordinate
    (sweep members each have their own primary; reference: utils/distributed/utils.py:11-20)."""
    if mesh is None:
        return True
    coord = mesh.get_coordinate()
    names = mesh.mesh_dim_names
    if coord is None or names is None:
        return False
    return all(c == 0 for n, c in zip(names, coord) if n != dim_name)


_group_cache: dict[tuple, dist.ProcessGroup | None] = {}


def get_process_group(mesh: DeviceMesh, dim_names: Sequence[str] | None = None) -> dist.ProcessGroup | None:
    """Process group spanning several mesh dimensions (all of them by default). Groups over more than one
    dimension are created once per distinct rank set and cached; every rank of the mesh must call this
    collectively the first time."""
    names = tuple(mesh.mesh_dim_names or ())
    dims = names if dim_names is None else tuple(dim_names)
    if len(dims) == 1:
        return mesh.get_group(dims[0])
    key = (id(mesh), dims)
    if key in _group_cache:
        return _group_cache[key]
    ranks = mesh.mesh  # tensor of global ranks shaped like the mesh
    keep = [names.index(d) for d in dims]
    other = [i for i in range(len(names)) if i not in keep]
    perm = other + keep
    flat = ranks.permute(perm).reshape(-1, functools.reduce(operator.mul, [ranks.size(i) for i in keep], 1))
    mine = None
    me = dist.get_rank()
    for row in flat.tolist():
        g = dist.new_group(ranks=row)
        if me in row:
            mine = g
    _group_cache[key] = mine
    return mine


class DimMap:
    """mesh dimension name -> tensor dimension that is sharded along it."""

    def __init__(self, dim_map: dict[str, int] | None = None):
        self._m: dict[str, int] = dict(dim_map or {})

    # mapping protocol
    def __getitem__(self, key: str) -> int:
        return self._m[key]

    def __contains__(self, key: object) -> bool:
        return key in self._m

    def __iter__(self):
        return iter(self._m)

    def items(self):
        return self._m.items()

    def keys(self):
        return self._m.keys()

    def values(self):
        return self._m.values()

    def to_dict(self) -> dict[str, int]:
        return dict(self._m)

    @classmethod
    def from_dict(cls, d: dict[str, int]) -> "DimMap":
        return cls(d)

    def __or__(self, other: "DimMap") -> "DimMap":
        return DimMap({**self._m, **other.to_dict()})

    def __eq__(self, other: object) -> bool:
        return isinstance(other, DimMap) and self._m == other._m

    def __ne__(self, other: object) -> bool:
        return not self.__eq__(other)

    def __hash__(self):
        return hash(tuple(sorted(self._m.items())))

    def __repr__(self) -> str:
        return f"DimMap({self._m})"

    def reverse(self) -> dict[int, str]:
        if len(set(self._m.values())) != len(self._m):
            raise ValueError("Dimension map values must be unique to reverse.")
        return {v: k for k, v in self._m.items()}

    # ---- local-shard operations (primary) ---------------------------------------------------------
    def local_slices(self, shape: Sequence[int], mesh: DeviceMesh | None) -> tuple[slice, ...]:
        """Slices of the full tensor that this rank owns (even sharding required)."""
        rev = self.reverse()
        out = []
        for i, n in enumerate(shape):
            name = rev.get(i if i in rev else i - len(shape))
            if name is None or not _has_dim(mesh, name):
                out.append(slice(None))
                continue
            parts = mesh_dim_size(mesh, name)
            assert n % parts == 0, f"dimension {i} of size {n} is not divisible by mesh dim {name}={parts}"
            step = n // parts
            r = mesh_local_rank(mesh, name)
            out.append(slice(r * step, (r + 1) * step))
        return tuple(out)

    def local_shape(self, shape: Sequence[int], mesh: DeviceMesh | None) -> tuple[int, ...]:
        return tuple(len(range(*s.indices(n))) for s, n in zip(self.local_slices(shape, mesh), shape))

    def shard(self, full: torch.Tensor, mesh: DeviceMesh | None) -> torch.Tensor:
        """Local shard of a full tensor that every rank holds."""
        return full[self.local_slices(tuple(full.shape), mesh)]

    def gather(self, local: torch.Tensor, mesh: DeviceMesh | None) -> torch.Tensor:
        """All-gather the shards into the full tensor (identical on every rank)."""
        out = local
        for name, d in self._m.items():
            if mesh_dim_size(mesh, name) == 1:
                continue
            g = mesh_group(mesh, name)
            d = d % out.ndim
            parts = [torch.empty_like(out) for _ in range(dist.get_world_size(g))]
            dist.all_gather(parts, out.contiguous(), group=g)
            out = torch.cat(parts, dim=d)
        return out

    # ---- DTensor compatibility --------------------------------------------------------------------
    def placements(self, mesh: DeviceMesh):
        from torch.distributed.tensor.placement_types import Replicate, Shard

        if mesh.mesh_dim_names is None:
            raise ValueError("Device mesh does not have mesh dimension names.")
        return [Shard(self._m[n]) if n in self._m else Replicate() for n in mesh.mesh_dim_names]

    def distribute(self, tensor: torch.Tensor, mesh: DeviceMesh):
        from torch.distributed.tensor import distribute_tensor

        return distribute_tensor(tensor, mesh, self.placements(mesh))

    def from_local(self, tensor: torch.Tensor, mesh: DeviceMesh):
        from torch.distributed.tensor import DTensor

        return DTensor.from_local(tensor, mesh, placements=self.placements(mesh))

    def redistribute(self, tensor):
        return tensor.redistribute(placements=self.placements(tensor.device_mesh))

    @classmethod
    def from_placements(cls, placements, mesh: DeviceMesh) -> "DimMap":
        from torch.distributed.tensor.placement_types import Replicate, Shard

        assert mesh.mesh_dim_names is not None, "Device mesh must have mesh dimension names"
        assert all(isinstance(p, (Shard, Replicate)) for p in placements), "All placements must be Shard or Replicate"
        return cls({n: p.dim for n, p in zip(mesh.mesh_dim_names, placements) if isinstance(p, Shard)})


def execute_and_broadcast(fn: Callable[[], Any], mesh: DeviceMesh | None, src_is_primary: bool = True) -> Any:
    """Run ``fn`` on the primary rank and give every rank of the mesh its result."""
    if mesh is None or not dist.is_initialized():
        return fn()
    group = get_process_group(mesh)
    value = [fn() if is_primary_rank(mesh, dim_name="") else None]
    src = dist.get_global_rank(group, 0) if group is not None else 0
    dist.broadcast_object_list(value, src=src, group=group)
    return value[0]
