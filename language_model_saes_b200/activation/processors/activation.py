"""Activation generation, 2-D -> 1-D flattening, re-batching with online shuffling, dtype override.

Behaviour follows activation/processors/activation.py of the reference project: BufferShuffleConfig (:18-22),
ActivationBuffer (:25-163), ActivationGenerator (:166-225), ActivationTransformer (:228-287),
ActivationBatchler (:297-394), OverrideDtypeProcessor (:397-406). Tensors here are plain per-rank tensors; under
data parallelism every rank batches its own stream and ``batch_size`` is the GLOBAL batch (each rank yields
``batch_size // dp`` rows). The buffer keeps a list of pieces and only concatenates when it shuffles or runs
out of whole pieces, instead of re-concatenating the whole buffer for every batch.
"""

from __future__ import annotations

from typing import Any, Iterable, Optional

import torch

from ...config import BaseConfig
from ...parallel.mesh import mesh_dim_size
from .core import BaseActivationProcessor


class BufferShuffleConfig(BaseConfig):
    perm_seed: int = 42
    generator_device: str | None = None
    cross_rank: bool = False
    """Under data parallelism, also permute rows ACROSS the data-parallel ranks each time the buffer is shuffled (CUDA
    tensors only; an all-to-all over NVLink peer memory, ``parallel.symm.ShuffleComm``). Off: every rank shuffles
    only what it generated itself, as the reference does."""


def _rows(d: dict[str, Any]) -> int:
    return len(next(iter(d.values())))


def _cat(parts: list[Any]):
    if isinstance(parts[0], torch.Tensor):
        return parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)
    return [x for p in parts for x in p]


class ActivationBuffer:
    """Out-of-place FIFO of activation records (dict of equally long tensors / lists)."""

    def __init__(self, buffer: list[dict[str, Any]] | None = None, device_mesh=None, generator: torch.Generator | None = None):
        self.buffer: list[dict[str, Any]] = list(buffer or [])
        self.device_mesh = device_mesh
        self.generator = generator if generator is not None else torch.Generator()

    def __len__(self) -> int:
        return sum(_rows(d) for d in self.buffer)

    def cat(self, activations: dict[str, Any]) -> "ActivationBuffer":
        return ActivationBuffer(self.buffer + [activations], self.device_mesh, self.generator)

    def consume(self) -> dict[str, Any]:
        keys = self.buffer[0].keys()
        return {k: _cat([d[k] for d in self.buffer]) for k in keys}

    def yield_batch(self, batch_size: int) -> tuple[dict[str, Any], "ActivationBuffer"]:
        """Split off the first ``batch_size // dp`` rows (fewer if the buffer is shorter)."""
        if len(self) == 0:
            raise ValueError("Buffer is empty")
        n = batch_size // mesh_dim_size(self.device_mesh, "data")
        taken: list[dict[str, Any]] = []
        rest = list(self.buffer)
        need = n
        while rest and need > 0:
            head = rest[0]
            r = _rows(head)
            if r <= need:
                taken.append(rest.pop(0))
                need -= r
            else:
                taken.append({k: v[:need] for k, v in head.items()})
                rest[0] = {k: v[need:] for k, v in head.items()}
                need = 0
        batch = {k: _cat([d[k] for d in taken]) for k in taken[0].keys()}
        return batch, ActivationBuffer(rest, self.device_mesh, self.generator)

    def shuffle(self, cross_rank: "CrossRankShuffler | None" = None) -> "ActivationBuffer":
        """Seeded random permutation of the rows held by this rank; with ``cross_rank`` the rows are then permuted
        across the data-parallel ranks too."""
        data = self.consume()
        assert all(isinstance(v, torch.Tensor) for v in data.values()), "All data must be tensors to perform shuffling"
        n = _rows(data)
        perm = torch.randperm(n, generator=self.generator, device=self.generator.device)
        data = {k: v[perm.to(v.device)] for k, v in data.items()}
        if cross_rank is not None:
            data = cross_rank(data)
        return ActivationBuffer([data], self.device_mesh, self.generator)


class CrossRankShuffler:
    """Mixes the shuffle buffers of the data-parallel ranks: the first ``m`` rows of every rank (``m`` = the smallest
    buffer length among the ranks) go through one seeded global permutation; rows beyond ``m`` stay where they are.
    All tensors of a record move with the same permutation. Rows whose byte size is not a multiple of 16 (token ids,
    masks) are padded for the transfer."""

    def __init__(self, device_mesh, seed: int, capacity_rows: int):
        self.group = device_mesh.get_group("data")
        self.seed = seed
        self.capacity = capacity_rows
        self.comm = None
        self.calls = 0

    def __call__(self, data: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        import torch.distributed as dist

        from ...parallel.symm import ShuffleComm

        first = next(iter(data.values()))
        assert first.is_cuda, "the cross-rank shuffle moves rows between GPUs: keep the buffer on the device"
        n = torch.tensor([_rows(data)], device=first.device)
        dist.all_reduce(n, op=dist.ReduceOp.MIN, group=self.group)
        m = int(n)
        if m == 0:
            return data
        row_bytes = {k: -(-(v[0].numel() * v.element_size()) // 16) * 16 for k, v in data.items()}
        if self.comm is None or m > self.comm.rows_per_rank or max(row_bytes.values()) > self.comm.max_row_bytes:
            self.comm = ShuffleComm(self.group, first.device, max(m, self.capacity), max(row_bytes.values()))
        self.calls += 1
        perm = self.comm.permutation(m, self.seed + self.calls)
        out = {}
        for k, v in data.items():
            head = v[:m].contiguous()
            raw = head.view(torch.uint8).reshape(m, -1)
            pad = row_bytes[k] - raw.shape[1]
            if pad:
                raw = torch.nn.functional.pad(raw, (0, pad))
            mixed = self.comm.shuffle(raw, 0, perm=perm)
            if pad:
                mixed = mixed[:, : raw.shape[1] - pad].contiguous()
            mixed = mixed.view(v.dtype).reshape(m, *v.shape[1:])
            out[k] = mixed if v.shape[0] == m else torch.cat([mixed, v[m:]], dim=0)
        return out


class ActivationGenerator(BaseActivationProcessor[Iterable[dict[str, Any]], Iterable[dict[str, Any]]]):
    """Raw records -> language-model activations at the requested hook points (+ tokens, masks, meta)."""

    def __init__(self, hook_points: list[str], batch_size: int, n_context: Optional[int] = None):
        self.hook_points = hook_points
        self.batch_size = batch_size
        self.n_context = n_context

    def batched(self, data: Iterable[dict[str, Any]]) -> Iterable[dict[str, Any]]:
        chunk: list[dict[str, Any]] = []
        for rec in data:
            chunk.append(rec)
            if len(chunk) == self.batch_size:
                yield {k: [r[k] for r in chunk] for k in chunk[0].keys()}
                chunk = []
        if chunk:
            yield {k: [r[k] for r in chunk] for k in chunk[0].keys()}

    @torch.no_grad()
    def process(self, data: Iterable[dict[str, Any]], *, model, model_name: str, **kwargs) -> Iterable[dict[str, Any]]:
        for d in self.batched(data):
            d = model.preprocess_raw_data(d)
            acts = model.to_activations(d, self.hook_points, n_context=self.n_context)
            n = len(next(iter(d.values())))
            existing = d.get("meta", [{} for _ in range(n)])
            yield {**acts, "meta": [{"model_name": model_name} | existing[i] for i in range(len(existing))]}


def _drop_masked(v: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """``v[mask]`` over the leading (batch, context) dimensions; activations on a GPU go through the one-pass scan +
    row-gather kernels instead of a boolean index (which materialises an index tensor and syncs twice)."""
    if v.is_cuda and v.ndim == mask.ndim + 1 and v.is_floating_point() and v.dtype in (torch.float32, torch.bfloat16):
        from ...ops.select_kernels import compact_rows

        return compact_rows(v.reshape(-1, v.shape[-1]), mask.reshape(-1))
    return v[mask]


class ActivationTransformer(BaseActivationProcessor[Iterable[dict[str, Any]], Iterable[dict[str, Any]]]):
    """``[batch, context, d]`` -> ``[kept tokens, d]``: drops masked tokens (or the given token ids) and the meta."""

    def process(self, data: Iterable[dict[str, Any]], *, ignore_token_ids: Optional[list[int]] = None, **kwargs):
        for d in data:
            tokens = d["tokens"]
            assert isinstance(tokens, torch.Tensor)
            if ignore_token_ids is not None:
                mask = torch.isin(tokens, torch.tensor(ignore_token_ids, device=tokens.device), invert=True)
            else:
                mask = d["mask"].bool()
            yield {k: _drop_masked(v, mask) for k, v in d.items() if isinstance(v, torch.Tensor)}


class ActivationBatchler(BaseActivationProcessor[Iterable[dict[str, Any]], Iterable[dict[str, Any]]]):
    """Re-batch a stream of variable-length records to ``batch_size`` rows, optionally through a shuffle buffer:
    when the buffer holds ``buffer_size`` rows it is shuffled and drained down to half."""

    def __init__(self, batch_size: int, buffer_size: Optional[int] = None,
                 buffer_shuffle_config: Optional[BufferShuffleConfig] = None, device_mesh=None):  # fmt: skip
        self.batch_size = batch_size
        self.buffer_size = buffer_size
        self.device_mesh = device_mesh
        self.perm_generator = torch.Generator()
        self.cross_rank: CrossRankShuffler | None = None
        if buffer_shuffle_config is not None:
            self.perm_generator = torch.Generator(buffer_shuffle_config.generator_device or "cpu")
            self.perm_generator.manual_seed(buffer_shuffle_config.perm_seed)
            dp = mesh_dim_size(device_mesh, "data")
            if buffer_shuffle_config.cross_rank and dp > 1 and buffer_size is not None:
                self.cross_rank = CrossRankShuffler(device_mesh, buffer_shuffle_config.perm_seed, max(buffer_size // dp, 1) * 2)

    def process(self, data: Iterable[dict[str, Any]], **kwargs) -> Iterable[dict[str, torch.Tensor]]:
        buffer = ActivationBuffer(device_mesh=self.device_mesh, generator=self.perm_generator)
        dp = mesh_dim_size(self.device_mesh, "data")
        local_batch = self.batch_size // dp
        local_cap = None if self.buffer_size is None else max(self.buffer_size // dp, local_batch)
        for d in data:
            sizes = {k: len(v) for k, v in d.items()}
            assert len(set(sizes.values())) == 1, f"All tensors and lists must have the same batch size, {sizes}"
            buffer = buffer.cat(d)
            if local_cap is not None:
                if len(buffer) >= local_cap:
                    buffer = buffer.shuffle(self.cross_rank)
                    while len(buffer) >= local_cap // 2 and len(buffer) >= local_batch:
                        batch, buffer = buffer.yield_batch(self.batch_size)
                        yield batch
            else:
                while len(buffer) >= local_batch:
                    batch, buffer = buffer.yield_batch(self.batch_size)
                    yield batch
        while len(buffer) > 0:
            batch, buffer = buffer.yield_batch(self.batch_size)
            yield batch


class OverrideDtypeProcessor(BaseActivationProcessor[Iterable[dict[str, Any]], Iterable[dict[str, Any]]]):
    """Cast every floating-point tensor of each record (token ids and masks keep their types)."""

    def __init__(self, dtype: torch.dtype):
        self.dtype = dtype

    def process(self, data: Iterable[dict[str, Any]], **kwargs: Any) -> Iterable[dict[str, Any]]:
        for rec in data:
            yield {k: (v.to(self.dtype) if isinstance(v, torch.Tensor) and v.is_floating_point() else v) for k, v in rec.items()}
