"""Read activation caches written by ``ActivationWriter`` (or by the reference project).

File contract (activation/processors/cached_activation.py:97-131,182-243 of the reference): one directory per
hook point holding ``shard-{N}-chunk-{N}`` / ``chunk-{N}`` files (``.safetensors`` with an optional
``.meta.json``, or ``.pt``) with keys ``activation, tokens, mask, attention_mask`` (+ ``meta``); chunks are
ordered by (shard, chunk); all hook points must have the same number of chunks and identical tokens per chunk.

Reading is overlapped with consumption: a small pool of threads loads upcoming chunks into pinned host memory
(bounded look-ahead) and, for a CUDA target, the host-to-device copy is issued on a side stream one chunk
ahead. Under data parallelism rank r reads chunks r, r+dp, r+2dp, ... (the reference's striding); ranks of the
same ``model`` / ``sweep`` group read the same chunks themselves (the page cache serves the repeats) instead of
loading different hook points and all-gathering them; with ``peer_broadcast`` only the first rank of a ``model`` group
reads, and one kernel pushes the rows into the other ranks' memory over NVLink.
"""

from __future__ import annotations

import json
import re
from collections import deque
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Iterable, Iterator, Mapping, Optional

import torch

from ...parallel.mesh import mesh_dim_size, mesh_local_rank
from .core import BaseActivationProcessor

_PATTERNS = ("shard-*-chunk-*.pt", "shard-*-chunk-*.safetensors", "chunk-*.pt", "chunk-*.safetensors")


@dataclass
class ChunkInfo:
    path: Path
    shard_id: int
    chunk_id: int

    @classmethod
    def from_path(cls, path: Path) -> "ChunkInfo":
        m = re.match(r"shard-(\d+)-chunk-(\d+)\.(pt|safetensors)$", path.name)
        if m:
            return cls(path=path, shard_id=int(m.group(1)), chunk_id=int(m.group(2)))
        m = re.match(r"chunk-(\d+)\.(pt|safetensors)$", path.name)
        if m:
            return cls(path=path, shard_id=0, chunk_id=int(m.group(1)))
        raise ValueError(
            f"Invalid chunk filename format: {path.name}. "
            "Expected 'shard-{N}-chunk-{N}.(pt|safetensors)' or 'chunk-{N}.(pt|safetensors)'"
        )


class CachedActivationLoader(BaseActivationProcessor[None, Iterable[dict[str, Any]]]):
    def __init__(
        self,
        cache_dirs: Mapping[str, str | Path],
        device: str = "cpu",
        dtype: Optional[torch.dtype] = None,
        num_workers: int = 0,
        prefetch_factor: int | None = None,
        device_mesh=None,
        peer_broadcast: bool = False,
    ):
        self.peer_broadcast = peer_broadcast
        self._bcast = None
        self.cache_dirs = {k: Path(v) for k, v in cache_dirs.items()}
        self.device = device
        self.dtype = dtype
        self.num_workers = num_workers
        self.prefetch_factor = prefetch_factor
        self.device_mesh = device_mesh

    # ---- files -------------------------------------------------------------------------------
    def _get_sorted_chunks(self, hook_point: str) -> list[ChunkInfo]:
        hook_dir = self.cache_dirs[hook_point]
        if not hook_dir.exists():
            raise FileNotFoundError(f"Hook point directory not found: {hook_dir}")
        chunks = [ChunkInfo.from_path(p) for pat in _PATTERNS for p in hook_dir.glob(pat)]
        return sorted(chunks, key=lambda c: (c.shard_id, c.chunk_id))

    def _load_chunk(self, chunk_path: Path) -> dict[str, Any]:
        if chunk_path.suffix == ".safetensors":
            from safetensors.torch import load_file

            data: dict[str, Any] = load_file(str(chunk_path), device="cpu")
            meta_path = chunk_path.with_suffix(".meta.json")
            if meta_path.exists():
                with open(meta_path, "r") as f:
                    data["meta"] = json.load(f)
            return data
        if chunk_path.suffix == ".pt":
            return torch.load(chunk_path, map_location="cpu", weights_only=True)
        raise ValueError(f"Invalid chunk file format: {chunk_path}. Expected .safetensors or .pt")

    def load_single_hook_chunk(self, chunk_idx: int, hook_point: str, hook_chunks: dict[str, list[ChunkInfo]]) -> dict[str, Any]:
        chunk = hook_chunks[hook_point][chunk_idx]
        data = self._load_chunk(chunk.path)
        for key in ("activation", "tokens", "mask", "attention_mask"):
            assert key in data, f"Loading cached activation {chunk.path} error: missing '{key}' field"
        return {"hook_point": hook_point, "chunk_idx": chunk_idx, **{k: data.get(k) for k in ("activation", "mask", "attention_mask", "tokens", "meta")}}

    def _load_all_hooks(self, chunk_idx: int, hook_chunks: dict[str, list[ChunkInfo]]) -> dict[str, Any]:
        out: dict[str, Any] = {}
        for hp in self.cache_dirs:
            d = self.load_single_hook_chunk(chunk_idx, hp, hook_chunks)
            if not out:
                out = {"tokens": d["tokens"], "mask": d["mask"], "attention_mask": d["attention_mask"], "meta": d["meta"]}
            elif not torch.equal(d["tokens"], out["tokens"]):
                raise AssertionError(f"Loading cached activation error: tokens mismatch for chunk {chunk_idx}")
            act = d["activation"]
            if self.dtype is not None:
                act = act.to(self.dtype)
            out[hp] = act
        if out.get("meta") is None:
            out.pop("meta", None)
        if torch.device(self.device).type == "cuda":
            out = {k: (v.pin_memory() if isinstance(v, torch.Tensor) else v) for k, v in out.items()}
        return out

    # ---- streaming ---------------------------------------------------------------------------
    def _my_chunks(self, n_chunks: int) -> list[int]:
        dp = mesh_dim_size(self.device_mesh, "data")
        usable = n_chunks // dp * dp
        return list(range(mesh_local_rank(self.device_mesh, "data"), usable, dp))

    def _to_device(self, rec: dict[str, Any], stream) -> dict[str, Any]:
        dev = torch.device(self.device)
        if dev.type != "cuda":
            return rec
        with torch.cuda.stream(stream):
            moved = {k: (v.to(dev, non_blocking=True) if isinstance(v, torch.Tensor) else v) for k, v in rec.items()}
        moved["_ready"] = stream.record_event()
        return moved

    def process(self, data: None = None, **kwargs) -> Iterator[dict[str, Any]]:
        tp = mesh_dim_size(self.device_mesh, "model")
        if self.peer_broadcast and tp > 1 and torch.device(self.device).type == "cuda":
            yield from self._process_peer_broadcast()
            return
        yield from self._process_local()

    # ---- one reader per model-parallel group, rows pushed to the peers over NVLink -----------------------
    def _process_peer_broadcast(self) -> Iterator[dict[str, Any]]:
        """The first rank of every ``model`` group reads, pins and uploads the chunks; every activation tensor then goes
        to the other ranks of the group through ``BroadcastComm`` (peer stores from one kernel), the small integer
        tensors and the meta through the process group. The other ranks open no file."""
        import torch.distributed as dist

        from ...parallel.dist_ops import broadcast_object
        from ...parallel.symm import BroadcastComm

        group = self.device_mesh.get_group("model")
        dev = torch.device(self.device)
        loader = mesh_local_rank(self.device_mesh, "model") == 0
        src_global = dist.get_global_rank(group, 0)
        stream = self._process_local() if loader else None
        while True:
            rec = next(stream, None) if loader else None
            header = None
            if loader and rec is not None:
                header = {k: ((tuple(v.shape), v.dtype) if isinstance(v, torch.Tensor) else ("obj", v)) for k, v in rec.items()}
            header = broadcast_object(header, group_src=0, group=group)
            if header is None:
                return
            out: dict[str, Any] = {}
            for key, info in header.items():
                if info[0] == "obj":
                    out[key] = info[1]
                    continue
                shape, dtype = info
                wide = dtype in (torch.float32, torch.bfloat16) and len(shape) >= 2 and shape[-1] % 8 == 0
                if wide:
                    d = shape[-1]
                    n_rows = 1
                    for s_ in shape[:-1]:
                        n_rows *= s_
                    if self._bcast is None or self._bcast.max_rows < n_rows or self._bcast.max_row_bytes < d * dtype.itemsize:
                        self._bcast = BroadcastComm(group, dev, n_rows, d * dtype.itemsize)
                    rows = rec[key].reshape(n_rows, d) if loader else None
                    out[key] = self._bcast.broadcast_rows(0, d, dtype, rows).view(*shape)
                else:
                    t = rec[key].contiguous() if loader else torch.empty(shape, dtype=dtype, device=dev)
                    dist.broadcast(t, src=src_global, group=group)
                    out[key] = t
            yield out

    def _process_local(self) -> Iterator[dict[str, Any]]:
        hook_chunks = {hp: self._get_sorted_chunks(hp) for hp in self.cache_dirs}
        counts = {hp: len(c) for hp, c in hook_chunks.items()}
        if len(set(counts.values())) != 1:
            raise ValueError(
                f"Hook points have different numbers of chunks: {counts}. All hook points must have the same number of chunks."
            )
        todo = self._my_chunks(next(iter(counts.values())))
        cuda = torch.device(self.device).type == "cuda"
        copy_stream = torch.cuda.Stream(torch.device(self.device)) if cuda else None
        if self.num_workers <= 0:
            for idx in todo:
                yield self._finish(self._to_device(self._load_all_hooks(idx, hook_chunks), copy_stream))
            return
        ahead = max(self.num_workers * (self.prefetch_factor or 2), 1)
        with ThreadPoolExecutor(max_workers=self.num_workers) as pool:
            pending: deque = deque()
            it = iter(todo)
            for idx in it:
                pending.append(pool.submit(self._load_all_hooks, idx, hook_chunks))
                if len(pending) >= ahead:
                    break
            staged = None
            while pending:
                rec = pending.popleft().result()
                nxt = next(it, None)
                if nxt is not None:
                    pending.append(pool.submit(self._load_all_hooks, nxt, hook_chunks))
                moved = self._to_device(rec, copy_stream)
                if staged is not None:
                    yield self._finish(staged)
                staged = moved
            if staged is not None:
                yield self._finish(staged)

    @staticmethod
    def _finish(rec: dict[str, Any]) -> dict[str, Any]:
        ev = rec.pop("_ready", None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        return rec
