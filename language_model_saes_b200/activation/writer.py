"""Write activation streams to disk in the reference project's cache format.

Layout and naming follow activation/writer.py of the reference (:19-193): one directory per hook point,
``chunk-%08d`` (single process) or ``shard-<data rank + start_shard>-chunk-%08d`` (under a mesh), one file per
chunk in ``safetensors`` (tensors ``activation, tokens, mask, attention_mask, ...`` plus ``.meta.json``) or
``pt`` (same dict with ``meta`` inside). With ``num_workers`` set, files are written by a thread pool with a
bounded number of writes in flight; device tensors are copied to host (pinned, asynchronously) before being
handed to the pool so that generation is not blocked by the disk.
"""

from __future__ import annotations

import json
from concurrent.futures import FIRST_COMPLETED, ThreadPoolExecutor, as_completed, wait
from pathlib import Path
from typing import Any, Iterable, Literal, Optional, Sequence

import torch
from tqdm import tqdm

from ..config import BaseConfig
from ..parallel.mesh import mesh_dim_size, mesh_local_rank
from ..utils.logging import get_distributed_logger
from ..utils.timer import timer

logger = get_distributed_logger("activation.writer")


class ActivationWriterConfig(BaseConfig):
    hook_points: list[str]
    total_generating_tokens: int | None = None
    n_samples_per_chunk: int | None = None
    cache_dir: str = "activations"
    format: Literal["pt", "safetensors"] = "safetensors"
    num_workers: int | None = None


def _chunks_of(data: Iterable[dict[str, Any]], n: int) -> Iterable[dict[str, Any]]:
    """Stack every ``n`` consecutive single-sample records into one chunk record."""

    def collate(batch: Sequence[dict[str, Any]]) -> dict[str, Any]:
        keys = batch[0].keys()
        assert all(k in d for d in batch for k in keys), f"All samples must have the same keys: {list(keys)}"
        return {k: (torch.stack([d[k] for d in batch]) if isinstance(batch[0][k], torch.Tensor) else [d[k] for d in batch]) for k in keys}

    buf: list[dict[str, Any]] = []
    for rec in data:
        buf.append(rec)
        if len(buf) == n:
            yield collate(buf)
            buf = []
    if buf:
        yield collate(buf)


class ActivationWriter:
    def __init__(self, cfg: ActivationWriterConfig, executor: Optional[ThreadPoolExecutor] = None):
        self.cfg = cfg
        self.cache_dir = Path(cfg.cache_dir)
        self.executor = None if cfg.num_workers is None else (executor or ThreadPoolExecutor(max_workers=cfg.num_workers))
        self._owned_executor = cfg.num_workers is not None and executor is None
        for hp in cfg.hook_points:
            (self.cache_dir / hp).mkdir(parents=True, exist_ok=True)

    def _write_chunk(self, hook_point: str, chunk_data: dict[str, Any], chunk_name: str, meta: Optional[list] = None) -> None:
        path = self.cache_dir / hook_point / f"{chunk_name}.{self.cfg.format}"
        if self.cfg.format == "pt":
            torch.save(chunk_data | ({"meta": meta} if meta is not None else {}), path)
        elif self.cfg.format == "safetensors":
            from safetensors.torch import save_file

            save_file({k: v.contiguous() for k, v in chunk_data.items()}, str(path))
            if meta is not None:
                with open(path.with_suffix(".meta.json"), "w") as f:
                    json.dump(meta, f)
        else:
            raise ValueError(f"Invalid format: {self.cfg.format}")

    @staticmethod
    def _to_host(t: torch.Tensor) -> torch.Tensor:
        if t.device.type != "cuda":
            return t
        host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
        host.copy_(t, non_blocking=True)
        return host

    def process(self, data: Iterable[dict[str, Any]], *, device_mesh=None, start_shard: int = 0) -> None:
        dp = mesh_dim_size(device_mesh, "data")
        total = self.cfg.total_generating_tokens
        if total is not None and device_mesh is not None:
            total //= dp
        pbar = tqdm(desc="Writing activations to disk", total=total)
        written = 0
        futures: set | None = set() if self.executor is not None else None
        if self.cfg.n_samples_per_chunk is not None:
            data = _chunks_of(data, self.cfg.n_samples_per_chunk)
        for chunk_id, chunk in enumerate(data):
            assert all(k in chunk for k in self.cfg.hook_points), f"All samples must have the hook points: {self.cfg.hook_points}"
            name = (
                f"chunk-{chunk_id:08d}"
                if device_mesh is None
                else f"shard-{mesh_local_rank(device_mesh, 'data') + start_shard}-chunk-{chunk_id:08d}"
            )
            meta = chunk.get("meta")
            shared = {k: self._to_host(v) for k, v in chunk.items() if k not in ("meta", *self.cfg.hook_points) and isinstance(v, torch.Tensor)}
            with timer.time("write_chunk"):
                for hp in self.cfg.hook_points:
                    payload = {"activation": self._to_host(chunk[hp])} | shared
                    if futures is None:
                        if torch.cuda.is_available():
                            torch.cuda.current_stream().synchronize()
                        self._write_chunk(hp, payload, name, meta)
                    else:
                        ev = torch.cuda.Event() if torch.cuda.is_available() else None
                        if ev is not None:
                            ev.record()

                        def job(hp=hp, payload=payload, name=name, meta=meta, ev=ev):
                            if ev is not None:
                                ev.synchronize()
                            self._write_chunk(hp, payload, name, meta)

                        futures.add(self.executor.submit(job))
                if futures is not None:
                    while len(futures) >= self.cfg.num_workers * 2:
                        done, futures = wait(futures, return_when=FIRST_COMPLETED)
                        for f in done:
                            f.result()
            if timer.enabled:
                logger.info(f"\nTimer Summary:\n{timer.summary()}\n")
            n = chunk["tokens"].numel()
            written += n
            pbar.update(n)
            if total is not None and written >= total:
                break
        if futures is not None:
            for f in as_completed(futures):
                f.result()
        pbar.close()

    def __del__(self) -> None:
        if getattr(self, "_owned_executor", False) and self.executor is not None:
            self.executor.shutdown(wait=True)
