"""Load datasets and language models from their configs.

Same entry points as resource_loaders.py of the reference project (:17-81): ``load_dataset`` gives every
data-parallel rank a contiguous shard of the dataset, ``load_dataset_shard`` an explicit shard, ``load_model``
picks the backend (``auto`` = the hooked backend for architectures it can convert, HuggingFace otherwise).
"""

from __future__ import annotations

from typing import Any

from .backend.language_model import (
    HookedLanguageModel,
    HuggingFaceLanguageModel,
    LanguageModel,
    LanguageModelConfig,
    QwenVLLanguageModel,
    TokenizerOnlyLanguageModel,
)
from .config import DatasetConfig
from .parallel.mesh import mesh_dim_size, mesh_local_rank


def _load_raw(cfg: DatasetConfig):
    import datasets

    if cfg.is_dataset_on_disk:
        ds = datasets.load_from_disk(cfg.dataset_name_or_path)
    else:
        ds = datasets.load_dataset(cfg.dataset_name_or_path, split="train", cache_dir=cfg.cache_dir)
    return ds


def load_dataset_shard(cfg: DatasetConfig, shard_idx: int, n_shards: int):
    return _load_raw(cfg).shard(num_shards=n_shards, index=shard_idx, contiguous=True)


def load_dataset(cfg: DatasetConfig, device_mesh=None, n_shards: int | None = None, start_shard: int = 0) -> tuple[Any, dict[str, Any] | None]:
    """Returns ``(dataset, metadata)``; under a mesh the dataset is this data rank's contiguous shard and the
    metadata records which one (``shard_idx``, ``n_shards``)."""
    ds = _load_raw(cfg)
    dp = mesh_dim_size(device_mesh, "data")
    if dp == 1 and n_shards is None:
        return ds, None
    n = n_shards if n_shards is not None else dp
    idx = start_shard + mesh_local_rank(device_mesh, "data")
    return ds.shard(num_shards=n, index=idx, contiguous=True), {"shard_idx": idx, "n_shards": n}


def infer_model_backend(model_name: str) -> str:
    name = model_name.lower()
    if "qwen" in name and "vl" in name:
        return "qwen_vl"
    return "hooked"


def load_model(cfg: LanguageModelConfig, device_mesh=None) -> LanguageModel:
    backend = cfg.backend
    if backend == "auto":
        backend = infer_model_backend(cfg.model_name)
    if backend in ("hooked", "transformer_lens"):
        try:
            return HookedLanguageModel(cfg, device_mesh)
        except ValueError:
            if cfg.backend != "auto":
                raise
            return HuggingFaceLanguageModel(cfg, device_mesh)
    if backend == "huggingface":
        return HuggingFaceLanguageModel(cfg, device_mesh)
    if backend == "qwen_vl":
        return QwenVLLanguageModel(cfg, device_mesh)
    if backend == "tokenizer_only":
        return TokenizerOnlyLanguageModel(cfg)
    raise ValueError(f"unknown backend {backend}")
