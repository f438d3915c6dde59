"""Cached loading of models, dataset shards and dictionaries for the server (server/logic/loaders.py of the reference
project)."""

from functools import lru_cache

from ..models.sparse_dictionary import SparseDictionary, SparseDictionaryConfig
from ..resource_loaders import load_dataset_shard, load_model
from . import config as C
from .common import synchronized


@synchronized
@lru_cache(maxsize=C.LRU_CACHE_SIZE_MODELS)
def get_model(*, name: str, device_mesh=None):
    cfg = C.client.get_model_cfg(name)
    if cfg is None:
        raise ValueError(f"Model {name} not found")
    if C.tokenizer_only:
        cfg.backend = "tokenizer_only"
    cfg.device, cfg.dtype = C.device, C.serving_dtype
    return load_model(cfg, device_mesh=device_mesh)


@synchronized
@lru_cache(maxsize=C.LRU_CACHE_SIZE_DATASETS)
def get_dataset(*, name: str, shard_idx: int = 0, n_shards: int = 1):
    cfg = C.client.get_dataset_cfg(name)
    assert cfg is not None, f"Dataset {name} not found"
    return load_dataset_shard(cfg, shard_idx, n_shards)


@synchronized
@lru_cache(maxsize=C.LRU_CACHE_SIZE_SAES)
def get_sae(*, name: str, device_mesh=None) -> SparseDictionary:
    path = C.client.get_sae_path(name, C.sae_series)
    assert path is not None, f"SAE {name} not found"
    return SparseDictionary.from_pretrained(path, device=C.device, dtype=C.serving_dtype, device_mesh=device_mesh).eval()


@synchronized
@lru_cache(maxsize=C.LRU_CACHE_SIZE_SAES)
def get_sae_cfg(*, name: str) -> SparseDictionaryConfig:
    rec = C.client.get_sae(name, C.sae_series)
    assert rec is not None, f"SAE {name} not found"
    return rec.cfg
