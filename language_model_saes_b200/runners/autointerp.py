"""``auto_interp``: explain the features of a dictionary with a chat model and store the explanations
(runners/autointerp.py:20-129 of the reference project)."""

from __future__ import annotations

import asyncio
from functools import lru_cache
from typing import Optional

from pydantic_settings import BaseSettings
from tqdm import tqdm

from ..analysis.autointerp import AutoInterpConfig, FeatureInterpreter
from ..backend.language_model import LanguageModelConfig
from ..database import MongoClient, MongoDBConfig
from ..resource_loaders import load_dataset_shard, load_model
from ..utils.logging import get_logger

logger = get_logger("runners.autointerp")


class AutoInterpSettings(BaseSettings):
    sae_name: str
    sae_series: str
    model: LanguageModelConfig
    model_name: str
    auto_interp: AutoInterpConfig
    mongo: MongoDBConfig
    features: Optional[list[int]] = None
    """Feature indices to interpret; all features when omitted."""
    analysis_name: str = "default"
    max_workers: int = 10
    """Concurrent chat requests."""


async def async_auto_interp(settings: AutoInterpSettings, client=None) -> None:
    mongo = MongoClient(settings.mongo)

    @lru_cache(maxsize=None)
    def get_dataset(name: str, shard_idx: int, n_shards: int):
        cfg = mongo.get_dataset_cfg(name)
        assert cfg is not None, f"Dataset {name} not found"
        return load_dataset_shard(cfg, shard_idx, n_shards)

    model = load_model(settings.model)
    interpreter = FeatureInterpreter(settings.auto_interp, mongo, client=client)
    bar: tqdm | None = None

    def progress(done: int, total: int, current: int) -> None:
        nonlocal bar
        if bar is None:
            bar = tqdm(total=total, desc="Interpreting features", unit="feature", dynamic_ncols=True)
        bar.n = done
        bar.set_postfix({"current": current})
        bar.refresh()

    async for result in interpreter.interpret_features(
        sae_name=settings.sae_name, sae_series=settings.sae_series, model=model, datasets=get_dataset,
        analysis_name=settings.analysis_name, feature_indices=settings.features, max_concurrent=settings.max_workers,
        progress_callback=progress,
    ):  # fmt: skip
        interpretation = {"text": result["explanation"]} if result["explanation"] is not None else None
        mongo.update_feature(settings.sae_name, result["feature_index"], {"interpretation": interpretation}, settings.sae_series)
    if bar is not None:
        bar.close()


def auto_interp(settings: AutoInterpSettings) -> None:
    asyncio.run(async_auto_interp(settings))
