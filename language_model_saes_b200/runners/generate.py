"""``generate_activations``: run a model over a dataset and write activation shards; and
``check_activation_consistency``: read several activation caches in lock-step, which fails on any mismatch
(runners/generate.py:31-224 of the reference project)."""

from __future__ import annotations

import os
from pathlib import Path
from typing import Literal, Optional

import torch
from pydantic_settings import BaseSettings

from ..activation.factory import ActivationFactory, ActivationFactoryConfig, ActivationFactoryDatasetSource, ActivationFactoryTarget
from ..activation.processors.cached_activation import CachedActivationLoader
from ..activation.writer import ActivationWriter, ActivationWriterConfig
from ..backend.language_model import LanguageModelConfig
from ..activation.processors.activation import BufferShuffleConfig
from ..config import DatasetConfig, OptionalTorchDType
from ..database import MongoClient, MongoDBConfig
from ..resource_loaders import load_dataset, load_model
from ..utils.logging import get_distributed_logger, setup_logging
from .utils import load_config, make_mesh

logger = get_distributed_logger("runners.generate")


class GenerateActivationsSettings(BaseSettings):
    model_config = {"arbitrary_types_allowed": True}
    model: Optional[LanguageModelConfig] = None
    model_name: str
    dataset: Optional[DatasetConfig] = None
    dataset_name: str
    hook_points: list[str]
    output_dir: str
    target: ActivationFactoryTarget = ActivationFactoryTarget.ACTIVATIONS_2D
    model_batch_size: int = 1
    batch_size: int
    buffer_size: Optional[int] = None
    buffer_shuffle: Optional[BufferShuffleConfig] = None
    total_tokens: Optional[int] = None
    context_size: int = 128
    n_samples_per_chunk: Optional[int] = None
    num_workers: Optional[int] = None
    format: Literal["pt", "safetensors"] = "safetensors"
    n_shards: Optional[int] = None
    start_shard: int = 0
    mongo: Optional[MongoDBConfig] = None
    ignore_token_ids: Optional[list[int]] = None
    device_type: str = "cuda"
    override_dtype: OptionalTorchDType = None


def generate_activations(settings: GenerateActivationsSettings) -> None:
    """Every process of the job takes its own dataset shards (mesh ``("data", "model") = (WORLD_SIZE, 1)``)."""
    setup_logging(level="INFO")
    world = os.environ.get("WORLD_SIZE")
    mesh = make_mesh(settings.device_type, (int(world), 1), ("data", "model")) if world is not None and int(world) > 1 else None
    mongo = MongoClient(settings.mongo) if settings.mongo is not None else None
    model_cfg = load_config(settings.model, settings.model_name, mongo, "model")
    dataset_cfg = load_config(settings.dataset, settings.dataset_name, mongo, "dataset")
    model = load_model(model_cfg)
    dataset, metadata = load_dataset(dataset_cfg, device_mesh=mesh, n_shards=settings.n_shards, start_shard=settings.start_shard)
    factory = ActivationFactory(ActivationFactoryConfig(
        sources=[ActivationFactoryDatasetSource(name=settings.dataset_name)], target=settings.target, hook_points=settings.hook_points,
        context_size=settings.context_size, model_batch_size=settings.model_batch_size, batch_size=settings.batch_size,
        buffer_size=settings.buffer_size, buffer_shuffle=settings.buffer_shuffle, ignore_token_ids=settings.ignore_token_ids,
        override_dtype=settings.override_dtype,
    ))  # fmt: skip
    writer = ActivationWriter(ActivationWriterConfig(
        hook_points=settings.hook_points, total_generating_tokens=settings.total_tokens, n_samples_per_chunk=settings.n_samples_per_chunk,
        cache_dir=settings.output_dir, format=settings.format, num_workers=settings.num_workers,
    ))  # fmt: skip
    logger.info("Starting activation generation and writing")
    stream = factory.process(model=model, model_name=settings.model_name, datasets={settings.dataset_name: (dataset, metadata)})
    writer.process(stream, device_mesh=mesh, start_shard=settings.start_shard)
    logger.info("Activation generation completed successfully")


class CheckActivationConsistencySettings(BaseSettings):
    paths: dict[str, Path]
    """hook point -> cache directory"""
    device: str = "cuda"
    num_workers: int = 0
    prefetch_factor: int | None = None


def check_activation_consistency(settings: CheckActivationConsistencySettings) -> None:
    """Iterate all caches together; the loader asserts that chunk names, token ids and metadata agree."""
    loader = CachedActivationLoader(cache_dirs=settings.paths, device=settings.device, num_workers=settings.num_workers,
                                    prefetch_factor=settings.prefetch_factor)  # fmt: skip
    n = 0
    for _ in loader.process():
        n += 1
    logger.info(f"{n} chunks are consistent across {len(settings.paths)} caches")
