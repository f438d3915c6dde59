"""ActivationFactory: turn datasets and/or activation caches into the batch stream that trainers, initialisers,
evaluators and analysers consume.

Configuration classes and the pipeline shape follow activation/factory.py of the reference project (:43-147
configs, :149-408 pipeline): per source a chain (dataset -> [activation generator] -> [2-D to 1-D transformer], or
cache reader -> [transformer]), a weighted random aggregator over the live sources, then re-batching (with
optional shuffle buffer) and dtype override. Three targets: TOKENS < ACTIVATIONS_2D < ACTIVATIONS_1D.

Batch contract of the resulting stream: one entry per hook point (``[B, d]`` for the 1-D target, ``[B, ctx, d]``
for 2-D), plus ``tokens``, ``mask``, ``attention_mask`` and, for 2-D / analysis, ``meta``.
"""

from __future__ import annotations

from enum import Enum
from pathlib import Path
from typing import Any, Callable, Iterable, Iterator, Optional

import numpy as np
from pydantic import BaseModel, ConfigDict

from ..config import BaseConfig, OptionalTorchDType
from .processors.activation import (
    ActivationBatchler,
    ActivationGenerator,
    ActivationTransformer,
    BufferShuffleConfig,
    OverrideDtypeProcessor,
)
from .processors.cached_activation import CachedActivationLoader
from .processors.huggingface import HuggingFaceDatasetLoader


class ActivationFactorySource(BaseModel):
    type: str
    name: str
    sample_weights: float = 1.0


class ActivationFactoryDatasetSource(ActivationFactorySource):
    type: str = "dataset"
    is_dataset_tokenized: bool = False
    prepend_bos: bool = True


class ActivationFactoryActivationsSource(ActivationFactorySource):
    model_config = ConfigDict(arbitrary_types_allowed=True)

    type: str = "activations"
    path: str | dict[str, str]
    device: str = "cpu"
    dtype: OptionalTorchDType = None
    num_workers: int = 4
    prefetch: int | None = 8
    peer_broadcast: bool = False
    """Under model parallelism: one rank of each ``model`` group reads the files and pushes the rows into the other ranks'
    GPU memory over NVLink instead of every rank reading them (CUDA devices only)."""


class ActivationFactoryTarget(Enum):
    TOKENS = "tokens"
    ACTIVATIONS_2D = "activations-2d"
    ACTIVATIONS_1D = "activations-1d"

    @property
    def stage(self) -> int:
        return {"tokens": 0, "activations-2d": 1, "activations-1d": 2}[self.value]

    def __lt__(self, other: "ActivationFactoryTarget") -> bool:
        return self.stage < other.stage

    def __le__(self, other: "ActivationFactoryTarget") -> bool:
        return self.stage <= other.stage

    def __gt__(self, other: "ActivationFactoryTarget") -> bool:
        return self.stage > other.stage

    def __ge__(self, other: "ActivationFactoryTarget") -> bool:
        return self.stage >= other.stage


class ActivationFactoryConfig(BaseConfig):
    model_config = ConfigDict(arbitrary_types_allowed=True)

    sources: list[ActivationFactoryDatasetSource | ActivationFactoryActivationsSource]
    target: ActivationFactoryTarget
    hook_points: list[str]
    batch_size: int | None
    num_workers: int = 4
    context_size: int | None = None
    model_batch_size: int = 1
    override_dtype: OptionalTorchDType = None
    buffer_size: int | None = None
    buffer_shuffle: BufferShuffleConfig | None = None
    ignore_token_ids: list[int] | None = None


class ActivationFactory:
    def __init__(
        self,
        cfg: ActivationFactoryConfig,
        before_aggregation_interceptor: Callable[[dict[str, Any], int], dict[str, Any]] | None = None,
        device_mesh: Optional[Any] = None,
    ):
        self.cfg = cfg
        self.device_mesh = device_mesh
        self.before_aggregation_interceptor = before_aggregation_interceptor
        self.pre_aggregation_processors = self.build_pre_aggregation_processors()
        self.post_aggregation_processor = self.build_post_aggregation_processor()
        self.aggregator = self.build_aggregator()

    def _intercept(self, stream: Iterable[dict[str, Any]], source_idx: int) -> Iterable[dict[str, Any]]:
        fn = self.before_aggregation_interceptor
        return stream if fn is None else (fn(x, source_idx) for x in stream)

    def _dataset_chain(self, source: ActivationFactoryDatasetSource, source_idx: int) -> Callable[..., Iterable[dict[str, Any]]]:
        loader = HuggingFaceDatasetLoader(batch_size=1, with_info=True, show_progress=True, num_workers=self.cfg.num_workers)
        steps = []
        if self.cfg.target >= ActivationFactoryTarget.ACTIVATIONS_2D:
            steps.append(ActivationGenerator(self.cfg.hook_points, batch_size=self.cfg.model_batch_size, n_context=self.cfg.context_size))
        if self.cfg.target >= ActivationFactoryTarget.ACTIVATIONS_1D:
            steps.append(ActivationTransformer())

        def run(**kwargs: Any) -> Iterable[dict[str, Any]]:
            datasets = kwargs.get("datasets")
            assert datasets is not None, "`datasets` must be provided for dataset sources"
            model = kwargs.get("model")
            assert model is not None, "`model` must be provided for dataset sources"
            model_name = kwargs.get("model_name")
            assert model_name is not None, "`model_name` must be provided for dataset sources"
            entry = datasets.get(source.name)
            assert entry is not None, f"Dataset {source.name} not found in `datasets`"
            dataset, metadata = entry
            stream = loader.process(dataset, dataset_name=source.name, metadata=metadata)
            for step in steps:
                stream = step.process(stream, model=model, model_name=model_name, ignore_token_ids=self.cfg.ignore_token_ids)
            return self._intercept(stream, source_idx)

        return run

    def _activations_chain(self, source: ActivationFactoryActivationsSource, source_idx: int) -> Callable[..., Iterable[dict[str, Any]]]:
        if self.cfg.target < ActivationFactoryTarget.ACTIVATIONS_2D:
            raise ValueError("Activations sources are only supported for target >= ACTIVATIONS_2D")
        dirs = source.path if isinstance(source.path, dict) else {hp: Path(source.path) / hp for hp in self.cfg.hook_points}
        loader = CachedActivationLoader(cache_dirs=dirs, device=source.device, dtype=source.dtype, num_workers=source.num_workers,
                                        prefetch_factor=source.prefetch, device_mesh=self.device_mesh,
                                        peer_broadcast=source.peer_broadcast)  # fmt: skip
        steps = [ActivationTransformer()] if self.cfg.target >= ActivationFactoryTarget.ACTIVATIONS_1D else []

        def run(**kwargs: Any) -> Iterable[dict[str, Any]]:
            stream: Iterable[dict[str, Any]] = loader.process()
            for step in steps:
                stream = step.process(stream, ignore_token_ids=self.cfg.ignore_token_ids, model=kwargs.get("model"))
            return self._intercept(stream, source_idx)

        return run

    def build_pre_aggregation_processors(self) -> list[Callable]:
        ds = [s for s in self.cfg.sources if isinstance(s, ActivationFactoryDatasetSource)]
        ac = [s for s in self.cfg.sources if isinstance(s, ActivationFactoryActivationsSource)]
        return [self._dataset_chain(s, i) for i, s in enumerate(ds)] + [self._activations_chain(s, i + len(ds)) for i, s in enumerate(ac)]

    def build_post_aggregation_processor(self) -> Callable:
        steps = []
        if self.cfg.batch_size is not None:
            steps.append(ActivationBatchler(batch_size=self.cfg.batch_size, buffer_size=self.cfg.buffer_size,
                                            buffer_shuffle_config=self.cfg.buffer_shuffle, device_mesh=self.device_mesh))  # fmt: skip
        if self.cfg.override_dtype is not None:
            steps.append(OverrideDtypeProcessor(dtype=self.cfg.override_dtype))

        def run(stream: Iterable[dict[str, Any]], **kwargs: Any) -> Iterable[dict[str, Any]]:
            for step in steps:
                stream = step.process(stream, **kwargs)
            return stream

        return run

    def build_aggregator(self) -> Callable:
        """Weighted random interleaving of the sources that still have data."""
        weights = np.array([s.sample_weights for s in self.cfg.sources], dtype=np.float64)

        def aggregate(streams: list[Iterable[dict[str, Any]]], **kwargs: Any) -> Iterator[dict[str, Any]]:
            its = [iter(s) for s in streams]
            alive = np.ones(len(its), dtype=bool)
            if len(its) == 1:
                yield from its[0]
                return
            while alive.any():
                p = np.where(alive, weights, 0.0)
                i = int(np.random.choice(len(its), p=p / p.sum()))
                try:
                    yield next(its[i])
                except StopIteration:
                    alive[i] = False

        return aggregate

    def process(self, **kwargs: Any) -> Iterable[dict[str, Any]]:
        streams = [chain(**kwargs) for chain in self.pre_aggregation_processors]
        return self.post_aggregation_processor(self.aggregator(streams), **kwargs)
