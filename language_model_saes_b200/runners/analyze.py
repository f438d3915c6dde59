"""``analyze_sae``, ``analyze_crosscoder``, ``direct_logit_attribute`` (runners/analyze.py:29-524 of the reference
project). Results go to the database when one is configured, otherwise to a pickle under
``output_dir/<sae_name>/<sae_series>/`` (feature shards of tensor-parallel ranks are merged by the first rank)."""

from __future__ import annotations

import pickle
import shutil
from pathlib import Path
from typing import Any, Optional

import torch
import torch.distributed as dist
from pydantic_settings import BaseSettings

from ..activation.factory import ActivationFactory, ActivationFactoryConfig
from ..analysis.direct_logit_attributor import DirectLogitAttributor, DirectLogitAttributorConfig
from ..analysis.feature_analyzer import FeatureAnalyzer, FeatureAnalyzerConfig
from ..backend.hooked_transformer import HookedTransformer
from ..backend.language_model import LanguageModelConfig
from ..config import DatasetConfig, TorchDType
from ..database import MongoClient, MongoDBConfig
from ..models.crosscoder import Crosscoder
from ..models.sparse_dictionary import SparseDictionary
from ..parallel.dist_ops import broadcast_object
from ..parallel.mesh import mesh_local_rank
from ..resource_loaders import load_dataset, load_model
from ..utils.logging import get_distributed_logger, setup_logging
from .utils import PretrainedSAE, load_config, make_mesh

logger = get_distributed_logger("runners.analyze")


def save_analysis_to_file(output_dir: Path, analysis_name: str, sae_name: str, sae_series: str, analysis: list[dict[str, Any]],
                          start_idx: int, device_mesh=None) -> Path:  # fmt: skip
    """Each record gets its global ``feature_idx``. Single process: one pickle. Tensor parallel: every rank writes
    ``<name>_shards/<first>_<last>.pkl``, rank 0 of the ``"model"`` dimension merges them in feature order."""
    out_dir = Path(output_dir) / sae_name / sae_series
    out_dir.mkdir(parents=True, exist_ok=True)
    analysis = [{**rec, "feature_idx": start_idx + i} for i, rec in enumerate(analysis)]
    if device_mesh is None:
        path = out_dir / f"{analysis_name}_analysis_{len(analysis)}_features.pkl"
        with open(path, "wb") as f:
            pickle.dump(analysis, f)
        return path
    shards = out_dir / f"{analysis_name}_shards"
    shards.mkdir(parents=True, exist_ok=True)
    with open(shards / f"{start_idx}_{start_idx + len(analysis) - 1}.pkl", "wb") as f:
        pickle.dump(analysis, f)
    group = device_mesh.get_group("model")
    dist.barrier(group=group)
    merged_path = None
    if device_mesh.get_local_rank("model") == 0:
        merged: list[dict[str, Any]] = []
        for p in shards.glob("*.pkl"):
            with open(p, "rb") as f:
                merged.extend(pickle.load(f))
        merged.sort(key=lambda r: r["feature_idx"])
        merged_path = out_dir / f"{analysis_name}_analysis_{len(merged)}_features.pkl"
        with open(merged_path, "wb") as f:
            pickle.dump(merged, f)
        shutil.rmtree(shards)
    return broadcast_object(merged_path, group_src=0, group=group)


class AnalyzeSAESettings(BaseSettings):
    model_config = {"arbitrary_types_allowed": True}
    sae: PretrainedSAE
    sae_name: str
    sae_series: str
    activation_factory: ActivationFactoryConfig
    model: Optional[LanguageModelConfig] = None
    model_name: Optional[str] = None
    datasets: Optional[dict[str, Optional[DatasetConfig]]] = None
    analyzer: FeatureAnalyzerConfig
    amp_dtype: TorchDType = torch.bfloat16
    feature_analysis_name: str = "default"
    mongo: MongoDBConfig | None = None
    output_dir: Optional[Path] = None
    """Used only when no database is configured."""
    model_parallel_size: int = 1
    device_type: str = "cuda"


def _store(result, settings, mongo, mesh) -> None:
    start_idx = mesh_local_rank(mesh, "model") * len(result)
    if mongo is not None:
        mongo.add_feature_analysis(name=settings.feature_analysis_name, sae_name=settings.sae_name, sae_series=settings.sae_series,
                                   analysis=result, start_idx=start_idx)  # fmt: skip
        logger.info("Results saved to the database")
    else:
        assert settings.output_dir is not None, "Output directory must be set when no database is used"
        path = save_analysis_to_file(settings.output_dir, settings.feature_analysis_name, settings.sae_name, settings.sae_series,
                                     result, start_idx, mesh)  # fmt: skip
        logger.info(f"Results saved to: {path}")


@torch.no_grad()
def analyze_sae(settings: AnalyzeSAESettings) -> None:
    setup_logging(level="INFO")
    mesh = make_mesh(settings.device_type, (settings.model_parallel_size,), ("model",))
    mongo = MongoClient(settings.mongo) if settings.mongo is not None else None
    assert mongo is not None or settings.output_dir is not None, "Output directory must be provided if no database is configured"
    model_cfg = load_config(settings.model, settings.model_name, mongo, "model", required=False)
    dataset_cfgs = {n: load_config(c, n, mongo, "dataset") for n, c in settings.datasets.items()} if settings.datasets is not None else None
    model = load_model(model_cfg) if model_cfg is not None else None
    datasets = {n: load_dataset(c, device_mesh=mesh) for n, c in dataset_cfgs.items()} if dataset_cfgs is not None else None
    factory = ActivationFactory(settings.activation_factory, device_mesh=mesh)
    sae = SparseDictionary.from_pretrained(
        settings.sae.pretrained_name_or_path, device_mesh=mesh, device=settings.sae.device, dtype=settings.sae.dtype,
        fold_activation_scale=settings.sae.fold_activation_scale, strict_loading=settings.sae.strict_loading,
    )  # fmt: skip
    logger.info(f"SAE model loaded: {type(sae).__name__}")
    with torch.amp.autocast(device_type=settings.device_type, dtype=settings.amp_dtype):
        result = FeatureAnalyzer(settings.analyzer).analyze_chunk(
            factory, sae=sae, device_mesh=mesh,
            activation_factory_process_kwargs={"model": model, "model_name": settings.model_name, "datasets": datasets},
        )  # fmt: skip
    _store(result, settings, mongo, mesh)
    logger.info("SAE analysis completed successfully")


class AnalyzeCrosscoderSettings(BaseSettings):
    model_config = {"arbitrary_types_allowed": True}
    sae: PretrainedSAE
    sae_name: str
    sae_series: str
    activation_factories: list[ActivationFactoryConfig]
    analyzer: FeatureAnalyzerConfig
    amp_dtype: TorchDType = torch.bfloat16
    feature_analysis_name: str = "default"
    mongo: MongoDBConfig | None = None
    output_dir: Optional[Path] = None
    device_type: str = "cuda"


@torch.no_grad()
def analyze_crosscoder(settings: AnalyzeCrosscoderSettings) -> None:
    """One activation factory per head-parallel rank; mesh ``("head", "model") = (n_factories, 1)``. Feature
    activations are identical on every head rank, so rank 0 of the head dimension stores the result."""
    setup_logging(level="INFO")
    n_heads_ranks = len(settings.activation_factories)
    mesh = make_mesh(settings.device_type, (n_heads_ranks, 1), ("head", "model"))
    mongo = MongoClient(settings.mongo) if settings.mongo is not None else None
    assert mongo is not None or settings.output_dir is not None, "Output directory must be provided if no database is configured"
    head_rank = mesh_local_rank(mesh, "head")
    factory = ActivationFactory(settings.activation_factories[head_rank])
    sae = SparseDictionary.from_pretrained(
        settings.sae.pretrained_name_or_path, device_mesh=mesh, device=settings.sae.device, dtype=settings.sae.dtype,
        fold_activation_scale=settings.sae.fold_activation_scale, strict_loading=settings.sae.strict_loading,
    )  # fmt: skip
    assert isinstance(sae, Crosscoder), "analyze_crosscoder needs a crosscoder checkpoint"
    with torch.amp.autocast(device_type=settings.device_type, dtype=settings.amp_dtype):
        result = FeatureAnalyzer(settings.analyzer).analyze_chunk(factory, sae=sae, device_mesh=mesh)
    if head_rank == 0:
        _store(result, settings, mongo, None)
    if mesh is not None:
        dist.barrier()
    logger.info("Crosscoder analysis completed successfully")


class DirectLogitAttributeSettings(BaseSettings):
    sae: PretrainedSAE
    sae_name: str
    layer_idx: Optional[int] = None
    sae_series: str
    model: Optional[LanguageModelConfig] = None
    model_name: str
    direct_logit_attributor: DirectLogitAttributorConfig
    mongo: MongoDBConfig | None = None
    analysis_file: Path | None = None
    """Pickle written by ``analyze_sae`` that gets a ``logits`` entry per feature when no database is configured."""
    device_type: str = "cuda"


@torch.no_grad()
def direct_logit_attribute(settings: DirectLogitAttributeSettings) -> None:
    setup_logging(level="INFO")
    mongo = MongoClient(settings.mongo) if settings.mongo is not None else None
    assert mongo is not None or settings.analysis_file is not None, "Analysis file must be provided if no database is configured"
    sae = SparseDictionary.from_pretrained(
        settings.sae.pretrained_name_or_path, device=settings.sae.device, dtype=settings.sae.dtype,
        fold_activation_scale=settings.sae.fold_activation_scale, strict_loading=settings.sae.strict_loading,
    )  # fmt: skip
    model_cfg = load_config(settings.model, settings.model_name, mongo, "model", required=True)
    model_cfg.device = settings.device_type
    model_cfg.dtype = sae.cfg.dtype
    model = load_model(model_cfg)
    assert isinstance(model, HookedTransformer), "DirectLogitAttributor only supports the hooked-transformer backend"
    results = DirectLogitAttributor(settings.direct_logit_attributor).direct_logit_attribute(sae, model, settings.layer_idx)
    if mongo is not None:
        mongo.update_features(sae_name=settings.sae_name, sae_series=settings.sae_series,
                              update_data=[{"logits": r} for r in results], start_idx=0)  # fmt: skip
    else:
        with open(settings.analysis_file, "rb") as f:
            data = pickle.load(f)
        assert len(data) == len(results), (
            f"Number of features in analysis file ({len(data)}) does not match number of results from direct logit attribution ({len(results)})"
        )
        for i, r in enumerate(results):
            assert data[i]["feature_idx"] == i, "Feature index mismatch"
            data[i]["logits"] = r
        with open(settings.analysis_file, "wb") as f:
            pickle.dump(data, f)
        logger.info(f"Updated {len(results)} features with logit attributions")
    logger.info("Direct logit attribution completed successfully")
