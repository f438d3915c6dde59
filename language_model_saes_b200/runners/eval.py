"""``evaluate_sae`` and ``evaluate_crosscoder`` (runners/eval.py:25-203 of the reference project)."""

from __future__ import annotations

from typing import Optional

from pydantic_settings import BaseSettings

from ..activation.factory import ActivationFactory, ActivationFactoryConfig
from ..backend.language_model import LanguageModelConfig
from ..config import DatasetConfig
from ..database import MongoClient, MongoDBConfig
from ..evaluator import EvalConfig, Evaluator
from ..models.sparse_dictionary import SparseDictionary
from ..parallel.mesh import mesh_local_rank
from ..resource_loaders import load_dataset, load_model
from ..trainer import WandbConfig
from ..utils.logging import get_distributed_logger, setup_logging
from .utils import PretrainedSAE, init_wandb, load_config, make_mesh

logger = get_distributed_logger("runners.eval")


class EvaluateSAESettings(BaseSettings):
    sae: PretrainedSAE
    sae_name: str
    sae_series: str
    activation_factory: ActivationFactoryConfig
    model: Optional[LanguageModelConfig] = None
    """With a model the downstream language-model loss is measured too."""
    model_name: Optional[str] = None
    datasets: Optional[dict[str, Optional[DatasetConfig]]] = None
    """Datasets of the activation factory's dataset sources (a value of None is looked up in the database by its name), so
    that a dictionary can be evaluated on activations computed on the fly; the reference's settings have the model only and
    so evaluate from cached activations."""
    mongo: Optional[MongoDBConfig] = None
    eval: EvalConfig
    model_parallel_size: int = 1
    fold_activation_scale: bool = False
    wandb: Optional[WandbConfig] = None
    device_type: str = "cuda"


def evaluate_sae(settings: EvaluateSAESettings) -> dict[str, float]:
    setup_logging(level="INFO")
    mesh = make_mesh(settings.device_type, (settings.model_parallel_size,), ("model",))
    factory = ActivationFactory(settings.activation_factory, device_mesh=mesh)
    sae = SparseDictionary.from_pretrained(
        settings.sae.pretrained_name_or_path, device_mesh=mesh, fold_activation_scale=settings.fold_activation_scale,
        device=settings.sae.device, dtype=settings.sae.dtype, strict_loading=settings.sae.strict_loading,
    )  # fmt: skip
    logger.info(f"SAE model loaded: {type(sae).__name__}")
    mongo = MongoClient(settings.mongo) if settings.mongo is not None else None
    model_cfg = load_config(settings.model, settings.model_name, mongo, "model", required=False)
    model = load_model(model_cfg) if model_cfg is not None else None
    datasets = None
    if settings.datasets is not None:
        datasets = {n: load_dataset(load_config(c, n, mongo, "dataset"), device_mesh=mesh) for n, c in settings.datasets.items()}
    wandb_logger = init_wandb(settings.wandb, settings, mesh)
    stream = factory.process(model=model, model_name=settings.model_name, datasets=datasets)
    results = Evaluator(settings.eval).evaluate(sae, stream, wandb_logger, model=model)
    logger.info("Evaluation completed")
    return results


class EvaluateCrosscoderSettings(BaseSettings):
    sae: PretrainedSAE
    sae_name: str
    sae_series: str
    activation_factories: list[ActivationFactoryConfig]
    eval: EvalConfig
    wandb: Optional[WandbConfig] = None
    device_type: str = "cuda"


def evaluate_crosscoder(settings: EvaluateCrosscoderSettings) -> dict[str, float]:
    """Head-parallel evaluation: mesh ``("head", "model") = (n_factories, 1)``, one activation factory per head rank."""
    setup_logging(level="INFO")
    mesh = make_mesh(settings.device_type, (len(settings.activation_factories), 1), ("head", "model"))
    factory = ActivationFactory(settings.activation_factories[mesh_local_rank(mesh, "head")])
    sae = SparseDictionary.from_pretrained(
        settings.sae.pretrained_name_or_path, device_mesh=mesh, device=settings.sae.device, dtype=settings.sae.dtype,
        fold_activation_scale=settings.sae.fold_activation_scale, strict_loading=settings.sae.strict_loading,
    )  # fmt: skip
    wandb_logger = init_wandb(settings.wandb, settings, mesh)
    results = Evaluator(settings.eval).evaluate(sae, factory.process(), wandb_logger)
    logger.info("Evaluation completed")
    return results
