"""``convert_topk_to_jumprelu``: calibrate a JumpReLU threshold for a top-k cross-layer transcoder on an activation
stream and save the converted model (runners/topk_to_jumprelu_conversion.py:26-173 of the reference project)."""

from __future__ import annotations

from pathlib import Path
from typing import Optional

from pydantic_settings import BaseSettings

from ..activation.factory import ActivationFactory, ActivationFactoryConfig
from ..backend.language_model import LanguageModelConfig
from ..config import DatasetConfig
from ..database import MongoClient, MongoDBConfig
from ..models.clt import CrossLayerTranscoder
from ..models.sparse_dictionary import SparseDictionary
from ..parallel.mesh import is_primary_rank
from ..resource_loaders import load_dataset, load_model
from ..utils.logging import get_distributed_logger, setup_logging
from ..utils.topk_to_jumprelu_conversion import topk_to_jumprelu_conversion
from .utils import PretrainedSAE, load_config, make_mesh

logger = get_distributed_logger("runners.topk_to_jumprelu_conversion")


class ConvertTopKToJumpReLUSettings(BaseSettings):
    sae: PretrainedSAE
    sae_name: str
    sae_series: str
    activation_factory: ActivationFactoryConfig
    model_parallel_size: int = 1
    mongo: Optional[MongoDBConfig] = None
    model: Optional[LanguageModelConfig] = None
    model_name: Optional[str] = None
    datasets: Optional[dict[str, Optional[DatasetConfig]]] = None
    device_type: str = "cuda"
    exp_result_path: str


def convert_topk_to_jumprelu(settings: ConvertTopKToJumpReLUSettings) -> None:
    setup_logging(level="INFO")
    mesh = make_mesh(settings.device_type, (settings.model_parallel_size,), ("model",))
    mongo = MongoClient(settings.mongo) if settings.mongo is not None else None
    model_cfg = load_config(settings.model, settings.model_name, mongo, "model", required=False)
    dataset_cfgs = {n: load_config(c, n, mongo, "dataset") for n, c in settings.datasets.items()} if settings.datasets is not None else None
    model = load_model(model_cfg) if model_cfg is not None else None
    datasets = {n: load_dataset(c, device_mesh=mesh) for n, c in dataset_cfgs.items()} if dataset_cfgs is not None else None
    stream = ActivationFactory(settings.activation_factory, device_mesh=mesh).process(model=model, model_name=settings.model_name, datasets=datasets)
    sae = SparseDictionary.from_pretrained(
        settings.sae.pretrained_name_or_path, device_mesh=mesh, fold_activation_scale=False, device=settings.sae.device,
        dtype=settings.sae.dtype, strict_loading=settings.sae.strict_loading,
    )  # fmt: skip
    assert isinstance(sae, CrossLayerTranscoder), "Current implementation only supports CLTs"
    sae = topk_to_jumprelu_conversion(sae, activations_stream=stream, device_mesh=mesh)
    sae.save_pretrained(save_path=settings.exp_result_path)
    if is_primary_rank(mesh):
        sae.cfg.save_hyperparameters(settings.exp_result_path)
        if mongo is not None:
            mongo.create_sae(name=settings.sae_name, series=settings.sae_series, path=str(Path(settings.exp_result_path).absolute()), cfg=sae.cfg)
    logger.info("CLT conversion completed successfully")
