"""Training runners: ``train_sae``, ``train_crosscoder``, ``train_clt``, ``train_lorsa``, ``train_molt``, ``sweep_sae``.

Settings classes and the flow of every runner follow runners/train.py of the reference project (settings
:33-85, :258-300, :478-527, :691-740, :906-955, :1120-1176; flows :88-247, :302-475, :530-688, :743-903,
:958-1117, :1179-1338): build the mesh, open the database, resolve model / dataset configs, load them, build the
activation stream, build or load the dictionary (initializer / pretrained / plain config), build or resume the
trainer, save ``config.json``, fit, then save a full trainer checkpoint when the stream ended early or the final
weights (optionally folded) otherwise, and register the dictionary in the database.

The five single-model runners share one implementation here; meshes are ``("data", "model")`` (also for MOLT),
``("data", "head", "model")`` for crosscoders and ``("sweep", "data", "model")`` for sweeps, where every sweep member
trains on the ("data", "model") sub-mesh of its coordinate and all members read the same stream.
"""

from __future__ import annotations

import torch

from pathlib import Path
from typing import Any, Iterable, Optional

from pydantic import BaseModel
from pydantic_settings import BaseSettings

from ..activation.factory import ActivationFactory, ActivationFactoryConfig
from ..backend.language_model import LanguageModelConfig
from ..config import DatasetConfig
from ..database import MongoClient, MongoDBConfig
from ..initializer import Initializer, InitializerConfig
from ..models.clt import CLTConfig
from ..models.crosscoder import CrosscoderConfig
from ..models.lorsa import LorsaConfig
from ..models.molt import MOLTConfig
from ..models.sae import SAEConfig
from ..models.sparse_dictionary import SparseDictionary
from ..parallel.mesh import is_primary_rank
from ..resource_loaders import load_dataset, load_model
from ..trainer import Trainer, TrainerConfig, WandbConfig
from ..utils.logging import get_distributed_logger, setup_logging
from .utils import PretrainedSAE, init_wandb, load_config, make_mesh

logger = get_distributed_logger("runners.train")

AnySAEConfig = SAEConfig | CrosscoderConfig | CLTConfig | LorsaConfig | MOLTConfig


class _TrainSettingsBase(BaseSettings):
    sae_name: str
    sae_series: str
    initializer: InitializerConfig | None = None
    trainer: TrainerConfig
    wandb: Optional[WandbConfig] = None
    eval: bool = False
    data_parallel_size: int = 1
    model_parallel_size: int = 1
    mongo: Optional[MongoDBConfig] = None
    model: Optional[LanguageModelConfig] = None
    model_name: Optional[str] = None
    datasets: Optional[dict[str, Optional[DatasetConfig]]] = None
    device_type: str = "cuda"
    fold_activation_scale: bool = True


class TrainSAESettings(_TrainSettingsBase):
    sae: SAEConfig | PretrainedSAE
    activation_factory: ActivationFactoryConfig


class TrainCLTSettings(_TrainSettingsBase):
    sae: CLTConfig | PretrainedSAE
    activation_factory: ActivationFactoryConfig


class TrainLorsaSettings(_TrainSettingsBase):
    sae: LorsaConfig | PretrainedSAE
    activation_factory: ActivationFactoryConfig


class TrainMOLTSettings(_TrainSettingsBase):
    sae: MOLTConfig | PretrainedSAE
    activation_factory: ActivationFactoryConfig


class TrainCrosscoderSettings(_TrainSettingsBase):
    sae: CrosscoderConfig | PretrainedSAE
    activation_factories: list[ActivationFactoryConfig]
    """One per head-parallel rank; ``len(activation_factories) * len(hook_points of each)`` = number of heads."""


def _resources(settings, device_mesh):
    mongo = MongoClient(settings.mongo) if settings.mongo is not None else None
    model_cfg = load_config(settings.model, settings.model_name, mongo, "model", required=False)
    dataset_cfgs = (
        {n: load_config(c, n, mongo, "dataset") for n, c in settings.datasets.items()} if settings.datasets is not None else None
    )
    logger.info("Loading model and datasets")
    model = load_model(model_cfg) if model_cfg is not None else None
    datasets = {n: load_dataset(c, device_mesh=device_mesh) for n, c in dataset_cfgs.items()} if dataset_cfgs is not None else None
    return mongo, model, datasets


def _build_sae(sae_cfg, initializer_cfg, stream: Iterable[dict[str, Any]], device_mesh, wandb_logger, model) -> SparseDictionary:
    if isinstance(sae_cfg, PretrainedSAE):
        assert initializer_cfg is None, "Cannot use an initializer for a pretrained SAE"
        return SparseDictionary.from_pretrained(
            sae_cfg.pretrained_name_or_path, device_mesh=device_mesh, fold_activation_scale=False,
            strict_loading=sae_cfg.strict_loading, device=sae_cfg.device, dtype=sae_cfg.dtype,
        )  # fmt: skip
    if initializer_cfg is not None:
        return Initializer(initializer_cfg).initialize_sae_from_config(
            sae_cfg, activation_stream=stream, device_mesh=device_mesh, wandb_logger=wandb_logger, model=model
        )
    return SparseDictionary.from_config(sae_cfg, device_mesh=device_mesh)


def _fit_and_save(sae: SparseDictionary, trainer_cfg: TrainerConfig, stream, wandb_logger, mongo, sae_name, sae_series,
                  fold_activation_scale: bool, eval_enabled: bool, device_mesh, model_name: str | None) -> None:  # fmt: skip
    if trainer_cfg.from_pretrained_path is not None:
        trainer = Trainer.from_checkpoint(sae, trainer_cfg.from_pretrained_path)
        trainer.wandb_logger = wandb_logger
    else:
        trainer = Trainer(trainer_cfg)
    logger.info(f"SAE initialized: {type(sae).__name__}")
    if is_primary_rank(device_mesh):
        sae.cfg.save_hyperparameters(trainer_cfg.exp_result_path)
    end_of_stream = trainer.fit(sae=sae, activation_stream=stream, eval_fn=(lambda x: None) if eval_enabled else None,
                                wandb_logger=wandb_logger)  # fmt: skip
    logger.info("Training completed, saving model")
    if end_of_stream:
        trainer.save_checkpoint(sae=sae, checkpoint_path=trainer_cfg.exp_result_path)
    else:
        sae.save_pretrained(save_path=trainer_cfg.exp_result_path, fold_activation_scale=fold_activation_scale)
        if is_primary_rank(device_mesh):
            sae.cfg.save_hyperparameters(trainer_cfg.exp_result_path)
        if is_primary_rank(device_mesh) and mongo is not None:
            assert sae_name is not None and sae_series is not None, "sae_name and sae_series must be provided when saving to the database"
            mongo.create_sae(name=sae_name, series=sae_series, path=str(Path(trainer_cfg.exp_result_path).absolute()),
                             cfg=sae.cfg, model_name=model_name)  # fmt: skip
    if wandb_logger is not None:
        wandb_logger.finish()


def _train_single(settings) -> None:
    setup_logging(level="INFO")
    mesh = make_mesh(settings.device_type, (settings.data_parallel_size, settings.model_parallel_size), ("data", "model"))
    logger.info(f"Device mesh initialized: {mesh}")
    mongo, model, datasets = _resources(settings, mesh)
    factory = ActivationFactory(settings.activation_factory, device_mesh=mesh)
    stream = factory.process(model=model, model_name=settings.model_name, datasets=datasets)
    wandb_logger = init_wandb(settings.wandb, settings, mesh)
    sae = _build_sae(settings.sae, settings.initializer, stream, mesh, wandb_logger, model)
    _fit_and_save(sae, settings.trainer, stream, wandb_logger, mongo, settings.sae_name, settings.sae_series,
                  settings.fold_activation_scale, settings.eval, mesh, settings.model_name)  # fmt: skip
    logger.info("Training completed successfully")


def train_sae(settings: TrainSAESettings) -> None:
    """Train a sparse autoencoder / transcoder."""
    _train_single(settings)


def train_clt(settings: TrainCLTSettings) -> None:
    """Train a cross-layer transcoder."""
    _train_single(settings)


def train_lorsa(settings: TrainLorsaSettings) -> None:
    """Train a low-rank sparse attention dictionary (2-D activations: ``[batch, context, d]``)."""
    _train_single(settings)


def train_molt(settings: TrainMOLTSettings) -> None:
    """Train a mixture of linear transforms."""
    _train_single(settings)


def train_crosscoder(settings: TrainCrosscoderSettings) -> None:
    """Train a crosscoder with one activation factory per head-parallel rank."""
    setup_logging(level="INFO")
    facs = settings.activation_factories
    if isinstance(settings.sae, CrosscoderConfig):
        assert all(len(f.hook_points) == len(facs[0].hook_points) for f in facs), "Number of hook points of activation factories must be the same"
        assert len(facs) * len(facs[0].hook_points) == settings.sae.n_heads, "Total number of hook points must match the number of heads"
    head = len(facs)
    mesh = make_mesh(settings.device_type, (settings.data_parallel_size, head, settings.model_parallel_size), ("data", "head", "model"))
    mongo, model, datasets = _resources(settings, mesh)
    head_rank = mesh.get_local_rank("head") if mesh is not None else 0
    sub_mesh = mesh["data", "model"] if mesh is not None else None
    if mesh is not None and datasets is None and settings.datasets is not None:
        datasets = None
    factory = ActivationFactory(facs[head_rank], device_mesh=sub_mesh)
    stream = factory.process(model=model, model_name=settings.model_name, datasets=datasets)
    wandb_logger = init_wandb(settings.wandb, settings, mesh)
    sae = _build_sae(settings.sae, settings.initializer, stream, mesh, wandb_logger, model)
    _fit_and_save(sae, settings.trainer, stream, wandb_logger, mongo, settings.sae_name, settings.sae_series,
                  settings.fold_activation_scale, settings.eval, mesh, settings.model_name)  # fmt: skip


class SweepingItem(BaseModel):
    sae: AnySAEConfig | PretrainedSAE
    sae_name: str
    sae_series: str
    initializer: InitializerConfig | None = None
    trainer: TrainerConfig


class SweepSAESettings(BaseSettings):
    items: list[SweepingItem]
    activation_factory: ActivationFactoryConfig
    wandb: Optional[WandbConfig] = None
    eval: bool = False
    data_parallel_size: int = 1
    model_parallel_size: int = 1
    mongo: Optional[MongoDBConfig] = None
    model: Optional[LanguageModelConfig] = None
    model_name: Optional[str] = None
    datasets: Optional[dict[str, Optional[DatasetConfig]]] = None
    device_type: str = "cuda"
    fold_activation_scale: bool = True
    share_activation_stream: bool = True
    """Produce the activation stream once (on sweep coordinate 0) and broadcast every batch to the other members, so that all
    members train on the very same batches and the language model runs once instead of once per member. False: every
    member builds its own factory."""


def _shared_sweep_stream(own_stream, group, device):
    """The stream of sweep member 0, seen by every member of ``group``: per batch one small object broadcast (keys, shapes,
    dtypes, non-tensor values; ``None`` ends the stream) and one tensor broadcast per entry."""
    import torch.distributed as dist

    src = dist.get_rank(group) == 0
    it = iter(own_stream) if src else None
    while True:
        meta = None
        batch = None
        if src:
            try:
                batch = next(it)
                meta = {k: (("t", tuple(v.shape), v.dtype) if isinstance(v, torch.Tensor) else ("o", v)) for k, v in batch.items()}
            except StopIteration:
                meta = None
        box = [meta]
        dist.broadcast_object_list(box, group=group, group_src=0)
        meta = box[0]
        if meta is None:
            return
        out = {}
        for k, spec in meta.items():
            if spec[0] == "o":
                out[k] = spec[1]
                continue
            t = batch[k].to(device).contiguous() if src else torch.empty(spec[1], dtype=spec[2], device=device)
            dist.broadcast(t, group=group, group_src=0)
            out[k] = t
        yield out


def sweep_sae(settings: SweepSAESettings) -> None:
    """Train ``len(items)`` dictionaries side by side; member i runs on the sweep coordinate i of the mesh
    (runners/train.py:1179-1338 of the reference project, which replicates one stream over the ``sweep`` dimension)."""
    setup_logging(level="INFO")
    n = len(settings.items)
    mesh = make_mesh(settings.device_type, (n, settings.data_parallel_size, settings.model_parallel_size), ("sweep", "data", "model"))
    mongo, model, datasets = _resources(settings, mesh)
    sub_mesh = mesh["data", "model"] if mesh is not None else None
    if sub_mesh is not None and all(sub_mesh.size(i) == 1 for i in range(sub_mesh.ndim)):
        sub_mesh = None
    item = settings.items[mesh.get_local_rank("sweep") if mesh is not None else 0]
    logger.info(f"Processing sweep item: {item.sae_name}/{item.sae_series}")
    shared = settings.share_activation_stream and mesh is not None and n > 1
    sweep_rank = mesh.get_local_rank("sweep") if mesh is not None else 0
    stream = None
    if not shared or sweep_rank == 0:
        factory = ActivationFactory(settings.activation_factory, device_mesh=sub_mesh)
        stream = factory.process(model=model, model_name=settings.model_name, datasets=datasets)
    if shared:
        dev = torch.device(item.sae.device) if hasattr(item.sae, "device") else torch.device(settings.device_type)
        if dev.type == "cuda" and dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        stream = _shared_sweep_stream(stream, mesh.get_group("sweep"), dev)
    wandb_logger = init_wandb(settings.wandb, settings, sub_mesh)
    sae = _build_sae(item.sae, item.initializer, stream, sub_mesh, wandb_logger, model)
    _fit_and_save(sae, item.trainer, stream, wandb_logger, mongo, item.sae_name, item.sae_series, settings.fold_activation_scale,
                  settings.eval, sub_mesh, settings.model_name)  # fmt: skip
