"""Helpers shared by the runners (runners/utils.py:34-72 of the reference project)."""

from __future__ import annotations

import os
from typing import Optional, TypeVar

from ..config import BaseModelConfig
from ..parallel.mesh import build_mesh, mesh_rank
from ..utils.logging import get_logger

logger = get_logger("runners.utils")
T = TypeVar("T")


def load_config(config: Optional[T], name: Optional[str], mongo_client, config_type: str, required: bool = True) -> Optional[T]:
    """Config given in the settings wins and is registered in the database under ``name``; otherwise it is
    looked up there. ``config_type`` is ``"model"`` or ``"dataset"``."""
    if mongo_client is not None and name is not None:
        if config is None:
            config = getattr(mongo_client, f"get_{config_type}_cfg")(name)
            logger.info(f"Loaded {config_type} config from database: {name}")
        else:
            getattr(mongo_client, f"add_{config_type}")(name, config)
            logger.info(f"Added {config_type} config to database: {name}")
    if required:
        assert config is not None, f"{config_type} config not provided and not found in database"
    return config


class PretrainedSAE(BaseModelConfig):
    pretrained_name_or_path: str
    fold_activation_scale: bool = True
    strict_loading: bool = True


def make_mesh(device_type: str, shape: tuple[int, ...], names: tuple[str, ...]):
    """Named device mesh, or None when every dimension is 1. On CUDA the process binds to ``LOCAL_RANK`` first."""
    if all(s == 1 for s in shape):
        return None
    if device_type == "cuda":
        import torch

        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    return build_mesh(device_type, shape, names)


def init_wandb(wandb_cfg, settings, device_mesh):
    """A wandb run on mesh rank 0 only (None elsewhere or when not configured)."""
    if wandb_cfg is None or (device_mesh is not None and mesh_rank(device_mesh) != 0):
        return None
    import wandb

    return wandb.init(
        project=wandb_cfg.wandb_project, config=settings.model_dump(mode="json"), name=wandb_cfg.exp_name,
        entity=wandb_cfg.wandb_entity, settings=wandb.Settings(x_disable_stats=True),
        mode=os.getenv("WANDB_MODE", "online"), resume=wandb_cfg.wandb_resume, id=wandb_cfg.wandb_run_id,
    )  # fmt: skip
