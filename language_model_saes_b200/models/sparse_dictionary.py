"""Base class, configuration and registry of sparse dictionaries.

Behavioural contract: models/sparse_dictionary.py of the reference project (config fields :95-148, registry
:49-87, checkpoint I/O :262-331 / :548-695, normalisation modes :427-499, activation functions :713-796,
compute_loss :841-1007). The implementation differs in one structural way: under a device mesh every
parameter is a plain tensor holding this rank's shard (``dim_maps()`` says which dimension is split over
which mesh dimension) and collectives are explicit, instead of DTensor parameters with implicit
redistribution. On-disk formats are unchanged: ``config.json`` plus ``sae_weights.safetensors`` (full, logical
shapes) / ``.pt`` / ``.dcp``.
"""

from __future__ import annotations

import json
import math
import os
import shutil
import tempfile
from abc import ABC, abstractmethod
from enum import Enum
from pathlib import Path
from typing import Any, Callable, Literal

import torch
import torch.distributed as dist

from ..activation_functions import JumpReLU
from ..config import BaseModelConfig
from ..hooks import HookedRootModule
from ..parallel.collectives import distributed_topk
from ..parallel.mesh import (
    DeviceMesh,
    DimMap,
    execute_and_broadcast,
    is_primary_rank,
    mesh_dim_size,
    mesh_group,
)
from ..utils.logging import get_distributed_logger
from ..ops.select_kernels import positive_topk
from ..utils.math import topk
from ..utils.tensor_specs import TensorSpecs, apply_token_mask
from ..utils.timer import timer
from .protocols import DatasetNormStandardizable, NormComputing

logger = get_distributed_logger("sparse_dictionary")

__version__ = "0.1.0"

SAE_TYPE_TO_CONFIG_CLASS: dict[str, Any] = {}
SAE_TYPE_TO_MODEL_CLASS: dict[str, Any] = {}


def register_sae_config(name: str):
    """Class decorator: make ``name`` resolve to this config class when a ``config.json`` is read."""

    def _register(cls):
        SAE_TYPE_TO_CONFIG_CLASS[name] = cls
        return cls

    return _register


def register_sae_model(name: str):
    """Class decorator: make ``name`` resolve to this model class in ``SparseDictionary.from_config``."""

    def _register(cls):
        SAE_TYPE_TO_MODEL_CLASS[name] = cls
        return cls

    return _register


class PretrainedSAEType(Enum):
    LOCAL = "local"
    HUGGINGFACE = "huggingface"
    SAELENS = "saelens"


def auto_infer_pretrained_sae_type(pretrained_name_or_path: str) -> PretrainedSAEType:
    """A path that exists is local; ``<repo>:<name>`` is a SAELens release when SAELens knows it, otherwise
    a HuggingFace repository (utils/auto.py:21-70 of the reference)."""
    import importlib.util

    if os.path.exists(pretrained_name_or_path):
        return PretrainedSAEType.LOCAL
    parts = pretrained_name_or_path.split(":")
    if len(parts) != 2:
        raise ValueError(
            f"Pretrained name or path {pretrained_name_or_path} is not on disk, nor given in the "
            "HuggingFace/SAELens format <repo_id/release>:<name>."
        )
    repo_id, name = parts
    if importlib.util.find_spec("sae_lens") is not None:
        from sae_lens.loading.pretrained_saes_directory import get_pretrained_saes_directory

        lookups = get_pretrained_saes_directory()
        if lookups.get(repo_id) is not None and lookups[repo_id].saes_map.get(name) is not None:
            return PretrainedSAEType.SAELENS
    return PretrainedSAEType.HUGGINGFACE


class SparseDictionaryConfig(BaseModelConfig, ABC):
    """Fields shared by every dictionary type."""

    sae_type: str
    d_model: int
    expansion_factor: float
    use_decoder_bias: bool = True
    act_fn: Literal["relu", "jumprelu", "topk", "batchtopk", "batchlayertopk", "layertopk"] = "relu"
    norm_activation: Literal["token-wise", "batch-wise", "dataset-wise", "inference"] = "dataset-wise"
    sparsity_include_decoder_norm: bool = True
    top_k: int = 50
    sae_pretrained_name_or_path: str | None = None
    strict_loading: bool = True
    use_triton_kernel: bool = False
    """Kept for config compatibility. Here it selects the hand-written sparse decoder kernel on CUDA."""
    sparsity_threshold_for_triton_spmm_kernel: float = 0.996
    jumprelu_threshold_window: float = 2.0

    @property
    def d_sae(self) -> int:
        return int(self.d_model * self.expansion_factor)

    @classmethod
    def from_pretrained(cls, pretrained_name_or_path: str, strict_loading: bool = True, **kwargs):
        kind = auto_infer_pretrained_sae_type(pretrained_name_or_path)
        if kind == PretrainedSAEType.LOCAL:
            path = os.path.join(pretrained_name_or_path, "config.json")
        elif kind == PretrainedSAEType.HUGGINGFACE:
            from huggingface_hub import hf_hub_download

            repo_id, name = pretrained_name_or_path.split(":")
            path = hf_hub_download(repo_id=repo_id, filename=f"{name}/config.json")
        else:
            raise ValueError("Configs cannot be built from a SAELens release; load the whole model instead.")
        with open(path, "r") as f:
            d = json.load(f)
        d["sae_pretrained_name_or_path"] = pretrained_name_or_path
        d["strict_loading"] = strict_loading
        if cls is SparseDictionaryConfig:
            cls = SAE_TYPE_TO_CONFIG_CLASS[d["sae_type"]]
        return cls.model_validate({**d, **kwargs})

    def save_hyperparameters(self, sae_path: str | Path, remove_loading_info: bool = True):
        assert os.path.exists(sae_path), f"{sae_path} does not exist. Unable to save hyperparameters."
        d = self.model_dump()
        if remove_loading_info:
            d.pop("sae_pretrained_name_or_path", None)
            d.pop("strict_loading", None)
        with open(os.path.join(sae_path, "config.json"), "w") as f:
            json.dump(d, f, indent=4)

    @property
    @abstractmethod
    def associated_hook_points(self) -> list[str]: ...

    @property
    @abstractmethod
    def hooks_in(self) -> list[str]: ...

    @property
    @abstractmethod
    def hooks_out(self) -> list[str]: ...


class SparseDictionary(HookedRootModule, ABC):
    """Abstract sparse dictionary. Concrete classes implement ``encode``, ``decode``, ``prepare_input``,
    ``prepare_label`` and ``dim_maps`` and opt into the capability protocols of ``models.protocols``."""

    specs: type[TensorSpecs] = TensorSpecs

    def __init__(self, cfg: SparseDictionaryConfig, device_mesh: DeviceMesh | None = None):
        super().__init__()
        self.cfg = cfg
        self.current_k = cfg.top_k
        self.dataset_average_activation_norm: dict[str, float] | None = None
        self.device_mesh: DeviceMesh | None = device_mesh
        self.activation_function: Callable[[torch.Tensor], torch.Tensor] = self.activation_function_factory(device_mesh)

    # ---- mesh helpers ------------------------------------------------------------------------
    @property
    def tp_size(self) -> int:
        return mesh_dim_size(self.device_mesh, "model")

    @property
    def dp_size(self) -> int:
        return mesh_dim_size(self.device_mesh, "data")

    @property
    def tp_group(self):
        return mesh_group(self.device_mesh, "model")

    @property
    def dp_group(self):
        return mesh_group(self.device_mesh, "data")

    def local_shape(self, name: str, shape: tuple[int, ...]) -> tuple[int, ...]:
        """Shape of this rank's shard of parameter ``name`` whose full shape is ``shape``."""
        return self.dim_maps().get(name, DimMap({})).local_shape(shape, self.device_mesh)

    # ---- small setters -----------------------------------------------------------------------
    @torch.no_grad()
    def set_dataset_average_activation_norm(self, dataset_average_activation_norm: dict[str, float]):
        self.dataset_average_activation_norm = dataset_average_activation_norm

    @torch.no_grad()
    def set_current_k(self, current_k: int):
        self.current_k = current_k

    # ---- state / checkpoints -----------------------------------------------------------------
    @torch.no_grad()
    def full_state_dict(self) -> dict[str, torch.Tensor]:
        """Full (un-sharded, contiguous) tensors under their logical names. Collective under a mesh."""
        maps = self.dim_maps()
        out: dict[str, torch.Tensor] = {}
        for k, v in self.state_dict().items():
            t = v.detach()
            if self.device_mesh is not None and k in maps:
                t = maps[k].gather(t, self.device_mesh)
            out[k] = t.contiguous()
        norms = self.dataset_average_activation_norm
        for hp in self.cfg.associated_hook_points:
            val = norms[hp] if norms is not None and hp in norms else float("nan")
            out[f"dataset_average_activation_norm.{hp}"] = torch.tensor(val, device=self.cfg.device, dtype=self.cfg.dtype)
        return out

    @torch.no_grad()
    def save_checkpoint(self, ckpt_path: Path | str) -> None:
        suffix = Path(ckpt_path).suffix
        if suffix == ".dcp":
            import torch.distributed.checkpoint as dcp
            from torch.distributed.checkpoint import FileSystemWriter

            assert self.device_mesh is not None, "device_mesh must be provided when saving a DCP checkpoint"
            maps = self.dim_maps()
            sd = {
                k: maps.get(k, DimMap({})).from_local(v.detach().contiguous(), self.device_mesh)
                for k, v in self.state_dict().items()
            }
            dcp.save(sd, storage_writer=FileSystemWriter(ckpt_path))
            return
        state = self.full_state_dict()
        if not is_primary_rank(self.device_mesh):
            return
        if suffix == ".safetensors":
            import safetensors.torch as safe

            safe.save_file({k: v.cpu() for k, v in state.items()}, str(ckpt_path), {"version": __version__})
        elif suffix == ".pt":
            torch.save({"sae": state, "version": __version__}, ckpt_path)
        else:
            raise ValueError(f"Invalid checkpoint path {ckpt_path}: use .safetensors, .pt or .dcp")

    @torch.no_grad()
    def save_pretrained(self, save_path: Path | str, fold_activation_scale: bool = False) -> None:
        os.makedirs(Path(save_path), exist_ok=True)
        if fold_activation_scale:
            assert isinstance(self, DatasetNormStandardizable), f"{type(self).__name__} cannot fold the dataset norm"
            self.standardize_parameters_of_dataset_norm()
        # One logical safetensors file also under a mesh: it is what single-process readers expect and
        # sharded readers slice it directly.
        self.save_checkpoint(Path(save_path) / "sae_weights.safetensors")

    def load_full_state_dict(self, state_dict: dict[str, torch.Tensor], strict: bool = True) -> None:
        """Load full logical tensors (each rank keeps its shard) plus the dataset norms."""
        prefix = "dataset_average_activation_norm."
        norms = {k[len(prefix) :]: float(v) for k, v in state_dict.items() if k.startswith(prefix)}
        if norms and not any(math.isnan(v) for v in norms.values()):
            self.set_dataset_average_activation_norm(norms)
        maps = self.dim_maps()
        own = self.state_dict()
        local: dict[str, torch.Tensor] = {}
        for k, v in state_dict.items():
            if k.startswith(prefix):
                continue
            if self.device_mesh is not None and k in maps and k in own and tuple(v.shape) != tuple(own[k].shape):
                v = maps[k].shard(v, self.device_mesh)
            local[k] = v
        self.load_state_dict(local, strict=strict)

    @classmethod
    def from_config(cls, cfg: SparseDictionaryConfig, device_mesh: DeviceMesh | None = None):
        if cls is SparseDictionary:
            cls = SAE_TYPE_TO_MODEL_CLASS[cfg.sae_type]
        if cfg.sae_pretrained_name_or_path is not None:
            return cls.from_pretrained(
                cfg.sae_pretrained_name_or_path,
                device_mesh=device_mesh,
                fold_activation_scale=False,
                strict_loading=cfg.strict_loading,
                device=cfg.device,
                dtype=cfg.dtype,
            )
        model = cls(cfg, device_mesh)
        n = sum(p.numel() for p in model.parameters()) / 1e9
        logger.info(f"Initializing {cfg.sae_type} with {n:.2f} B parameters on this rank")
        return model

    @classmethod
    def from_local(
        cls,
        path: str,
        device_mesh: DeviceMesh | None = None,
        strict_loading: bool = True,
        fold_activation_scale: bool = False,
        **kwargs,
    ):
        cfg = SparseDictionaryConfig.from_pretrained(
            path if os.path.isdir(path) else str(Path(path).parent), strict_loading=strict_loading, **kwargs
        )
        cfg.sae_pretrained_name_or_path = None
        model = cls.from_config(cfg, device_mesh=device_mesh)
        ckpt = _find_checkpoint(path)
        if ckpt.endswith(".safetensors"):
            from safetensors import safe_open

            maps = model.dim_maps()
            overrides = model.override_dtypes()
            state: dict[str, torch.Tensor] = {}
            with safe_open(ckpt, framework="pt", device="cpu") as f:
                for key in f.keys():
                    sl = f.get_slice(key)
                    shape = tuple(sl.get_shape())
                    if device_mesh is not None and key in maps and len(shape) > 0:
                        t = sl[maps[key].local_slices(shape, device_mesh)]
                    else:
                        t = f.get_tensor(key)
                    if not key.startswith("dataset_average_activation_norm."):
                        t = t.to(device=cfg.device, dtype=overrides.get(key, cfg.dtype) if t.is_floating_point() else t.dtype)
                    state[key] = t
        elif ckpt.endswith(".pt"):
            state = torch.load(ckpt, map_location=cfg.device, weights_only=True)["sae"]
        elif ckpt.endswith(".dcp"):
            import torch.distributed.checkpoint as dcp
            from torch.distributed.checkpoint import FileSystemReader

            assert device_mesh is not None, "loading a .dcp checkpoint needs a device mesh"
            maps = model.dim_maps()
            dt = {
                k: maps.get(k, DimMap({})).from_local(v.detach().contiguous(), device_mesh)
                for k, v in model.state_dict().items()
            }
            dcp.load(dt, storage_reader=FileSystemReader(ckpt))
            state = {k: v.to_local() for k, v in dt.items()}
        else:
            raise ValueError(f"Unsupported checkpoint format: {ckpt}")
        model.load_full_state_dict(state, strict=strict_loading)
        if fold_activation_scale and cfg.norm_activation == "dataset-wise":
            # checkpoints saved with the scale already folded carry norm_activation="inference" and need nothing
            assert isinstance(model, DatasetNormStandardizable), f"{type(model).__name__} cannot fold the dataset norm"
            model.standardize_parameters_of_dataset_norm()
        return model

    @classmethod
    def from_pretrained(
        cls,
        pretrained_name_or_path: str,
        *,
        device_mesh: DeviceMesh | None = None,
        fold_activation_scale: bool = False,
        strict_loading: bool = True,
        **kwargs: Any,
    ):
        """Local directory, ``<hf repo>:<name>`` or ``<saelens release>:<sae id>``."""
        kind = auto_infer_pretrained_sae_type(pretrained_name_or_path)
        if kind == PretrainedSAEType.LOCAL:
            return cls.from_local(
                pretrained_name_or_path,
                device_mesh=device_mesh,
                fold_activation_scale=fold_activation_scale,
                strict_loading=strict_loading,
                **kwargs,
            )
        if kind == PretrainedSAEType.HUGGINGFACE:
            repo_id, name = pretrained_name_or_path.split(":")
            return cls.from_hf(
                repo_id, name, device_mesh=device_mesh, fold_activation_scale=fold_activation_scale,
                strict_loading=strict_loading, **kwargs,
            )  # fmt: skip
        assert device_mesh is None, "SAELens checkpoints load on a single process; shard afterwards"
        from sae_lens import SAE

        from .sae import SparseAutoEncoder

        assert cls is SparseDictionary or cls is SparseAutoEncoder, "SAELens only has the vanilla SAE architecture"
        release, sae_id = pretrained_name_or_path.split(":")
        return SparseAutoEncoder.from_saelens(SAE.from_pretrained(release, sae_id), **kwargs)

    def upload_to_hf(self, repo_id: str, name: str, lm_config=None, *, token: str | None = None, private: bool = False):
        from huggingface_hub import create_repo, upload_folder

        tmp_root = execute_and_broadcast(lambda: tempfile.mkdtemp(prefix="sae_upload_"), self.device_mesh)
        try:
            self.save_pretrained(tmp_root)
            if is_primary_rank(self.device_mesh):
                self.cfg.save_hyperparameters(tmp_root)
                if lm_config is not None:
                    lm_config.save_lm_config(tmp_root)
                create_repo(repo_id=repo_id, private=private, exist_ok=True, token=token)
                upload_folder(
                    folder_path=tmp_root, repo_id=repo_id, path_in_repo=name,
                    commit_message=f"Upload pretrained sparse dictionary {name}", token=token,
                )  # fmt: skip
        finally:
            if is_primary_rank(self.device_mesh):
                shutil.rmtree(tmp_root, ignore_errors=True)

    @classmethod
    def from_hf(cls, repo_id: str, name: str, *, device_mesh=None, token=None, strict_loading=True,
                fold_activation_scale=False, **kwargs):  # fmt: skip
        from huggingface_hub import snapshot_download

        snapshot = execute_and_broadcast(
            lambda: snapshot_download(repo_id=repo_id, allow_patterns=[f"{name}/*"], token=token), device_mesh
        )
        local = os.path.join(snapshot, name)
        if not (Path(local) / "config.json").exists():
            raise FileNotFoundError(f"Sparse dictionary {name} does not exist in repo {repo_id}")
        return cls.from_local(local, device_mesh=device_mesh, strict_loading=strict_loading,
                              fold_activation_scale=fold_activation_scale, **kwargs)  # fmt: skip


    # ---- activation normalisation ------------------------------------------------------------
    def compute_norm_factor(self, x: torch.Tensor, hook_point: str) -> torch.Tensor:
        """Scale that brings activations to an average norm of sqrt(d_model) under the configured mode."""
        mode = self.cfg.norm_activation
        root = math.sqrt(self.cfg.d_model)
        if mode == "token-wise":
            return root / torch.norm(x, 2, dim=-1, keepdim=True)
        if mode == "batch-wise":
            return root / torch.norm(x, 2, dim=-1, keepdim=True).mean(dim=-2, keepdim=True)
        if mode == "dataset-wise":
            assert self.dataset_average_activation_norm is not None, (
                "dataset_average_activation_norm must be provided from Initializer"
            )
            return torch.tensor(root / self.dataset_average_activation_norm[hook_point], device=x.device, dtype=x.dtype)
        if mode == "inference":
            return torch.tensor(1.0, device=x.device, dtype=x.dtype)
        raise ValueError(f"Not implemented norm_activation {mode}")

    @timer.time("normalize_activations")
    def normalize_activations(self, batch: dict[str, torch.Tensor], *, return_scale_factor: bool = False):
        hooks = set(self.cfg.associated_hook_points)
        scale = {k: self.compute_norm_factor(v, hook_point=k) for k, v in batch.items() if k in hooks}
        out = {k: (v * scale[k] if k in hooks else v) for k, v in batch.items()}
        return (out, scale) if return_scale_factor else out

    def denormalize_activations(self, batch: dict[str, torch.Tensor], scale_factors: dict[str, torch.Tensor]):
        return {k: v / scale_factors[k] for k, v in batch.items()}

    # ---- optimisation helpers ----------------------------------------------------------------
    def get_parameters(self) -> list[dict[str, Any]]:
        """Two parameter groups: ``jumprelu`` (threshold, own learning-rate factor) and ``others``."""
        jr = list(self.activation_function.parameters()) if isinstance(self.activation_function, JumpReLU) else []
        jr_ids = {id(p) for p in jr}
        others = [p for p in self.parameters() if id(p) not in jr_ids]
        return [{"params": others, "name": "others"}, {"params": jr, "name": "jumprelu"}]

    @torch.no_grad()
    def log_statistics(self) -> dict[str, Any]:
        out: dict[str, Any] = {}
        if isinstance(self, NormComputing):
            out["metrics/encoder_norm"] = self._mean_over_shards(self.encoder_norm())
            out["metrics/decoder_norm"] = self._mean_over_shards(self.decoder_norm())
            if self.cfg.use_decoder_bias:
                out["metrics/decoder_bias_norm"] = float(self.decoder_bias_norm().mean())
        if "topk" in self.cfg.act_fn:
            out["sparsity/k"] = self.current_k
        if isinstance(self.activation_function, JumpReLU):
            out["metrics/mean_jumprelu_threshold"] = self._mean_over_shards(
                self.activation_function.log_jumprelu_threshold.exp()
            )
        return out

    def _mean_over_shards(self, t: torch.Tensor) -> float:
        """Mean of a per-feature quantity whose feature axis may be sharded over ``model``."""
        s = torch.stack([t.float().sum(), torch.tensor(float(t.numel()), device=t.device)])
        if self.tp_size > 1:
            dist.all_reduce(s, group=self.tp_group)
        return float(s[0] / s[1])

    # ---- activation functions ----------------------------------------------------------------
    def activation_function_factory(self, device_mesh: DeviceMesh | None = None):
        """relu | jumprelu | topk | batchtopk on (possibly feature-sharded) pre-activations.

        Single-process TopK applies ReLU first and keeps exactly k entries; under feature sharding the global
        k-th value is found with one candidate all-gather. BatchTopK keeps the ``k * batch`` largest entries
        of the whole (local-batch x full-feature) matrix.
        """
        act = self.cfg.act_fn.lower()
        assert act in ("relu", "topk", "jumprelu", "batchtopk"), f"Not implemented activation function {act}"
        if act == "relu":
            return lambda x: x * x.gt(0).to(x.dtype)
        if act == "jumprelu":
            return JumpReLU(
                self.cfg.jumprelu_threshold_window, shape=(self.cfg.d_sae,), device=self.cfg.device,
                dtype=self.cfg.dtype, device_mesh=device_mesh,
            )  # fmt: skip
        if act == "topk":

            def topk_activation(x: torch.Tensor):
                if self.tp_size > 1:
                    return distributed_topk(x, self.current_k, self.tp_group, dim=-1)
                x = x * x.gt(0).to(x.dtype)
                return topk(x, k=min(self.current_k, x.shape[-1]), dim=-1)

            return topk_activation

        def batch_topk(x: torch.Tensor):
            x = x * x.gt(0).to(x.dtype)
            shape = x.shape
            if x.ndim == 3:
                x = x.flatten(end_dim=1)
            k_total = self.current_k * x.size(0)
            # on a GPU: exact threshold by radix select (two streaming passes; shards add their histograms)
            out = positive_topk(x, k_total, (-2, -1), self.tp_group if self.tp_size > 1 else None)
            if out is None and self.tp_size > 1:
                out = distributed_topk(x, k_total, self.tp_group, dim=(-2, -1))
            elif out is None:
                out = topk(x, k=min(k_total, x.numel()), dim=(-2, -1), abs=True)
            return out.reshape(shape)

        return batch_topk

    @torch.no_grad()
    def init_parameters(self, **kwargs):
        if isinstance(self.activation_function, JumpReLU):
            self.activation_function.log_jumprelu_threshold.data.fill_(kwargs["init_log_jumprelu_threshold_value"])

    # ---- abstract model interface ------------------------------------------------------------
    @abstractmethod
    def encode(self, x: torch.Tensor, return_hidden_pre: bool = False, **kwargs): ...

    @abstractmethod
    def decode(self, feature_acts: torch.Tensor, **kwargs) -> torch.Tensor: ...

    @timer.time("forward")
    def forward(self, x: torch.Tensor, encoder_kwargs: dict[str, Any] = {}, decoder_kwargs: dict[str, Any] = {}):
        return self.decode(self.encode(x, **encoder_kwargs), **decoder_kwargs)

    @abstractmethod
    def prepare_input(self, batch: dict[str, torch.Tensor], **kwargs) -> tuple[torch.Tensor, dict[str, Any], dict[str, Any]]: ...

    @abstractmethod
    def prepare_label(self, batch: dict[str, torch.Tensor], **kwargs) -> torch.Tensor: ...

    @torch.no_grad()
    def compute_training_metrics(self, **kwargs) -> dict[str, float]:
        return {}

    def dim_maps(self) -> dict[str, DimMap]:
        maps: dict[str, DimMap] = {}
        if isinstance(self.activation_function, JumpReLU):
            maps.update({f"activation_function.{k}": v for k, v in self.activation_function.dim_maps().items()})
        return maps

    def override_dtypes(self) -> dict[str, torch.dtype]:
        if isinstance(self.activation_function, JumpReLU):
            return {f"activation_function.{k}": v for k, v in self.activation_function.override_dtypes().items()}
        return {}

    def _sum_over_features(self, t: torch.Tensor) -> torch.Tensor:
        """Finish a sum over the (sharded) feature axis: adds the other shards' partial sums."""
        if self.tp_size > 1:
            from ..parallel.collectives import all_reduce_sum

            return all_reduce_sum(t, self.tp_group)
        return t

    # ---- loss --------------------------------------------------------------------------------
    @timer.time("compute_loss")
    def compute_loss(
        self,
        batch: dict[str, torch.Tensor],
        label: torch.Tensor | None = None,
        *,
        sparsity_loss_type: Literal["power", "tanh", "tanh-quad", None] = None,
        tanh_stretch_coefficient: float = 4.0,
        frequency_scale: float = 0.01,
        p: int = 1,
        l1_coefficient: float = 1.0,
        lp_coefficient: float = 0.0,
        auxk_coefficient: float = 0.0,
        k_aux: int = 512,
        update_dead_statistics: Callable[[torch.Tensor, torch.Tensor | None, tuple[str, ...]], torch.Tensor] | None = None,
        return_aux_data: bool = True,
        **kwargs,
    ):
        """Reconstruction MSE (sum over d_model, mean over tokens) plus the optional sparsity, JumpReLU-Lp and
        Aux-K terms. Inputs must already be normalised. Under feature sharding ``feature_acts`` and
        ``hidden_pre`` are local shards and per-token sums over features are completed across shards; under
        data parallelism the returned loss is the mean over this rank's tokens."""
        x, encoder_kwargs, decoder_kwargs = self.prepare_input(batch)
        label = self.prepare_label(batch, **kwargs)
        mask = batch.get("mask")

        with timer.time("encode"):
            feature_acts, hidden_pre = self.encode(x, return_hidden_pre=True, **encoder_kwargs)
        with timer.time("decode"):
            reconstructed = self.decode(feature_acts, **decoder_kwargs)

        full_mask = mask
        with timer.time("loss_calculation"):
            l_rec = (reconstructed - label).pow(2).sum(dim=-1)
            if mask is not None and mask.ndim < l_rec.ndim:
                # per-token losses with extra trailing axes (heads / layers): every entry of a token shares its mask
                mask = mask.reshape(*mask.shape, *([1] * (l_rec.ndim - mask.ndim))).expand_as(l_rec)
            l_rec, _ = apply_token_mask(l_rec, self.specs.loss(l_rec), mask, "mean")
            loss_dict: dict[str, torch.Tensor | None] = {"l_rec": l_rec}
            loss = l_rec

            if sparsity_loss_type is not None:
                assert isinstance(self, NormComputing), "NormComputing is required for sparsity loss computation"
                gated = feature_acts * self.decoder_norm()
                if sparsity_loss_type == "power":
                    if p == 1:
                        l_s = self._sum_over_features(gated.abs().sum(dim=-1))
                    else:
                        l_s = self._sum_over_features(gated.abs().pow(p).sum(dim=-1)).pow(1.0 / p)
                elif sparsity_loss_type == "tanh":
                    l_s = self._sum_over_features(torch.tanh(tanh_stretch_coefficient * gated).sum(dim=-1))
                elif sparsity_loss_type == "tanh-quad":
                    score = torch.tanh(tanh_stretch_coefficient * gated)
                    freq = score.reshape(-1, score.shape[-1]).mean(dim=0)
                    if self.dp_size > 1:
                        from ..parallel.collectives import all_reduce_sum

                        freq = all_reduce_sum(freq, self.dp_group) / self.dp_size
                    l_s = self._sum_over_features((freq * (1 + freq / frequency_scale)).sum(dim=-1))
                else:
                    raise ValueError(f"sparsity_loss_type {sparsity_loss_type} not supported.")
                l_s = l1_coefficient * l_s
                loss_dict["l_s"] = l_s
                if l_s.ndim > 0:
                    l_s, _ = apply_token_mask(l_s, self.specs.loss(l_s), mask, "mean")
                loss = loss + l_s
            else:
                loss_dict["l_s"] = None

            if lp_coefficient > 0.0 and isinstance(self.activation_function, JumpReLU):
                assert isinstance(self, NormComputing), "NormComputing is required for Lp loss computation"
                thr = self.activation_function.get_jumprelu_threshold()
                l_p = torch.nn.functional.relu(thr - hidden_pre) * self.decoder_norm()
                l_p = lp_coefficient * self._sum_over_features(l_p.sum(dim=-1))
                l_p, _ = apply_token_mask(l_p, self.specs.loss(l_p), mask, "mean")
                loss_dict["l_p"] = l_p
                loss = loss + l_p
            else:
                loss_dict["l_p"] = None

            if auxk_coefficient > 0.0:
                assert update_dead_statistics is not None, "update_dead_statistics must be set when auxk_coefficient > 0.0"
                is_dead = update_dead_statistics(feature_acts, mask, self.specs.feature_acts(feature_acts))
                e = label - reconstructed
                saved_k = self.current_k
                n_dead = is_dead.sum()
                if self.tp_size > 1:
                    n_dead = n_dead.clone()
                    dist.all_reduce(n_dead, group=self.tp_group)
                self.current_k = min(k_aux, int(n_dead))
                if self.current_k > 0:
                    gate = self.decoder_norm() if self.cfg.sparsity_include_decoder_norm else None  # type: ignore[attr-defined]
                    dead_pre = hidden_pre * is_dead.to(hidden_pre.dtype)
                    if gate is not None:
                        dead_pre = dead_pre * gate
                    dead_acts = self.activation_function(dead_pre)
                    if gate is not None:
                        dead_acts = dead_acts / gate
                    aux_rec = self._sum_over_features(self._decode_linear(dead_acts))
                    l_aux = auxk_coefficient * (e - aux_rec).pow(2).sum(dim=-1)
                    l_aux, _ = apply_token_mask(l_aux, self.specs.loss(l_aux), mask, "mean")
                    loss_dict["l_aux"] = l_aux
                    loss = loss + l_aux
                else:
                    loss_dict["l_aux"] = torch.zeros_like(l_rec)
                self.current_k = saved_k

        if not return_aux_data:
            return loss
        n_tokens = batch["tokens"].numel() if full_mask is None else int(full_mask.sum())
        return {
            "loss": loss,
            **loss_dict,
            "label": label,
            "mask": full_mask,
            "n_tokens": n_tokens,
            "feature_acts": feature_acts,
            "reconstructed": reconstructed,
            "hidden_pre": hidden_pre,
            "l1_coefficient": l1_coefficient,
            "lp_coefficient": lp_coefficient,
            "auxk_coefficient": auxk_coefficient,
        }

    def _decode_linear(self, feature_acts: torch.Tensor) -> torch.Tensor:
        """``feature_acts @ W_D`` on the local shard, without bias, hooks or cross-shard reduction
        (the Aux-K reconstruction of models/sparse_dictionary.py:975 in the reference)."""
        return feature_acts @ self.W_D  # type: ignore[attr-defined]


def _find_checkpoint(path: str) -> str:
    """Weights file for a checkpoint directory, in the reference's priority order."""
    if path.endswith((".pt", ".safetensors", ".dcp")):
        return path
    for stem in ("sae_weights", "checkpoints/pruned", "checkpoints/final"):
        for ext in ("safetensors", "pt", "dcp"):
            cand = f"{path}/{stem}.{ext}"
            if os.path.exists(cand):
                return cand
    raise FileNotFoundError(f"Pretrained model not found at {path}")
