"""Initialisation of a sparse dictionary before training.

Steps and options follow initializer.py of the reference project (InitializerConfig :30-56,
initialize_parameters :64-81, initialization_search :83-162, initialize_sae_from_config :164-271):
uniform parameter init, encoder <- decoder^T, dataset-norm estimation, optional initialisation from the
language model's attention / MLP, optional active-subspace projection, decoder bias <- mean label, coarse (50
points in [0.1, 5]) then fine (20 points around the best) grid search of the decoder row norm, optional encoder
bias <- -mean pre-activation.

The grid search evaluates ~70 forward passes on one batch; the loss values stay on the device and are read back
once per sweep instead of once per candidate.
"""

from __future__ import annotations

from typing import Iterable, Literal

import torch
from torch import Tensor

from .config import BaseConfig
from .models.protocols import (
    ActiveSubspaceInitializable,
    EncoderBiasInitializable,
    EncoderInitializable,
    NormConstrainable,
)
from .models.sparse_dictionary import SparseDictionary, SparseDictionaryConfig
from .utils.logging import get_distributed_logger
from .utils.misc import calculate_activation_norm

logger = get_distributed_logger("initializer")


class InitializerConfig(BaseConfig):
    bias_init_method: Literal["all_zero", "geometric_median"] = "all_zero"
    decoder_uniform_bound: float = 1.0
    encoder_uniform_bound: float = 1.0
    init_encoder_with_decoder_transpose: bool = True
    init_encoder_with_decoder_transpose_factor: float = 1.0
    init_log_jumprelu_threshold_value: float | None = None
    grid_search_init_norm: bool = False
    initialize_W_D_with_active_subspace: bool = False
    d_active_subspace: int | None = None
    initialize_lorsa_with_mhsa: bool | None = None
    initialize_tc_with_mlp: bool | None = None
    model_layer: int | None = None
    init_encoder_bias_with_mean_hidden_pre: bool = False


class Initializer:
    def __init__(self, cfg: InitializerConfig):
        self.cfg = cfg

    @torch.no_grad()
    def initialize_parameters(self, sae: SparseDictionary) -> SparseDictionary:
        sae.init_parameters(
            encoder_uniform_bound=self.cfg.encoder_uniform_bound,
            decoder_uniform_bound=self.cfg.decoder_uniform_bound,
            init_log_jumprelu_threshold_value=self.cfg.init_log_jumprelu_threshold_value,
        )
        self._tie_encoder(sae)
        return sae

    def _tie_encoder(self, sae: SparseDictionary) -> None:
        if self.cfg.init_encoder_with_decoder_transpose:
            assert isinstance(sae, EncoderInitializable), f"{type(sae).__name__} cannot tie its encoder to its decoder"
            sae.init_encoder_with_decoder_transpose(self.cfg.init_encoder_with_decoder_transpose_factor)

    def _init_encoder_bias(self, sae: SparseDictionary, batch: dict[str, Tensor]) -> None:
        if self.cfg.init_encoder_bias_with_mean_hidden_pre:
            assert isinstance(sae, EncoderBiasInitializable), f"{type(sae).__name__} cannot initialise its encoder bias"
            sae.init_encoder_bias_with_mean_hidden_pre(batch)

    @torch.no_grad()
    def _init_decoder_bias(self, sae: SparseDictionary, batch: dict[str, Tensor]) -> None:
        """``"geometric_median"`` sets b_D to the per-dimension MEAN of the (normalised) labels, like the
        reference does despite the option's name."""
        from .models.clt import CrossLayerTranscoder

        if isinstance(sae, CrossLayerTranscoder):
            for i, hp in enumerate(sae.cfg.hook_points_out):
                sae.b_D[i].copy_(batch[hp].reshape(-1, batch[hp].shape[-1]).mean(0))
            return
        label = sae.prepare_label(batch)
        if not hasattr(sae, "b_D") or sae.b_D.ndim != 1:
            raise ValueError(f"Bias initialization method {self.cfg.bias_init_method} is not supported for {sae.cfg.sae_type}")
        sae.b_D.copy_(label.reshape(-1, label.shape[-1]).mean(0))

    @torch.no_grad()
    def initialization_search(self, sae: SparseDictionary, activation_batch: dict[str, Tensor], wandb_logger=None):
        batch = sae.normalize_activations(activation_batch)
        if self.cfg.bias_init_method == "geometric_median":
            self._init_decoder_bias(sae, batch)

        def sweep(norms: list[float]) -> float:
            assert isinstance(sae, NormConstrainable), f"{type(sae).__name__} does not support norm constraints"
            losses = []
            for norm in norms:
                sae.set_decoder_to_fixed_norm(norm, force_exact=True)
                self._tie_encoder(sae)
                self._init_encoder_bias(sae, batch)
                losses.append(sae.compute_loss(batch)["l_rec"].float().mean())
            return norms[int(torch.stack(losses).argmin())]

        if self.cfg.grid_search_init_norm:
            coarse = sweep(torch.linspace(0.1, 5.0, 50).tolist())
            best = sweep(torch.linspace(coarse - 0.09, coarse + 0.1, 20).tolist())
            logger.info(f"The best (i.e. lowest MSE) initialized norm is {best}")
            if wandb_logger is not None:
                wandb_logger.log({"best_norm_fine_grained": best})
            sae.set_decoder_to_fixed_norm(best, force_exact=True)  # type: ignore[attr-defined]
        self._tie_encoder(sae)
        self._init_encoder_bias(sae, batch)
        return sae

    def initialize_sae_from_config(
        self,
        cfg: SparseDictionaryConfig,
        activation_stream: Iterable[dict[str, Tensor]] | None = None,
        activation_norm: dict[str, float] | None = None,
        device_mesh=None,
        wandb_logger=None,
        model=None,
    ) -> SparseDictionary:
        from .models.lorsa import LowRankSparseAttention
        from .models.sae import SparseAutoEncoder

        sae = SparseDictionary.from_config(cfg, device_mesh=device_mesh)
        if cfg.sae_pretrained_name_or_path is not None:
            return sae
        sae = self.initialize_parameters(sae)
        if sae.cfg.norm_activation == "dataset-wise":
            if activation_norm is None:
                assert activation_stream is not None, "Activation iterator must be provided for dataset-wise normalization"
                activation_norm = calculate_activation_norm(activation_stream, cfg.associated_hook_points, device_mesh=device_mesh)
            sae.set_dataset_average_activation_norm(activation_norm)

        layer = self.cfg.model_layer
        if isinstance(sae, LowRankSparseAttention) and self.cfg.initialize_lorsa_with_mhsa:
            assert sae.cfg.norm_activation == "dataset-wise", "Lorsa MHSA initialisation needs dataset-wise normalisation"
            assert model is not None and layer is not None, "a hooked language model and model_layer are required"
            sae.init_lorsa_with_mhsa(model.attention_module(layer))

        assert activation_stream is not None, "Activation iterator must be provided for initialization search"
        activation_batch = next(iter(activation_stream))
        dev = next(sae.parameters()).device
        activation_batch = {k: (v.to(dev) if isinstance(v, Tensor) else v) for k, v in activation_batch.items()}

        if isinstance(sae, SparseAutoEncoder) and sae.cfg.hook_point_in != sae.cfg.hook_point_out and self.cfg.initialize_tc_with_mlp:
            assert sae.cfg.norm_activation == "dataset-wise" and model is not None and layer is not None
            sae.init_tc_with_mlp(batch=sae.normalize_activations(activation_batch), mlp=model.mlp_module(layer))

        if self.cfg.initialize_W_D_with_active_subspace:
            batch = sae.normalize_activations(activation_batch)
            if isinstance(sae, LowRankSparseAttention):
                assert sae.cfg.norm_activation == "dataset-wise" and model is not None and layer is not None
                sae.init_W_V_with_active_subspace_per_head(batch=batch, mhsa=model.attention_module(layer))
            else:
                assert self.cfg.d_active_subspace is not None, "d_active_subspace must be provided"
                assert isinstance(sae, ActiveSubspaceInitializable), f"{type(sae).__name__} has no active-subspace init"
                sae.init_W_D_with_active_subspace(batch=batch, d_active_subspace=self.cfg.d_active_subspace)

        return self.initialization_search(sae, activation_batch, wandb_logger=wandb_logger)
