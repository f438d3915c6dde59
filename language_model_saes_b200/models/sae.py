"""Sparse autoencoder / transcoder (optionally with a GLU encoder).

Behaviour follows models/sae.py of the reference project: parameters and logical shapes ``W_E [d, F]``,
``b_E [F]``, ``W_D [F, d]``, ``b_D [d]`` (+ ``W_E_glu``, ``b_E_glu``) (:66-75), decoder-norm gating around the
activation function (:333-341), norm utilities (:136-212), dataset-norm folding (:214-255), initialisers
(:389-515) and SAELens conversion (:517-663).

Storage differs on purpose: ``W_E`` is a *transposed view* of a feature-major ``[F, d]`` buffer, so both
weight matrices are row-per-feature in memory. That is the K-major operand layout the tcgen05 encoder GEMM
reads through TMA and the layout in which the fused sparse-gradient Adam kernel walks both matrices; the
logical shape, state-dict key and checkpoint format are unchanged. Under feature (``model``) parallelism each
rank holds ``F / tp`` features.
"""

from __future__ import annotations

import math
from typing import Any

import torch
import torch.distributed as dist
from torch import nn

from ..activation_functions import JumpReLU
from ..hooks import HookPoint
from ..parallel.collectives import all_reduce_sum
from ..parallel.mesh import DeviceMesh, DimMap, mesh_local_rank
from .sparse_dictionary import SparseDictionary, SparseDictionaryConfig, register_sae_config, register_sae_model


@register_sae_config("sae")
class SAEConfig(SparseDictionaryConfig):
    sae_type: str = "sae"
    hook_point_in: str
    hook_point_out: str
    use_glu_encoder: bool = False

    @property
    def associated_hook_points(self) -> list[str]:
        return [self.hook_point_in, self.hook_point_out]

    @property
    def hooks_in(self) -> list[str]:
        return [self.hook_point_in]

    @property
    def hooks_out(self) -> list[str]:
        return [self.hook_point_out]


def _feature_major_param(d: int, f: int, device, dtype) -> nn.Parameter:
    """Parameter of logical shape [d, f] stored as a contiguous [f, d] buffer."""
    return nn.Parameter(torch.empty(f, d, device=device, dtype=dtype).t())


def shard_generator(device_mesh: DeviceMesh | None, device) -> torch.Generator:
    """Generator whose seed is shared by all data-parallel replicas of a shard and differs between
    feature shards, so that random initialisation is consistent without materialising full tensors."""
    seed = torch.randint(0, 2**31 - 1, (1,), dtype=torch.int64)
    if device_mesh is not None and dist.is_initialized():
        seed = seed.to(device) if torch.device(device).type == "cuda" else seed
        dist.broadcast(seed, src=0)
        seed = seed.cpu()
    g = torch.Generator(device=device)
    g.manual_seed(int(seed) + 7919 * mesh_local_rank(device_mesh, "model") + 104729 * mesh_local_rank(device_mesh, "head"))
    return g


@register_sae_model("sae")
class SparseAutoEncoder(SparseDictionary):
    def __init__(self, cfg: SAEConfig, device_mesh: DeviceMesh | None = None):
        super().__init__(cfg, device_mesh=device_mesh)
        self.cfg: SAEConfig = cfg
        d, F = cfg.d_model, cfg.d_sae
        (F_l,) = DimMap({"model": 0}).local_shape((F,), device_mesh)
        self.d_sae_local = F_l
        dev, dt = cfg.device, cfg.dtype
        self.W_E = _feature_major_param(d, F_l, dev, dt)
        self.b_E = nn.Parameter(torch.empty(F_l, device=dev, dtype=dt))
        self.W_D = nn.Parameter(torch.empty(F_l, d, device=dev, dtype=dt))
        if cfg.use_decoder_bias:
            self.b_D = nn.Parameter(torch.empty(d, device=dev, dtype=dt))
        if cfg.use_glu_encoder:
            self.W_E_glu = _feature_major_param(d, F_l, dev, dt)
            self.b_E_glu = nn.Parameter(torch.empty(F_l, device=dev, dtype=dt))
        self.hook_hidden_pre = HookPoint()
        self.hook_feature_acts = HookPoint()
        self.hook_reconstructed = HookPoint()
        self.setup()

    # ---- sharding ----------------------------------------------------------------------------
    def dim_maps(self) -> dict[str, DimMap]:
        maps = {"W_E": DimMap({"model": 1}), "W_D": DimMap({"model": 0}), "b_E": DimMap({"model": 0})}
        if self.cfg.use_decoder_bias:
            maps["b_D"] = DimMap({})
        if self.cfg.use_glu_encoder:
            maps["W_E_glu"] = DimMap({"model": 1})
            maps["b_E_glu"] = DimMap({"model": 0})
        return super().dim_maps() | maps

    # ---- norms -------------------------------------------------------------------------------
    def encoder_norm(self, keepdim: bool = False) -> torch.Tensor:
        return torch.norm(self.W_E, p=2, dim=0, keepdim=keepdim)

    def decoder_norm(self, keepdim: bool = False) -> torch.Tensor:
        return torch.norm(self.W_D, p=2, dim=1, keepdim=keepdim)

    def decoder_bias_norm(self) -> torch.Tensor:
        if not self.cfg.use_decoder_bias:
            raise ValueError("Decoder bias is not used")
        return torch.norm(self.b_D, p=2, dim=0, keepdim=True)

    @torch.no_grad()
    def set_decoder_to_fixed_norm(self, value: float, force_exact: bool):
        n = self.decoder_norm(keepdim=True)
        self.W_D.mul_(value / (n if force_exact else torch.clamp(n, min=value)))

    @torch.no_grad()
    def set_encoder_to_fixed_norm(self, value: float):
        self.W_E.mul_(value / self.encoder_norm(keepdim=True))

    @torch.no_grad()
    def transform_to_unit_decoder_norm(self):
        self.W_D.div_(self.decoder_norm(keepdim=True))

    @torch.no_grad()
    def standardize_parameters_of_dataset_norm(self):
        """Fold the dataset-wise input / output scales into b_E, b_D and W_D so that raw activations can be
        fed directly; switches ``norm_activation`` to ``"inference"``."""
        assert self.cfg.norm_activation == "dataset-wise"
        assert self.dataset_average_activation_norm is not None
        root = math.sqrt(self.cfg.d_model)
        f_in = root / self.dataset_average_activation_norm[self.cfg.hook_point_in]
        f_out = root / self.dataset_average_activation_norm[self.cfg.hook_point_out]
        self.b_E.div_(f_in)
        if self.cfg.use_decoder_bias:
            self.b_D.div_(f_out)
        self.W_D.mul_(f_in / f_out)
        if isinstance(self.activation_function, JumpReLU):
            # The pre-activations shrink by f_in (compared on their own) or, gated by the decoder norms (which grow by
            # f_in / f_out), by f_out: the thresholds follow, or other features would fire after folding. (The reference
            # leaves them as they are, models/sae.py:242-255 there; its cross-layer transcoder does move them.)
            shift = math.log(f_out if self.cfg.sparsity_include_decoder_norm else f_in)
            self.activation_function.log_jumprelu_threshold.data.sub_(shift)
        self.cfg.norm_activation = "inference"

    # ---- forward -----------------------------------------------------------------------------
    def encode(self, x: torch.Tensor, return_hidden_pre: bool = False, **kwargs):
        x = x.to(self.W_E.dtype)
        hidden_pre = x @ self.W_E + self.b_E
        if self.cfg.use_glu_encoder:
            hidden_pre = hidden_pre * torch.sigmoid(x @ self.W_E_glu + self.b_E_glu)
        hidden_pre = self.hook_hidden_pre(hidden_pre)
        if self.cfg.sparsity_include_decoder_norm:
            norm = self.decoder_norm()
            feature_acts = self.activation_function(hidden_pre * norm) / norm
        else:
            feature_acts = self.activation_function(hidden_pre)
        feature_acts = self.hook_feature_acts(feature_acts)
        return (feature_acts, hidden_pre) if return_hidden_pre else feature_acts

    def _use_sparse_kernels(self, feature_acts: torch.Tensor) -> bool:
        """``use_triton_kernel`` (the reference's name for "decode through the sparse kernels") applies on CUDA when
        the activations are sparse enough and nothing listens on the hook points."""
        if not (self.cfg.use_triton_kernel and feature_acts.is_cuda and self.cfg.d_model % 8 == 0 and self.cfg.d_model <= 8192):
            return False
        sparsity = 1.0 - float((feature_acts != 0).sum()) / feature_acts.numel()
        return sparsity >= self.cfg.sparsity_threshold_for_triton_spmm_kernel

    def decode(self, feature_acts: torch.Tensor, **kwargs) -> torch.Tensor:
        if self._use_sparse_kernels(feature_acts):
            from ..ops.sparse_autograd import sparse_decode

            partial = sparse_decode(feature_acts, self.W_D)
        else:
            partial = feature_acts @ self.W_D
        reconstructed = all_reduce_sum(partial, self.tp_group)
        if self.cfg.use_decoder_bias:
            reconstructed = reconstructed + self.b_D
        return self.hook_reconstructed(reconstructed)

    def decode_coo(self, feature_acts: torch.Tensor) -> torch.Tensor:
        """Decode a sparse COO ``[tokens, F]`` tensor in fp32 (used by attribution code)."""
        out = torch.sparse.mm(feature_acts.to(torch.float32), self.W_D.to(torch.float32))
        if self.cfg.use_decoder_bias:
            out = out + self.b_D
        return out.to(self.cfg.dtype)

    def prepare_input(self, batch: dict[str, torch.Tensor], **kwargs) -> tuple[torch.Tensor, dict[str, Any], dict[str, Any]]:
        return batch[self.cfg.hook_point_in], {}, {}

    def prepare_label(self, batch: dict[str, torch.Tensor], **kwargs) -> torch.Tensor:
        return batch[self.cfg.hook_point_out]

    # ---- initialisation ----------------------------------------------------------------------
    @torch.no_grad()
    def init_parameters(self, **kwargs):
        super().init_parameters(**kwargs)
        g = shard_generator(self.device_mesh, self.W_D.device)
        eb, db = kwargs["encoder_uniform_bound"], kwargs["decoder_uniform_bound"]
        self.W_E.t().uniform_(-eb, eb, generator=g)
        self.W_D.uniform_(-db, db, generator=g)
        self.b_E.zero_()
        if self.cfg.use_decoder_bias:
            self.b_D.zero_()
        if self.cfg.use_glu_encoder:
            self.W_E_glu.t().uniform_(-eb, eb, generator=g)
            self.b_E_glu.zero_()

    @torch.no_grad()
    def init_encoder_with_decoder_transpose(self, factor: float = 1.0):
        self.W_E.t().copy_(self.W_D * factor)

    def _shared_across_data(self, t: torch.Tensor) -> torch.Tensor:
        """Make a per-rank batch identical on every data-parallel rank (rank 0 of the data group wins)."""
        if self.dp_size > 1:
            t = t.contiguous().clone()
            dist.broadcast(t, group=self.dp_group, group_src=0)
        return t

    @torch.no_grad()
    def init_W_D_with_active_subspace(self, batch: dict[str, torch.Tensor], d_active_subspace: int):
        """Project the decoder onto the span of the top ``d_active_subspace`` principal directions of the labels."""
        label = self._shared_across_data(self.prepare_label(batch)).reshape(-1, self.cfg.d_model)
        centered = (label - label.mean(dim=0)).to(torch.float32)
        U, _, _ = torch.linalg.svd(centered.T, full_matrices=False)
        proj = U[:, :d_active_subspace].to(self.cfg.dtype)
        self.W_D.copy_(self.W_D[:, :d_active_subspace] @ proj.T)

    @torch.no_grad()
    def init_tc_with_mlp(self, batch: dict[str, torch.Tensor], mlp):
        """Transcoder initialisation: decoder rows = normalised, de-meaned MLP responses to the encoder
        directions placed at the data mean (models/sae.py:470-507 of the reference)."""
        assert self.cfg.norm_activation == "dataset-wise" and self.dataset_average_activation_norm is not None
        f_in = math.sqrt(self.cfg.d_model) / self.dataset_average_activation_norm[self.cfg.hook_point_in]
        x = self._shared_across_data(self.prepare_input(batch)[0]).reshape(-1, self.cfg.d_model) / f_in
        mean = x.mean(dim=0)
        radius = (x - mean).norm(dim=1).mean()
        dirs = self.W_E / self.W_E.norm(dim=0, keepdim=True)
        out = mlp.forward(mean + (dirs * radius).T)
        out = out - out.mean(dim=0)
        self.W_E.copy_(dirs)
        self.W_D.copy_(out / out.norm(dim=1, keepdim=True))

    @torch.no_grad()
    def init_encoder_bias_with_mean_hidden_pre(self, batch: dict[str, torch.Tensor]):
        x = self.prepare_input(batch)[0]
        _, hidden_pre = self.encode(x, return_hidden_pre=True)
        mean = hidden_pre.reshape(-1, hidden_pre.shape[-1]).mean(dim=0)
        if self.dp_size > 1:
            dist.all_reduce(mean, group=self.dp_group)
            mean /= self.dp_size
        self.b_E.sub_(mean)

    # ---- SAELens interchange -----------------------------------------------------------------
    @classmethod
    @torch.no_grad()
    def from_saelens(cls, sae_saelens, **kwargs):
        from sae_lens import JumpReLUSAE, StandardSAE, TopKSAE

        assert isinstance(sae_saelens, (JumpReLUSAE, StandardSAE, TopKSAE)), f"unsupported SAELens class {type(sae_saelens)}"
        c = sae_saelens.cfg
        assert c.reshape_activations == "none" and not c.apply_b_dec_to_input and c.normalize_activations == "none"
        act, k, gate, window = "relu", 0, False, 0.0
        if isinstance(sae_saelens, TopKSAE):
            act, k, gate = "topk", c.k, c.rescale_acts_by_decoder_norm
        elif isinstance(sae_saelens, JumpReLUSAE):
            act, window = "jumprelu", 2.0
        cfg = SAEConfig(
            hook_point_in=c.metadata.hook_name, hook_point_out=c.metadata.hook_name, dtype=sae_saelens.W_enc.dtype,
            d_model=c.d_in, act_fn=act, jumprelu_threshold_window=window, top_k=k, expansion_factor=c.d_sae / c.d_in,
            sparsity_include_decoder_norm=gate, **kwargs,
        )  # fmt: skip
        model = cls.from_config(cfg, None)
        model.W_D.copy_(sae_saelens.W_dec)
        model.W_E.copy_(sae_saelens.W_enc)
        model.b_D.copy_(sae_saelens.b_dec)
        model.b_E.copy_(sae_saelens.b_enc)
        if isinstance(sae_saelens, JumpReLUSAE):
            assert isinstance(model.activation_function, JumpReLU)
            model.activation_function.log_jumprelu_threshold.copy_(torch.log(sae_saelens.threshold.detach()))
        return model

    @torch.no_grad()
    def to_saelens(self, model_name: str = "unknown"):
        from sae_lens import JumpReLUSAE, JumpReLUSAEConfig, StandardSAE, StandardSAEConfig, TopKSAE, TopKSAEConfig
        from sae_lens.saes.sae import SAEMetadata

        assert self.cfg.hook_point_in == self.cfg.hook_point_out, "transcoders have no SAELens counterpart"
        assert self.device_mesh is None and not self.cfg.use_glu_encoder
        common = dict(d_in=self.cfg.d_model, d_sae=self.cfg.d_sae, dtype=str(self.cfg.dtype), device="cpu",
                      apply_b_dec_to_input=False, normalize_activations="none",
                      metadata=SAEMetadata(model_name=model_name, hook_name=self.cfg.hook_point_in))  # fmt: skip
        if self.cfg.act_fn == "relu":
            out = StandardSAE(StandardSAEConfig(**common))
        elif self.cfg.act_fn == "jumprelu":
            out = JumpReLUSAE(JumpReLUSAEConfig(**common))
        elif self.cfg.act_fn == "topk":
            out = TopKSAE(TopKSAEConfig(k=self.cfg.top_k, rescale_acts_by_decoder_norm=self.cfg.sparsity_include_decoder_norm, **common))
        else:
            raise TypeError(f"activation {self.cfg.act_fn} has no SAELens counterpart")
        out.W_dec.copy_(self.W_D)
        out.W_enc.copy_(self.W_E)
        out.b_dec.copy_(self.b_D)
        out.b_enc.copy_(self.b_E)
        if isinstance(out, JumpReLUSAE):
            out.threshold.copy_(self.activation_function.log_jumprelu_threshold.exp())
        return out
