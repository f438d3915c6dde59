"""Mixture of linear transforms (MOLT): a sparse set of low-rank linear maps standing in for an MLP.

Behaviour follows models/molt.py of the reference project: config with ``rank_counts`` and
``d_sae = sum(counts)`` (:36-127); parameters ``W_E [d, F]``, ``b_E [F]``, ``U_matrices.<rank> [count, d, rank]``,
``V_matrices.<rank> [count, rank, d]``, ``b_D [d]`` (:181-202); SAE-style encoder with gating by the decoder
norm ``||U_i V_i||_F`` (:501-541); decoder ``sum_i f_i U_i V_i x`` evaluated as ``U (f * (V x))`` per rank
group (:543-589) and summed over feature shards (:591-673); norm utilities (:309-468); init (:716-778);
per-rank-group metrics (:804-831).

Sharding: every rank group is divided evenly over the ``model`` dimension, and the encoder's feature axis is
laid out in the same (rank group, local index) order on each rank, so encoder outputs feed the local decoder
shards directly. The Frobenius norm of ``U V`` is computed from the rank x rank Gram matrices
(``||UV||_F^2 = <U^T U, V V^T>``) instead of materialising ``count`` d x d products.
"""

from __future__ import annotations

import math
from typing import Any

import torch
from torch import nn

from ..hooks import HookPoint
from ..parallel.collectives import all_reduce_sum
from ..parallel.mesh import DeviceMesh, DimMap
from .sae import _feature_major_param, shard_generator
from .sparse_dictionary import SparseDictionary, SparseDictionaryConfig, register_sae_config, register_sae_model


@register_sae_config("molt")
class MOLTConfig(SparseDictionaryConfig):
    sae_type: str = "molt"
    hook_point_in: str
    hook_point_out: str
    rank_counts: dict[int, int]
    """rank -> number of transforms of that rank, e.g. {4: 128, 8: 256, 16: 128}."""

    def model_post_init(self, __context):
        super().model_post_init(__context)
        assert self.rank_counts, "rank_counts cannot be empty"
        for rank, count in self.rank_counts.items():
            assert rank > 0, f"Rank must be positive, got {rank}"
            assert count > 0, f"Count for rank {rank} must be positive, got {count}"
        assert abs(self.expansion_factor - self.d_sae / self.d_model) < 0.1, (
            f"Expansion factor {self.expansion_factor} is not close to d_sae / d_model {self.d_sae / self.d_model}"
        )

    def generate_rank_assignments(self) -> list[int]:
        return [r for r in sorted(self.rank_counts) for _ in range(self.rank_counts[r])]

    def get_local_rank_assignments(self, model_parallel_size: int) -> list[int]:
        out: list[int] = []
        for r in sorted(self.rank_counts):
            n = self.rank_counts[r]
            assert n % model_parallel_size == 0, f"rank {r}: {n} transforms not divisible by {model_parallel_size} shards"
            out.extend([r] * (n // model_parallel_size))
        return out

    @property
    def d_sae(self) -> int:  # type: ignore[override]
        return sum(self.rank_counts.values())

    @property
    def available_ranks(self) -> list[int]:
        return sorted(self.rank_counts)

    @property
    def num_rank_types(self) -> int:
        return len(self.rank_counts)

    @property
    def associated_hook_points(self) -> list[str]:
        return [self.hook_point_in, self.hook_point_out]

    @property
    def hooks_in(self) -> list[str]:
        return [self.hook_point_in]

    @property
    def hooks_out(self) -> list[str]:
        return [self.hook_point_out]


@register_sae_model("molt")
class MixtureOfLinearTransform(SparseDictionary):
    def __init__(self, cfg: MOLTConfig, device_mesh: DeviceMesh | None = None) -> None:
        super().__init__(cfg, device_mesh=device_mesh)
        self.cfg: MOLTConfig = cfg
        self.rank_assignments = cfg.get_local_rank_assignments(self.tp_size)
        F_l = len(self.rank_assignments)
        self.d_sae_local = F_l
        dev, dt, d = cfg.device, cfg.dtype, cfg.d_model
        self.W_E = _feature_major_param(d, F_l, dev, dt)
        self.b_E = nn.Parameter(torch.empty(F_l, device=dev, dtype=dt))
        self.U_matrices = nn.ParameterDict()
        self.V_matrices = nn.ParameterDict()
        for r in cfg.available_ranks:
            n = self.rank_assignments.count(r)
            self.U_matrices[str(r)] = nn.Parameter(torch.empty(n, d, r, device=dev, dtype=dt))
            self.V_matrices[str(r)] = nn.Parameter(torch.empty(n, r, d, device=dev, dtype=dt))
        if cfg.use_decoder_bias:
            self.b_D = nn.Parameter(torch.empty(d, device=dev, dtype=dt))
        self.hook_hidden_pre = HookPoint()
        self.hook_feature_acts = HookPoint()
        self.hook_reconstructed = HookPoint()
        self.setup()

    def dim_maps(self) -> dict[str, DimMap]:
        maps = {"b_D": DimMap({}), "U_matrices": DimMap({"model": 0}), "V_matrices": DimMap({"model": 0})}
        for r in self.cfg.available_ranks:
            maps[f"U_matrices.{r}"] = DimMap({"model": 0})
            maps[f"V_matrices.{r}"] = DimMap({"model": 0})
        # The encoder's feature axis is ordered (rank group, shard, index-in-shard) when gathered; see
        # full_state_dict / load_full_state_dict below, which re-order to the logical (rank group, index) order.
        maps["W_E"] = DimMap({"model": 1})
        maps["b_E"] = DimMap({"model": 0})
        return super().dim_maps() | maps

    def _logical_permutation(self) -> torch.Tensor | None:
        """Index such that ``gathered[..., perm]`` is in logical (rank group, global index) order."""
        tp = self.tp_size
        if tp == 1:
            return None
        local_counts = [self.rank_assignments.count(r) for r in self.cfg.available_ranks]
        F_l = sum(local_counts)
        perm = []
        off = 0
        for c in local_counts:
            for shard in range(tp):
                perm.extend(range(shard * F_l + off, shard * F_l + off + c))
            off += c
        return torch.tensor(perm)

    @torch.no_grad()
    def full_state_dict(self) -> dict[str, torch.Tensor]:
        sd = super().full_state_dict()
        perm = self._logical_permutation()
        if perm is not None:
            sd["W_E"] = sd["W_E"][:, perm.to(sd["W_E"].device)].contiguous()
            sd["b_E"] = sd["b_E"][perm.to(sd["b_E"].device)].contiguous()
        return sd

    def load_full_state_dict(self, state_dict: dict[str, torch.Tensor], strict: bool = True) -> None:
        perm = self._logical_permutation()
        if perm is not None and "W_E" in state_dict and state_dict["W_E"].shape[1] == self.cfg.d_sae:
            inv = torch.empty_like(perm)
            inv[perm] = torch.arange(perm.numel())
            state_dict = dict(state_dict)
            state_dict["W_E"] = state_dict["W_E"][:, inv.to(state_dict["W_E"].device)]
            state_dict["b_E"] = state_dict["b_E"][inv.to(state_dict["b_E"].device)]
        super().load_full_state_dict(state_dict, strict=strict)

    # ---- norms -------------------------------------------------------------------------------
    def encoder_norm(self, keepdim: bool = False) -> torch.Tensor:
        return torch.norm(self.W_E, p=2, dim=0, keepdim=keepdim)

    def _uv_norms(self, rank: int) -> torch.Tensor:
        U, V = self.U_matrices[str(rank)], self.V_matrices[str(rank)]
        gram = torch.einsum("cdr,cds->crs", U, U) * torch.einsum("crd,csd->crs", V, V)
        return gram.sum(dim=(1, 2)).clamp_min(0).sqrt()

    def decoder_norm(self, keepdim: bool = False) -> torch.Tensor:
        """``||U_i V_i||_F`` per local transform, in local feature order."""
        n = torch.cat([self._uv_norms(r) for r in self.cfg.available_ranks])
        return n.unsqueeze(-1) if keepdim else n

    def decoder_bias_norm(self) -> torch.Tensor:
        assert self.cfg.use_decoder_bias, "Decoder bias is not used"
        return torch.norm(self.b_D, p=2, dim=0, keepdim=True)

    @torch.no_grad()
    def set_decoder_to_fixed_norm(self, value: float, force_exact: bool) -> None:
        for r in self.cfg.available_ranks:
            cur = self._uv_norms(r)
            s = (value / cur) ** 0.5
            if not force_exact:
                s = torch.where(cur >= value, s, torch.ones_like(s))
            self.U_matrices[str(r)].data.mul_(s.view(-1, 1, 1))
            self.V_matrices[str(r)].data.mul_(s.view(-1, 1, 1))

    @torch.no_grad()
    def set_encoder_to_fixed_norm(self, value: float) -> None:
        self.W_E.mul_(value / self.encoder_norm(keepdim=True))

    @torch.no_grad()
    def transform_to_unit_decoder_norm(self) -> None:
        self.set_decoder_to_fixed_norm(1.0, force_exact=True)

    @torch.no_grad()
    def standardize_parameters_of_dataset_norm(self) -> None:
        assert self.cfg.norm_activation == "dataset-wise" and self.dataset_average_activation_norm is not None
        root = math.sqrt(self.cfg.d_model)
        f_in = root / self.dataset_average_activation_norm[self.cfg.hook_point_in]
        f_out = root / self.dataset_average_activation_norm[self.cfg.hook_point_out]
        self.b_E.div_(f_in)
        if self.cfg.use_decoder_bias:
            self.b_D.div_(f_out)
        # The gate shrinks to a / f_in (the bias is divided, the encoder kept) and the transforms now see raw inputs
        # x = x_n / f_in: keeping sum_c a_c U_c V_c x_n / f_out needs U V scaled by f_in^2 / f_out. (The reference scales by
        # f_in / f_out, as for a dictionary whose decoder does not read the input, which changes the folded model's
        # output by the factor 1 / f_in: models/molt.py:446-468 there.)
        s = (f_in * f_in / f_out) ** 0.5
        for r in self.cfg.available_ranks:
            self.U_matrices[str(r)].data.mul_(s)
            self.V_matrices[str(r)].data.mul_(s)
        self.cfg.norm_activation = "inference"

    # ---- forward -----------------------------------------------------------------------------
    def encode(self, x: torch.Tensor, return_hidden_pre: bool = False, **kwargs):
        hidden_pre = self.hook_hidden_pre(x.to(self.W_E.dtype) @ self.W_E + self.b_E)
        if self.cfg.sparsity_include_decoder_norm:
            n = self.decoder_norm()
            feature_acts = self.activation_function(hidden_pre * n) / n
        else:
            feature_acts = self.activation_function(hidden_pre)
        feature_acts = self.hook_feature_acts(feature_acts)
        return (feature_acts, hidden_pre) if return_hidden_pre else feature_acts

    def _decode_local(self, feature_acts: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        out = torch.zeros_like(x, dtype=feature_acts.dtype)
        off = 0
        for r in self.cfg.available_ranks:
            U, V = self.U_matrices[str(r)], self.V_matrices[str(r)]
            n = U.shape[0]
            f = feature_acts[..., off : off + n]
            off += n
            if self.cfg.use_triton_kernel and n > 0:
                # only the active (token, transform) pairs: gather kernels instead of two dense products over all transforms
                from ..ops.molt_sparse import molt_group_decode

                out = out + molt_group_decode(f, x, U, V).to(out.dtype)
                continue
            Vx = torch.einsum("...d,crd->...cr", x.to(V.dtype), V)
            out = out + torch.einsum("...cr,cdr->...d", f.unsqueeze(-1) * Vx, U)
        return out

    def decode(self, feature_acts: torch.Tensor, **kwargs) -> torch.Tensor:
        assert "original_x" in kwargs, "MOLT decode requires 'original_x' in kwargs"
        out = all_reduce_sum(self._decode_local(feature_acts, kwargs["original_x"]), self.tp_group)
        if self.cfg.use_decoder_bias:
            out = out + self.b_D
        return self.hook_reconstructed(out)

    def forward(self, x: torch.Tensor, encoder_kwargs: dict[str, Any] = {}, decoder_kwargs: dict[str, Any] = {}):
        return self.decode(self.encode(x, **encoder_kwargs), original_x=x)

    @torch.no_grad()
    def init_parameters(self, **kwargs) -> None:
        super().init_parameters(**kwargs)
        g = shard_generator(self.device_mesh, self.b_E.device)
        b = 1.0 / math.sqrt(self.cfg.d_sae)
        self.W_E.t().uniform_(-b, b, generator=g)
        self.b_E.zero_()
        for r in self.cfg.available_ranks:
            self.U_matrices[str(r)].uniform_(-b, b, generator=g)
            self.V_matrices[str(r)].uniform_(-b, b, generator=g)
        if self.cfg.use_decoder_bias:
            self.b_D.zero_()

    def prepare_input(self, batch: dict[str, torch.Tensor], **kwargs) -> tuple[torch.Tensor, dict[str, Any], dict[str, Any]]:
        x = batch[self.cfg.hook_point_in]
        return x, {}, {"original_x": x}

    def prepare_label(self, batch: dict[str, torch.Tensor], **kwargs) -> torch.Tensor:
        return batch[self.cfg.hook_point_out]

    @torch.no_grad()
    def compute_training_metrics(self, *, l0: torch.Tensor, feature_acts: torch.Tensor, **kwargs) -> dict[str, float]:
        """L0 per rank group (summed over feature shards) and the activation-weighted total rank."""
        out: dict[str, float] = {}
        off, total = 0, 0.0
        for r in self.cfg.available_ranks:
            n = self.rank_assignments.count(r)
            cnt = (feature_acts[..., off : off + n] > 0).float().sum(-1).mean()
            off += n
            mean = self._sum_over_features(cnt.reshape(1)).item() if self.tp_size > 1 else float(cnt)
            out[f"molt_metrics/l0_rank{r}"] = mean
            out[f"molt_metrics/l0_rank{r}_ratio"] = mean / self.cfg.rank_counts[r]
            total += mean * r
        out["molt_metrics/total_rank_sum"] = total
        return out
