"""Crosscoder: several "heads" (model snapshots, layers, ...) share one latent space.

Behaviour follows models/crosscoder.py of the reference project: parameters ``W_E [H, d, F]``, ``b_E [H, F]``,
``W_D [H, F, d]``, ``b_D [H, d]`` (:111-119); every head encodes its own activation, the pre-activations are
SUMMED over heads, and each head applies the activation function to the sum gated by ITS decoder norms
(:350-378); every head decodes with its own decoder (:384-469); all heads start from identical weights
(:160-219); folding the dataset norm only rescales the biases (:519-538); per-head training metrics (:637-675);
decoder inner-product / similarity matrices (:696-710).

Parallel layout: heads are split over the ``head`` mesh dimension, features over ``model``. The sum over heads is
a local sum followed by one all-reduce over the head group whose backward is also an all-reduce (each rank uses
the shared sum for its own heads). Each head rank receives only its own hook points in the batch.
"""

from __future__ import annotations

import math
from typing import Any

import torch
import torch.distributed as dist
from torch import nn

from ..parallel.collectives import all_reduce_sum, all_reduce_sum_both
from ..parallel.mesh import DeviceMesh, DimMap, mesh_dim_size, mesh_group
from ..utils.tensor_specs import TensorSpecs
from .sae import shard_generator
from .sparse_dictionary import SparseDictionary, SparseDictionaryConfig, register_sae_config, register_sae_model


class CrosscoderSpecs(TensorSpecs):
    @staticmethod
    def feature_acts(tensor: torch.Tensor) -> tuple[str, ...]:
        return {3: ("batch", "heads", "sae"), 4: ("batch", "context", "heads", "sae")}[tensor.ndim]

    @staticmethod
    def reconstructed(tensor: torch.Tensor) -> tuple[str, ...]:
        return {3: ("batch", "heads", "model"), 4: ("batch", "context", "heads", "model")}[tensor.ndim]

    @staticmethod
    def label(tensor: torch.Tensor) -> tuple[str, ...]:
        return CrosscoderSpecs.reconstructed(tensor)


@register_sae_config("crosscoder")
class CrosscoderConfig(SparseDictionaryConfig):
    sae_type: str = "crosscoder"
    hook_points: list[str]
    fused_head_sum: bool | None = None
    """Sum the encoder pre-activations over heads with the native kernels (local heads in the K loop of one tcgen05 GEMM
    that stores into a symmetric buffer, other ranks of the ``head`` group by the one-kernel in-place all-reduce).
    None: on for bf16 models under head parallelism on CUDA; True also uses the GEMM without a ``head`` group."""

    @property
    def associated_hook_points(self) -> list[str]:
        return self.hook_points

    @property
    def hooks_in(self) -> list[str]:
        return self.hook_points

    @property
    def hooks_out(self) -> list[str]:
        return self.hook_points

    @property
    def n_heads(self) -> int:
        return len(self.hook_points)


class _HeadSumEncode(torch.autograd.Function):
    """``sum over all heads of (x_h W_E[h] + b_E[h])`` through ``HeadSumComm`` (bf16 operands and partial sums, fp32
    accumulation). The value is used by every rank's own heads, so the incoming gradient is summed over the group first
    (as in ``all_reduce_sum_both``); the weight and input gradients are plain batched products."""

    @staticmethod
    def forward(ctx, x, W_E, b_E, comm, group):
        B, H, d = x.shape
        F = W_E.shape[-1]
        x16 = x.detach().to(torch.bfloat16).reshape(B, H * d).contiguous()
        w16 = W_E.detach().transpose(1, 2).to(torch.bfloat16).contiguous().view(H * F, d)  # feature-major blocks
        out = comm.head_sum(x16, w16, b_E.detach().float().sum(dim=0).contiguous(), H, F, torch.float32)
        ctx.save_for_backward(x16, w16)
        ctx.group, ctx.shape, ctx.dtypes = group, (B, H, d, F), (x.dtype, W_E.dtype, b_E.dtype)
        return out

    @staticmethod
    def backward(ctx, grad):
        x16, w16 = ctx.saved_tensors
        B, H, d, F = ctx.shape
        g = grad.contiguous().float()
        if ctx.group is not None and dist.get_world_size(ctx.group) > 1:
            g = g.clone()
            dist.all_reduce(g, group=ctx.group)
        g16 = g.to(torch.bfloat16)
        dx = dW = db = None
        if ctx.needs_input_grad[0]:
            dx = torch.einsum("bf,hfd->bhd", g16, w16.view(H, F, d)).to(ctx.dtypes[0])
        if ctx.needs_input_grad[1]:
            dW = torch.einsum("bhd,bf->hdf", x16.view(B, H, d), g16).to(ctx.dtypes[1])
        if ctx.needs_input_grad[2]:
            db = g.sum(dim=0).to(ctx.dtypes[2]).unsqueeze(0).expand(H, F)
        return dx, dW, db, None, None


@register_sae_model("crosscoder")
class Crosscoder(SparseDictionary):
    specs: type[TensorSpecs] = CrosscoderSpecs

    def __init__(self, cfg: CrosscoderConfig, device_mesh: DeviceMesh | None = None):
        super().__init__(cfg, device_mesh)
        self.cfg: CrosscoderConfig = cfg
        assert cfg.sparsity_include_decoder_norm, "Sparsity should include decoder norm in Crosscoder"
        assert cfg.use_decoder_bias, "Decoder bias should be used in Crosscoder"
        H, d, F = cfg.n_heads, cfg.d_model, cfg.d_sae
        H_l, F_l = DimMap({"head": 0, "model": 1}).local_shape((H, F), device_mesh)
        self.n_heads_local, self.d_sae_local = H_l, F_l
        dev, dt = cfg.device, cfg.dtype
        # feature-major storage for both weight tensors (see models/sae.py)
        self.W_E = nn.Parameter(torch.empty(H_l, F_l, d, device=dev, dtype=dt).transpose(1, 2))
        self.b_E = nn.Parameter(torch.empty(H_l, F_l, device=dev, dtype=dt))
        self.W_D = nn.Parameter(torch.empty(H_l, F_l, d, device=dev, dtype=dt))
        self.b_D = nn.Parameter(torch.empty(H_l, d, device=dev, dtype=dt))
        self._head_sum_comm = None
        self.setup()

    @property
    def head_group(self):
        return mesh_group(self.device_mesh, "head")

    @property
    def head_size(self) -> int:
        return mesh_dim_size(self.device_mesh, "head")

    def local_hook_points(self) -> list[str]:
        sl = DimMap({"head": 0}).local_slices((self.cfg.n_heads,), self.device_mesh)[0]
        return self.cfg.hook_points[sl]

    def dim_maps(self) -> dict[str, DimMap]:
        return super().dim_maps() | {
            "W_E": DimMap({"head": 0, "model": 2}),
            "W_D": DimMap({"head": 0, "model": 1}),
            "b_E": DimMap({"head": 0, "model": 1}),
            "b_D": DimMap({"head": 0}),
        }

    @torch.no_grad()
    def init_parameters(self, **kwargs) -> None:
        """Every head starts from the same random encoder / decoder."""
        super().init_parameters(**kwargs)
        g = shard_generator(self.device_mesh, self.W_D.device)
        # heads must agree: the generator seed must not depend on the head coordinate
        if self.head_size > 1:
            seed = torch.tensor([g.initial_seed()], dtype=torch.int64, device=self.W_D.device)
            dist.broadcast(seed, group=self.head_group, group_src=0)
            g.manual_seed(int(seed))
        eb, db = kwargs["encoder_uniform_bound"], kwargs["decoder_uniform_bound"]
        we = torch.empty(self.d_sae_local, self.cfg.d_model, device=self.W_D.device, dtype=self.cfg.dtype).uniform_(-eb, eb, generator=g)
        wd = torch.empty_like(we).uniform_(-db, db, generator=g)
        self.W_E.transpose(1, 2).copy_(we.unsqueeze(0).expand(self.n_heads_local, -1, -1))
        self.W_D.copy_(wd.unsqueeze(0).expand(self.n_heads_local, -1, -1))
        self.b_E.zero_()
        self.b_D.zero_()

    # ---- norms -------------------------------------------------------------------------------
    def decoder_norm(self, keepdim: bool = False) -> torch.Tensor:
        return torch.norm(self.W_D, dim=-1, keepdim=keepdim)

    def encoder_norm(self, keepdim: bool = False) -> torch.Tensor:
        return torch.norm(self.W_E, dim=-2, keepdim=keepdim)

    def decoder_bias_norm(self) -> torch.Tensor:
        return torch.norm(self.b_D, dim=-1, keepdim=True)

    @torch.no_grad()
    def set_decoder_to_fixed_norm(self, value: float, force_exact: bool):
        n = self.decoder_norm(keepdim=True)
        self.W_D.mul_(value / (n if force_exact else torch.clamp(n, min=value)))

    @torch.no_grad()
    def set_encoder_to_fixed_norm(self, value: float):
        self.W_E.mul_(value / self.encoder_norm(keepdim=True))

    @torch.no_grad()
    def transform_to_unit_decoder_norm(self):
        raise NotImplementedError("Transform to unit decoder norm is not supported for Crosscoder")

    @torch.no_grad()
    def standardize_parameters_of_dataset_norm(self):
        assert self.cfg.norm_activation == "dataset-wise" and self.dataset_average_activation_norm is not None
        f = torch.tensor(
            [math.sqrt(self.cfg.d_model) / self.dataset_average_activation_norm[hp] for hp in self.local_hook_points()],
            dtype=self.cfg.dtype, device=self.b_E.device,
        ).view(-1, 1)  # fmt: skip
        self.b_E.div_(f)
        self.b_D.div_(f)
        self.cfg.norm_activation = "inference"

    @torch.no_grad()
    def init_encoder_with_decoder_transpose(self, factor: float = 1.0):
        self.W_E.transpose(1, 2).copy_(self.W_D * factor)

    # ---- forward -----------------------------------------------------------------------------
    def _per_head_pre(self, x: torch.Tensor) -> torch.Tensor:
        """[..., H_l, d] -> [..., H_l, F_l]"""
        return torch.einsum("...hd,hdf->...hf", x.to(self.W_E.dtype), self.W_E) + self.b_E

    def _fused_head_sum_ok(self, x: torch.Tensor) -> bool:
        want = self.cfg.fused_head_sum
        if want is None:
            want = self.cfg.dtype == torch.bfloat16 and self.head_size > 1
        return bool(
            want and x.is_cuda and x.ndim >= 2 and self.cfg.d_model % 64 == 0
            and self.d_sae_local % 8 == 0
        )  # fmt: skip

    def _summed_pre(self, x: torch.Tensor) -> torch.Tensor:
        """Pre-activations summed over ALL heads (local heads and the other ranks of the ``head`` group)."""
        if self._fused_head_sum_ok(x):
            # one tcgen05 GEMM over K = local heads x d_model into a symmetric buffer, summed over the head ranks in place
            from ..parallel.symm import HeadSumComm

            rows = x[..., 0, 0].numel()
            if self._head_sum_comm is None or self._head_sum_comm.max_rows < rows:
                self._head_sum_comm = HeadSumComm(self.head_group, x.device, rows, self.d_sae_local)
            lead = x.shape[:-2]
            out = _HeadSumEncode.apply(x.reshape(rows, *x.shape[-2:]), self.W_E, self.b_E, self._head_sum_comm, self.head_group)
            return out.reshape(*lead, self.d_sae_local).to(self.cfg.dtype)
        summed = self._per_head_pre(x).sum(dim=-2)
        return all_reduce_sum_both(summed, self.head_group)

    def encode(self, x: torch.Tensor, return_hidden_pre: bool = False, **kwargs):
        summed = self._summed_pre(x)
        hidden_pre = summed.unsqueeze(-2).expand(*summed.shape[:-1], self.n_heads_local, summed.shape[-1])
        norm = self.decoder_norm()
        feature_acts = self.activation_function(hidden_pre * norm) / norm
        return (feature_acts, hidden_pre) if return_hidden_pre else feature_acts

    def decode(self, feature_acts: torch.Tensor, **kwargs) -> torch.Tensor:
        rec = torch.einsum("...hf,hfd->...hd", feature_acts, self.W_D)
        return all_reduce_sum(rec, self.tp_group) + self.b_D

    def _decode_linear(self, feature_acts: torch.Tensor) -> torch.Tensor:
        return torch.einsum("...hf,hfd->...hd", feature_acts, self.W_D)

    def prepare_input(self, batch: dict[str, torch.Tensor], **kwargs) -> tuple[torch.Tensor, dict[str, Any], dict[str, Any]]:
        """Stack this rank's hook points to ``[..., H_l, d_model]`` (narrower activations are zero-padded)."""

        def pad(x: torch.Tensor) -> torch.Tensor:
            if x.shape[-1] > self.cfg.d_model:
                raise ValueError(f"Input tensor has {x.shape[-1]} dimensions, but expected {self.cfg.d_model}.")
            if x.shape[-1] < self.cfg.d_model:
                return torch.nn.functional.pad(x, (0, self.cfg.d_model - x.shape[-1]))
            return x

        return torch.stack([pad(batch[hp]) for hp in self.local_hook_points()], dim=-2), {}, {}

    def prepare_label(self, batch: dict[str, torch.Tensor], **kwargs) -> torch.Tensor:
        return self.prepare_input(batch)[0]

    def compute_loss(self, batch, *args, return_aux_data: bool = True, **kwargs):
        """Base loss over this rank's heads; under head parallelism the returned value is the mean over ALL
        heads while its gradient is that of this rank's share (so that summed gradients match one process)."""
        out = super().compute_loss(batch, *args, return_aux_data=True, **kwargs)
        if self.head_size > 1:
            out["loss"] = all_reduce_sum(out["loss"] / self.head_size, self.head_group)
        return out if return_aux_data else out["loss"]

    # ---- analysis helpers --------------------------------------------------------------------
    @torch.no_grad()
    def compute_training_metrics(self, *, feature_acts, l_rec, l0, explained_variance, **kwargs) -> dict[str, float]:
        hooks = self.local_hook_points()
        out: dict[str, float] = {}
        ev = explained_variance.reshape(-1, len(hooks)).mean(0) if explained_variance.numel() >= len(hooks) else None
        acts = feature_acts.reshape(-1, *feature_acts.shape[-2:])
        l0_h = (acts > 0).float().sum(-1).mean(0)
        rec = kwargs.get("reconstructed")
        lab = kwargs.get("label")
        for i, hp in enumerate(hooks):
            if ev is not None:
                out[f"crosscoder_metrics/{hp}/explained_variance"] = float(ev[i])
            out[f"crosscoder_metrics/{hp}/l0"] = float(l0_h[i])
            if rec is not None and lab is not None:
                err = (rec.float() - lab.float()).pow(2).sum(-1).reshape(-1, len(hooks)).mean(0)
                out[f"crosscoder_metrics/{hp}/l_rec"] = float(err[i])
        fired = acts.amax(dim=1) > 0  # [tokens, F_l]
        norms = self.decoder_norm()  # [H_l, F_l]
        tok, feat = fired.nonzero(as_tuple=True)
        if tok.numel() > 0:
            a = acts[tok, :, feat]  # [n, H_l]
            n = norms[:, feat].T
            if (a == 0).any():
                out["crosscoder_metrics/mean_decoder_norm_non_activated_in_activated"] = float(n[a == 0].mean())
            out["crosscoder_metrics/mean_decoder_norm_activated_in_activated"] = float(n[a != 0].mean())
        return out

    @torch.no_grad()
    def decoder_inner_product_matrices(self) -> torch.Tensor:
        """``[F_l, H, H]`` inner products between the heads' decoder rows of each feature (local heads only)."""
        return torch.einsum("ifd,jfd->fij", self.W_D, self.W_D)

    @torch.no_grad()
    def decoder_similarity_matrices(self) -> torch.Tensor:
        n = self.decoder_norm()
        return self.decoder_inner_product_matrices() / torch.einsum("if,jf->fij", n, n)
