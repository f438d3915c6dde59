"""Low-rank sparse attention (Lorsa): an attention layer rewritten as many rank-1 OV heads that share a small
number of QK heads, with a sparse activation over the OV heads.

Behaviour follows models/lorsa.py of the reference project: config (:49-105), parameters ``W_Q, W_K [nqk, d,
dqk]``, ``b_Q, b_K [nqk, dqk]``, ``W_V, W_O [F, d]``, ``b_V [F]``, ``b_D [d]`` and persistent buffers ``mask``,
``IGNORE``, ``rotary_sin``, ``rotary_cos`` (:108-240); initialisation (:259-278) and initialisation from a
model's attention (:280-347) or its per-head active subspaces (:349-503); rotary embeddings incl. NTK-by-parts
(:525-575, :864-904); per-head RMS QK-norm (:1017-1062); fast path = fused causal attention with grouped heads,
slow path materialising scores / patterns for the hooks (:682-762, :906-943); z-pattern extraction (:831-862);
QK-head expansion on load (:960-980).

Each QK head serves ``ov_group_size = d_sae / n_qk_heads`` consecutive OV heads: the value "head dimension" of
the attention is that group, one scalar per OV head. Under ``model`` parallelism QK heads and their OV groups
are sharded together.
"""

from __future__ import annotations

import math
from typing import Any, Literal

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

from ..hooks import HookPoint
from ..ops import attention as attention_kernels
from ..parallel.collectives import all_reduce_sum
from ..parallel.mesh import DeviceMesh, DimMap, mesh_local_rank
from .sae import shard_generator
from .sparse_dictionary import SparseDictionary, SparseDictionaryConfig, register_sae_config, register_sae_model


@register_sae_config("lorsa")
class LorsaConfig(SparseDictionaryConfig):
    sae_type: str = "lorsa"
    hook_point_in: str
    hook_point_out: str
    n_qk_heads: int
    d_qk_head: int
    positional_embedding_type: Literal["rotary", "none"] = "rotary"
    rotary_dim: int
    rotary_base: int = 10000
    rotary_adjacent_pairs: bool = True
    rotary_scale: int = 1
    use_NTK_by_parts_rope: bool = False
    NTK_by_parts_factor: float = 1.0
    NTK_by_parts_low_freq_factor: float = 1.0
    NTK_by_parts_high_freq_factor: float = 1.0
    old_context_len: int = 2048
    n_ctx: int
    attn_scale: float | None = None
    attention_kernel: Literal["library", "tensor_core"] = "library"
    """``tensor_core``: this package's tcgen05 kernels (``ops/csrc/attention.cu``: forward, dQ, dK/dV; bf16 models, d_qk 64
    or 128, OV group a multiple of 64). ``library``: ``scaled_dot_product_attention`` restricted to its memory-efficient
    backend (``ops.attention.library_attention_backends`` says why the cuDNN backend is kept out)."""
    use_post_qk_ln: bool = False
    normalization_type: Literal["LN", "RMS"] | None = None
    eps: float = 1e-6

    @property
    def n_ov_heads(self) -> int:
        return self.d_sae

    @property
    def ov_group_size(self) -> int:
        return self.n_ov_heads // self.n_qk_heads

    @property
    def associated_hook_points(self) -> list[str]:
        return [self.hook_point_in, self.hook_point_out]

    @property
    def hooks_in(self) -> list[str]:
        return [self.hook_point_in]

    @property
    def hooks_out(self) -> list[str]:
        return [self.hook_point_out]

    def model_post_init(self, __context):
        super().model_post_init(__context)
        assert self.hook_point_in != self.hook_point_out, "hook_point_in and hook_point_out must be different"
        assert self.n_ov_heads % self.n_qk_heads == 0, "n_ov_heads must be divisible by n_qk_heads"
        if self.attn_scale is None:
            self.attn_scale = self.d_qk_head**0.5


class RMSNormPerHead(nn.Module):
    """RMS normalisation over the head dimension with a learned scale per (QK head, channel)."""

    def __init__(self, cfg: LorsaConfig, n_heads: int, device_mesh: DeviceMesh | None = None):
        super().__init__()
        self.cfg = cfg
        self.eps = cfg.eps
        (n_local,) = DimMap({"model": 0}).local_shape((n_heads,), device_mesh)
        self.w = nn.Parameter(torch.ones(n_local, cfg.d_qk_head, dtype=cfg.dtype, device=cfg.device))
        self.hook_scale = HookPoint()
        self.hook_normalized = HookPoint()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float() if x.dtype not in (torch.float32, torch.float64) else x
        scale = self.hook_scale((xf.pow(2).mean(-1, keepdim=True) + self.eps).sqrt())
        return self.hook_normalized((xf / scale * self.w).to(x.dtype))

    def dim_maps(self) -> dict[str, DimMap]:
        return {"w": DimMap({"model": 0})}


@register_sae_model("lorsa")
class LowRankSparseAttention(SparseDictionary):
    def __init__(self, cfg: LorsaConfig, device_mesh: DeviceMesh | None = None):
        super().__init__(cfg, device_mesh=device_mesh)
        self.cfg: LorsaConfig = cfg
        dev, dt = cfg.device, cfg.dtype
        (nqk_l,) = DimMap({"model": 0}).local_shape((cfg.n_qk_heads,), device_mesh)
        (F_l,) = DimMap({"model": 0}).local_shape((cfg.d_sae,), device_mesh)
        self.n_qk_heads_local, self.d_sae_local = nqk_l, F_l
        p = lambda *shape: nn.Parameter(torch.empty(*shape, dtype=dt, device=dev))  # noqa: E731
        self.W_Q = p(nqk_l, cfg.d_model, cfg.d_qk_head)
        self.W_K = p(nqk_l, cfg.d_model, cfg.d_qk_head)
        self.W_V = p(F_l, cfg.d_model)
        self.W_O = p(F_l, cfg.d_model)
        self.b_Q = p(nqk_l, cfg.d_qk_head)
        self.b_K = p(nqk_l, cfg.d_qk_head)
        self.b_V = p(F_l)
        if cfg.use_decoder_bias:
            self.b_D = p(cfg.d_model)
        self.register_buffer("mask", torch.tril(torch.ones(cfg.n_ctx, cfg.n_ctx, device=dev, dtype=torch.bool)))
        self.register_buffer("IGNORE", torch.tensor(-torch.inf, device=dev))
        if cfg.use_post_qk_ln:
            if cfg.normalization_type != "RMS":
                raise ValueError(f"Invalid normalization type for QK-norm: {cfg.normalization_type}")
            self.ln_q = RMSNormPerHead(cfg, cfg.n_qk_heads, device_mesh)
            self.ln_k = RMSNormPerHead(cfg, cfg.n_qk_heads, device_mesh)
        if cfg.positional_embedding_type == "rotary":
            sin, cos = self._calculate_sin_cos_rotary(cfg.rotary_dim, cfg.n_ctx, base=cfg.rotary_base, dtype=dt, device=dev)
            self.register_buffer("rotary_sin", sin)
            self.register_buffer("rotary_cos", cos)
        for name in ("hidden_pre", "feature_acts", "reconstructed", "attn_pattern", "attn_score", "q", "k", "q_post_rot", "k_post_rot"):
            setattr(self, f"hook_{name}", HookPoint())
        self.setup()

    # ---- aliases used by generic code ---------------------------------------------------------
    @property
    def W_D(self) -> torch.Tensor:
        return self.W_O

    @property
    def W_E(self) -> torch.Tensor:
        return self.W_V.T

    @property
    def b_O(self):
        return self.b_D

    @property
    def attn_scale(self) -> float:
        assert self.cfg.attn_scale is not None
        return self.cfg.attn_scale

    def dim_maps(self) -> dict[str, DimMap]:
        maps = {k: DimMap({"model": 0}) for k in ("W_Q", "W_K", "W_V", "W_O", "b_Q", "b_K", "b_V")}
        maps["b_D"] = DimMap({})
        for k in ("mask", "IGNORE", "rotary_sin", "rotary_cos"):
            maps[k] = DimMap({})
        if self.cfg.use_post_qk_ln:
            maps["ln_q.w"] = DimMap({"model": 0})
            maps["ln_k.w"] = DimMap({"model": 0})
        return super().dim_maps() | maps

    # ---- initialisation ----------------------------------------------------------------------
    @torch.no_grad()
    def init_parameters(self, **kwargs):
        super().init_parameters(**kwargs)
        g = shard_generator(self.device_mesh, self.W_V.device)
        d, dq = self.cfg.d_model, self.cfg.d_qk_head
        # Xavier-uniform with the fans of the FULL [n_qk_heads, d, dqk] tensor (fan_in = d*dqk, fan_out = nqk*dqk)
        bound = math.sqrt(6.0 / (d * dq + self.cfg.n_qk_heads * dq))
        self.W_Q.uniform_(-bound, bound, generator=g)
        self.W_K.uniform_(-bound, bound, generator=g)
        self.W_V.normal_(0, 1 / math.sqrt(self.cfg.d_sae), generator=g)
        self.W_O.normal_(0, 1 / math.sqrt(d), generator=g)
        for b in (self.b_Q, self.b_K, self.b_V):
            b.zero_()
        if self.cfg.use_decoder_bias:
            self.b_D.zero_()

    def _local_qk_indices(self) -> torch.Tensor:
        r = mesh_local_rank(self.device_mesh, "model")
        return torch.arange(r * self.n_qk_heads_local, (r + 1) * self.n_qk_heads_local)

    @torch.no_grad()
    def init_lorsa_with_mhsa(self, mhsa):
        """Copy (and repeat) the language model's attention Q/K projections. ``mhsa`` exposes ``W_Q, W_K
        [n_heads, d_model, d_head]`` (and ``ln_q.w / ln_k.w`` when QK-norm is used)."""
        n_orig = mhsa.W_Q.size(0)
        assert self.cfg.n_qk_heads % n_orig == 0 and self.cfg.d_qk_head == mhsa.W_Q.size(2)
        assert self.dataset_average_activation_norm is not None
        f_in = math.sqrt(self.cfg.d_model) / self.dataset_average_activation_norm[self.cfg.hook_point_in]
        rep = self.cfg.n_qk_heads // n_orig
        src = (self._local_qk_indices() // rep).to(mhsa.W_Q.device)
        W_K_full = mhsa.W_K
        if W_K_full.size(0) != n_orig:  # grouped-query attention: expand the KV heads
            W_K_full = torch.repeat_interleave(W_K_full, n_orig // W_K_full.size(0), dim=0)
        self.W_Q.copy_(mhsa.W_Q[src].to(self.cfg.dtype) / f_in)
        self.W_K.copy_(W_K_full[src].to(self.cfg.dtype) / f_in)
        if self.cfg.use_post_qk_ln and hasattr(mhsa, "ln_q"):
            self.ln_q.w.copy_(mhsa.ln_q.w[src].to(self.cfg.dtype))
            kw = mhsa.ln_k.w
            if kw.size(0) != n_orig:
                kw = torch.repeat_interleave(kw, n_orig // kw.size(0), dim=0)
            self.ln_k.w.copy_(kw[src].to(self.cfg.dtype))

    def _orig_head_ranges(self, n_orig: int):
        """(original head index, slice of local OV heads initialised from it)."""
        per = self.cfg.n_ov_heads // n_orig
        r = mesh_local_rank(self.device_mesh, "model")
        lo = r * self.d_sae_local
        for h in range(n_orig):
            a, b = max(h * per, lo), min((h + 1) * per, lo + self.d_sae_local)
            if a < b:
                yield h, slice(a - lo, b - lo)

    @torch.no_grad()
    def init_W_V_with_active_subspace_per_head(self, batch: dict[str, torch.Tensor], mhsa):
        """For the OV heads derived from original head h: put W_V inside the top-``d_qk_head`` principal
        subspace of that head's value read-out and set W_O = W_V W_V^h W_O^h; rows are then normalised.
        ``mhsa`` exposes ``W_V [n_heads, d_model, d_head]`` and ``W_O [n_heads, d_head, d_model]``."""
        x = self.prepare_input(batch)[0].reshape(-1, self.cfg.d_model).to(mhsa.W_V.dtype)
        if self.dp_size > 1:
            x = x.contiguous().clone()
            dist.broadcast(x, group=self.dp_group, group_src=0)
        n_orig = mhsa.W_V.size(0)
        for h, sl in self._orig_head_ranges(n_orig):
            v = (x @ mhsa.W_V[h]) @ mhsa.W_V[h].T
            centered = (v - v.mean(dim=0)).float()
            U, _, _ = torch.linalg.svd(centered.T, full_matrices=False)
            proj = U[:, : self.cfg.d_qk_head].to(self.cfg.dtype)
            self.W_V[sl] = self.W_V[sl, : self.cfg.d_qk_head] @ proj.T
            self.W_O[sl] = (self.W_V[sl].to(mhsa.W_V.dtype) @ mhsa.W_V[h] @ mhsa.W_O[h]).to(self.cfg.dtype)
        self.W_V.div_(self.W_V.norm(dim=1, keepdim=True))
        self.W_O.div_(self.W_O.norm(dim=1, keepdim=True))

    @torch.no_grad()
    def init_W_D_with_active_subspace_per_head(self, batch: dict[str, torch.Tensor], mhsa):
        """Same idea from the output side: W_O inside the principal subspace of each original head's output
        (``mhsa.head_outputs(x)`` -> ``[batch, seq, n_heads, d_model]``), W_V = W_O (W_V^h W_O^h)^T."""
        x = self.prepare_input(batch)[0]
        out = mhsa.head_outputs(x.to(mhsa.W_V.dtype))
        n_orig = mhsa.W_V.size(0)
        for h, sl in self._orig_head_ranges(n_orig):
            o = out[..., h, :].reshape(-1, self.cfg.d_model)
            centered = (o - o.mean(dim=0)).float()
            U, _, _ = torch.linalg.svd(centered.T, full_matrices=False)
            proj = U[:, : self.cfg.d_qk_head].to(self.cfg.dtype)
            self.W_O[sl] = self.W_O[sl, : self.cfg.d_qk_head] @ proj.T
            self.W_V[sl] = (self.W_O[sl].to(mhsa.W_V.dtype) @ (mhsa.W_V[h] @ mhsa.W_O[h]).T).to(self.cfg.dtype)
        self.W_V.div_(self.W_V.norm(dim=1, keepdim=True))
        self.W_O.div_(self.W_O.norm(dim=1, keepdim=True))

    @torch.no_grad()
    def init_encoder_bias_with_mean_hidden_pre(self, batch: dict[str, torch.Tensor]):
        _, hidden_pre = self.encode(self.prepare_input(batch)[0], return_hidden_pre=True)
        mean = hidden_pre.mean(dim=[0, 1])
        if self.dp_size > 1:
            dist.all_reduce(mean, group=self.dp_group)
            mean /= self.dp_size
        self.b_V.sub_(mean)

    @torch.no_grad()
    def reverse_for_off_center(self, batch: dict[str, torch.Tensor]):
        """Flip the sign of OV heads whose pre-activation is positive on fewer than 20 % of the tokens."""
        _, hidden_pre = self.encode(self.prepare_input(batch)[0], return_hidden_pre=True)
        flat = hidden_pre.flatten(0, 1)
        flip = ((flat > 0).float().mean(dim=0) < 0.2).to(self.W_V.dtype) * -2 + 1
        self.W_V.mul_(flip.unsqueeze(1))
        self.W_O.mul_(flip.unsqueeze(1))

    # ---- rotary ------------------------------------------------------------------------------
    def _calculate_sin_cos_rotary(self, rotary_dim: int, n_ctx: int, base: int = 10000, dtype=torch.float32, device="cpu"):
        hp = torch.float64 if dtype == torch.float64 else torch.float32
        pos = torch.arange(n_ctx, dtype=hp, device=device)
        if self.cfg.use_NTK_by_parts_rope:
            inv = 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.int64, device=device).float() / rotary_dim))
            fac, lo, hi, old = (self.cfg.NTK_by_parts_factor, self.cfg.NTK_by_parts_low_freq_factor,
                                self.cfg.NTK_by_parts_high_freq_factor, self.cfg.old_context_len)  # fmt: skip
            wavelen = 2 * math.pi / inv
            inv_l = torch.where(wavelen > old / lo, inv / fac, inv)
            smooth = (old / wavelen - lo) / (hi - lo)
            smoothed = (1 - smooth) * inv_l / fac + smooth * inv_l
            medium = ~(wavelen < old / hi) & ~(wavelen > old / lo)
            freq = 1 / torch.where(medium, smoothed, inv_l)
        else:
            freq = base ** (torch.arange(rotary_dim // 2, dtype=hp, device=device) / (rotary_dim / 2))
        freq = freq.repeat_interleave(2) if self.cfg.rotary_adjacent_pairs else freq.repeat(2)
        angles = pos[:, None] / freq[None, :]
        return torch.sin(angles).to(dtype), torch.cos(angles).to(dtype)

    def _rotate_every_two(self, x: torch.Tensor) -> torch.Tensor:
        if self.cfg.rotary_adjacent_pairs:
            return torch.stack((-x[..., 1::2], x[..., ::2]), dim=-1).flatten(-2)
        n = x.size(-1) // 2
        return torch.cat((-x[..., n:], x[..., :n]), dim=-1)

    def _apply_rotary(self, x: torch.Tensor) -> torch.Tensor:
        """``x [batch, pos, heads, d_head]``"""
        if self.cfg.rotary_scale != 1:
            x = x.repeat_interleave(self.cfg.rotary_scale, dim=-1)
        rd = self.cfg.rotary_dim
        n = x.size(1)
        x_rot, x_pass = (x[..., :rd], x[..., rd:]) if rd < x.size(-1) else (x, x[..., :0])
        cos = self.rotary_cos[None, :n, None, :].to(x.dtype)
        sin = self.rotary_sin[None, :n, None, :].to(x.dtype)
        return torch.cat([x_rot * cos + self._rotate_every_two(x_rot) * sin, x_pass], dim=-1)

    # ---- norms / folding -----------------------------------------------------------------------
    def encoder_norm(self, keepdim: bool = False) -> torch.Tensor:
        return torch.norm(self.W_V, p=2, dim=1, keepdim=keepdim)

    def decoder_norm(self, keepdim: bool = False) -> torch.Tensor:
        return torch.norm(self.W_O, p=2, dim=1, keepdim=keepdim)

    def decoder_bias_norm(self) -> torch.Tensor:
        if not self.cfg.use_decoder_bias:
            raise ValueError("Decoder bias not used")
        return torch.norm(self.b_D, p=2, dim=0, keepdim=True)

    @torch.no_grad()
    def transform_to_unit_decoder_norm(self):
        n = self.decoder_norm(keepdim=True)
        self.W_O.div_(n)
        self.W_V.mul_(n)
        self.b_V.mul_(n.squeeze(1))

    @torch.no_grad()
    def set_decoder_to_fixed_norm(self, value: float, force_exact: bool):
        """Rescales by the MEAN row norm (all rows by one factor), as the reference does for this model."""
        mean = self._mean_over_shards(self.decoder_norm())
        self.W_O.mul_(value / (mean if force_exact else max(mean, value)))

    @torch.no_grad()
    def set_encoder_to_fixed_norm(self, value: float):
        raise NotImplementedError("set_encoder_to_fixed_norm does not make sense for lorsa")

    @torch.no_grad()
    def standardize_parameters_of_dataset_norm(self):
        assert self.cfg.norm_activation == "dataset-wise" and self.dataset_average_activation_norm is not None
        root = math.sqrt(self.cfg.d_model)
        f_in = root / self.dataset_average_activation_norm[self.cfg.hook_point_in]
        f_out = root / self.dataset_average_activation_norm[self.cfg.hook_point_out]
        self.W_Q.data.mul_(f_in)
        self.W_K.data.mul_(f_in)
        self.W_V.data.mul_(f_in)
        self.W_O.data.div_(f_out)
        if self.cfg.use_decoder_bias:
            self.b_D.data.div_(f_out)
        self.cfg.norm_activation = "inference"

    # ---- forward -----------------------------------------------------------------------------
    def _tensor_core_attention(self, x: torch.Tensor) -> bool:
        """Whether the forward pass of ``x [b, s, d]`` goes through this package's attention kernels."""
        group = self.W_V.shape[0] // max(self.n_qk_heads_local, 1)
        return (
            self.cfg.attention_kernel == "tensor_core" and x.is_cuda and x.ndim == 3 and self.W_Q.dtype == torch.bfloat16
            and self.cfg.d_qk_head in (64, 128) and group % 64 == 0 and x.shape[1] % 8 == 0
        )  # fmt: skip

    def _compute_qkv(self, x: torch.Tensor, with_v: bool = True) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor | None]:
        """``x [b, s, d]`` -> ``q, k [b, s, nqk_l, dqk]``, ``v [b, s, F_l]`` (None when not wanted)."""
        x = x.to(self.W_Q.dtype)
        q = self.hook_q(torch.einsum("bsd,hdq->bshq", x, self.W_Q) + self.b_Q)
        k = self.hook_k(torch.einsum("bsd,hdq->bshq", x, self.W_K) + self.b_K)
        v = x @ self.W_V.T + self.b_V if with_v else None
        if self.cfg.use_post_qk_ln:
            q, k = self.ln_q(q), self.ln_k(k)
        if self.cfg.positional_embedding_type == "rotary":
            q, k = self._apply_rotary(q), self._apply_rotary(k)
        return self.hook_q_post_rot(q), self.hook_k_post_rot(k), v

    def _apply_causal_mask(self, scores: torch.Tensor) -> torch.Tensor:
        n = scores.size(-2)
        return torch.where(self.mask[None, None, -n:, -n:], scores, self.IGNORE.to(scores.dtype))

    def _compute_attention_pattern(self, q: torch.Tensor, k: torch.Tensor) -> torch.Tensor:
        """``[nqk_l, b, q_pos, k_pos]`` causal softmax patterns."""
        scores = torch.einsum("bqhd,bkhd->hbqk", q, k) / self.attn_scale
        return F.softmax(self._apply_causal_mask(scores), dim=-1)

    def _compute_head_outputs(self, pattern: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """``pattern [b, nqk_l, q, k]``, ``v [b, s, F_l]`` -> ``z [b, s, F_l]``."""
        b, s, _ = v.shape
        vg = v.view(b, s, self.n_qk_heads_local, -1)  # [b, k, h, group]
        z = torch.einsum("bhqk,bkhg->bqhg", pattern, vg)
        return z.reshape(b, s, -1)

    def compute_hidden_pre(self, x: torch.Tensor) -> torch.Tensor:
        q, k, v = self._compute_qkv(x, with_v=not self._tensor_core_attention(x))
        return self._attend(q, k, v, x)

    def _attend(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, x: torch.Tensor | None = None) -> torch.Tensor:
        """Fused causal attention: one attention head per QK head whose value / output width is the OV group."""
        b, s, h, _ = q.shape
        if v is None:
            # tcgen05 kernels (forward, dQ, dK/dV) that take a value width different from the query/key width; the values
            # are produced straight in the layout the forward kernel reads, [b, h, group, s]: one GEMM, no transpose pass
            assert x is not None
            vt = (torch.matmul(self.W_V, x.to(self.W_V.dtype).transpose(1, 2)) + self.b_V[:, None]).view(b, h, -1, s)
            return attention_kernels.causal_attention(q, k, None, 1 / self.attn_scale, vt=vt).reshape(b, s, -1)
        vg = v.view(b, s, h, -1)
        value = vg.permute(0, 2, 1, 3)
        import contextlib

        # on CUDA the library's cuDNN backend is kept out: its backward pass was seen to return wrong gradients here
        with attention_kernels.library_attention_backends() if q.is_cuda else contextlib.nullcontext():
            z = F.scaled_dot_product_attention(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), value,
                                               scale=1 / self.attn_scale, is_causal=True)  # fmt: skip
        return z.permute(0, 2, 1, 3).reshape(b, s, -1)

    def encode(
        self,
        x: torch.Tensor,
        return_hidden_pre: bool = False,
        return_attention_pattern: bool = False,
        return_attention_score: bool = False,
        hook_attn_scores: bool = False,
        **kwargs,
    ):
        """``x [batch, seq, d_model]`` -> sparse OV-head activations ``[batch, seq, F_l]``."""
        pattern = scores = None
        slow = return_attention_pattern or return_attention_score or hook_attn_scores
        slow = slow or bool(self.hook_attn_pattern.fwd_hooks or self.hook_attn_score.fwd_hooks)
        q, k, v = self._compute_qkv(x, with_v=slow or not self._tensor_core_attention(x))
        if not slow:
            hidden_pre = self._attend(q, k, v, x)
        else:
            scores = torch.einsum("bqhd,bkhd->bhqk", q, k) / self.attn_scale
            scores = self.hook_attn_score(self._apply_causal_mask(scores))
            pattern = self.hook_attn_pattern(F.softmax(scores, dim=-1))
            hidden_pre = self._compute_head_outputs(pattern, v)
        hidden_pre = self.hook_hidden_pre(hidden_pre)
        if self.cfg.sparsity_include_decoder_norm:
            norm = self.decoder_norm()
            feature_acts = self.activation_function(hidden_pre * norm) / norm
        else:
            feature_acts = self.activation_function(hidden_pre)
        out = [self.hook_feature_acts(feature_acts)]
        if return_hidden_pre:
            out.append(hidden_pre)
        if return_attention_pattern and pattern is not None:
            out.append(pattern)
        if return_attention_score and scores is not None:
            out.append(scores)
        return tuple(out) if len(out) > 1 else out[0]

    def decode(self, feature_acts: torch.Tensor, **kwargs) -> torch.Tensor:
        if feature_acts.layout == torch.sparse_coo:
            out = torch.sparse.mm(feature_acts.to(torch.float32), self.W_O.to(torch.float32)).to(self.cfg.dtype)
        else:
            out = feature_acts @ self.W_O
        out = all_reduce_sum(out, self.tp_group)
        if self.cfg.use_decoder_bias:
            out = out + self.b_D
        return self.hook_reconstructed(out)

    def _decode_linear(self, feature_acts: torch.Tensor) -> torch.Tensor:
        return feature_acts @ self.W_O

    def encode_z_pattern_for_head(self, x: torch.Tensor, head_idx: torch.Tensor) -> torch.Tensor:
        """Per selected OV head, the contribution of every source position to every target position:
        ``pattern[qk(head)] * v[head]`` -> ``[n_heads_selected, q_pos, k_pos]`` (``x``: ``[1, seq, d]``)."""
        assert x.size(0) == 1, f"x must be of shape (1, seq_len, d_model), but got {x.shape}"
        q, k, v = self._compute_qkv(x)
        patterns = self._compute_attention_pattern(q, k)
        pattern = patterns[head_idx // self.cfg.ov_group_size, 0]
        return pattern * v[0, :, head_idx].T.unsqueeze(1)

    def encode_z_patterns(self, x: torch.Tensor) -> torch.Tensor:
        return self.encode_z_pattern_for_head(x, torch.arange(self.d_sae_local, device=x.device))

    def load_full_state_dict(self, state_dict: dict[str, torch.Tensor], strict: bool = True) -> None:
        """Checkpoints with fewer QK heads are expanded by repeating each head."""
        state_dict = dict(state_dict)
        if "W_Q" in state_dict:
            n_ckpt = state_dict["W_Q"].size(0)
            n_want = self.cfg.n_qk_heads if state_dict["W_Q"].size(0) != self.n_qk_heads_local or self.tp_size == 1 else n_ckpt
            if n_want != n_ckpt and n_want % n_ckpt == 0 and n_ckpt != self.n_qk_heads_local:
                rep = n_want // n_ckpt
                keys = ["W_Q", "W_K", "b_Q", "b_K"] + (["ln_q.w", "ln_k.w"] if self.cfg.use_post_qk_ln else [])
                for key in keys:
                    if key in state_dict:
                        state_dict[key] = torch.repeat_interleave(state_dict[key], rep, dim=0)
        super().load_full_state_dict(state_dict, strict=strict)

    def prepare_input(self, batch: dict[str, torch.Tensor], **kwargs) -> tuple[torch.Tensor, dict[str, Any], dict[str, Any]]:
        return batch[self.cfg.hook_point_in], {}, {}

    def prepare_label(self, batch: dict[str, torch.Tensor], **kwargs) -> torch.Tensor:
        return batch[self.cfg.hook_point_out]
