"""One training step of a low-rank sparse attention dictionary (Lorsa) with a TopK activation over its OV heads as a short
fixed sequence of kernels, without an autograd graph over the model.

What it computes is the reference's step for a ``LowRankSparseAttention`` (models/lorsa.py:642-661 projections and rotary
embedding, :714-725 attention with the OV group as the value width, :764-782 activation gated by the decoder norms,
:784-829 decode; MSE over tokens) with Adam. On the generic path that step is some 230 kernel launches, two thirds of
them small element-wise kernels that autograd and autocast put around the few products that matter; here it is:

1. three tcgen05 GEMMs ``x W^T + b`` for Q, K (all QK heads in one product each) and V, bf16 results
2. rotary embedding of Q and K (one kernel for both), attention with one head per QK head whose
   value width is the head's OV group (this package's tcgen05 kernels, or the library's memory-efficient backend for
   shapes they do not take)                                          -> pre-activations z [tokens, F] bf16
3. radix row top-k of ``z * ||W_O row||`` (positive entries)          -> codes (idx, act) [tokens, k]
4. sparse decode fused with the loss, d x_hat and d act (the kernel of the TopK SAE step; feature shards: sparse decode,
   all-reduce, loss kernel, code-gradient kernel)
5. d z = d act scattered to its positions; attention backward (the dQ and dK/dV kernels, or the library's, through a
   one-node autograd call on the attention alone); inverse rotation of d q, d k
6. three library GEMMs for the projection gradients (``d q^T x`` ...), column sums for the biases
7. updates: ``W_O`` by the sparse gradient + Adam kernel (rows rebuilt from the codes, bf16 shadow and row norms in the
   same pass), the dense projections and biases by the flat Adam kernel.

Restrictions: ``topk`` activation, rotary or no positional embedding (no ``rotary_scale``; the per-head RMS norm of Q and K
only on request, see ``QK_NORM_ON_FUSED_PATH``), Adam, fp32
parameters with bf16 compute; heads sharded over ``model``, sequences split over ``data`` (replicas sum their dense
gradients in one collective and gather codes and output gradients for the sparse update of ``W_O``).
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..parallel.mesh import mesh_dim_size, mesh_group, mesh_local_rank
from . import attention as attention_kernels
from .attention import library_attention_backends
from . import sae_kernels as K
from .fused_step import _mm_f32, merge_codes_over_shards


def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, adjacent: bool, rd: int) -> torch.Tensor:
    """Rotary embedding of ``x [b, s, h, d_head]`` on its first ``rd`` channels (models/lorsa.py:666-712 of the reference
    project); with ``-sin`` the same call is the inverse rotation, which is also the backward pass of the forward one."""
    xr = x[..., :rd]
    if adjacent:
        turned = torch.stack((-xr[..., 1::2], xr[..., ::2]), dim=-1).flatten(-2)
    else:
        n = rd // 2
        turned = torch.cat((-xr[..., n:], xr[..., :n]), dim=-1)
    out = xr * cos + turned * sin
    return out if rd == x.shape[-1] else torch.cat([out, x[..., rd:]], dim=-1)


def rotate_pair(a: torch.Tensor, b: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, adjacent: bool, inverse: bool = False):
    """Rotary embedding (or its inverse) of two ``[batch, seq, heads, width]`` tensors with tables ``cos, sin [n_ctx, rd]``:
    one kernel for both on a GPU (bf16 tensors, fp32 tables, aligned widths), ``_rotate`` otherwise."""
    bsz, s, h, w = a.shape
    rd = cos.shape[-1]
    fast = (a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and cos.dtype == torch.float32 and w % 8 == 0
            and rd % (8 if adjacent else 16) == 0 and cos.is_contiguous() and sin.is_contiguous())  # fmt: skip
    if not fast:
        c, sn = cos[None, :s, None, :].to(a.dtype), sin[None, :s, None, :].to(a.dtype)
        sn = -sn if inverse else sn
        return _rotate(a, c, sn, adjacent, rd), _rotate(b, c, sn, adjacent, rd)
    a, b = a.contiguous(), b.contiguous()
    oa, ob = torch.empty_like(a), torch.empty_like(b)
    K._ext().rotary_pair(a.view(bsz * s, h, w), b.view(bsz * s, h, w), oa.view(bsz * s, h, w), ob.view(bsz * s, h, w), cos, sin, s, adjacent,
                         -1.0 if inverse else 1.0)  # fmt: skip
    return oa, ob


def QK_NORM_ON_FUSED_PATH() -> bool:
    """The per-head RMS norm of Q and K on the fused step is verified against autograd on the CPU (it is a second small
    autograd node of torch statements in front of the rotation), but has not run on a GPU: taken only on request."""
    return "1" in (os.environ.get("LMSAE_FUSED_LORSA_QK_NORM", "0"), os.environ.get("LMSAE_FUSED_CPU_VERIFIED", "0"))


class FusedLorsaStep:
    def __init__(self, lorsa, betas: tuple[float, float] = (0.9, 0.999), eps: float = 1e-8, attention: str | None = None):
        """``attention``: ``"tensor_core"`` (this package's tcgen05 forward, dQ and dK/dV kernels, where the shape allows:
        d_qk 64 or 128, OV group a multiple of 64, sequence a multiple of 8) or ``"library"``; default from
        ``LMSAE_LORSA_ATTENTION``, else ``tensor_core``."""
        cfg = lorsa.cfg
        self.attention = attention or os.environ.get("LMSAE_LORSA_ATTENTION", "tensor_core")
        assert self.attention in ("tensor_core", "library"), self.attention
        self.m = lorsa
        self.betas, self.eps = betas, eps
        self.tp = mesh_dim_size(lorsa.device_mesh, "model")
        self.tp_rank = mesh_local_rank(lorsa.device_mesh, "model")
        self.tp_group = mesh_group(lorsa.device_mesh, "model")
        self.dp = mesh_dim_size(lorsa.device_mesh, "data")
        self.dp_group = mesh_group(lorsa.device_mesh, "data")
        self.h, self.d, self.dqk = lorsa.W_Q.shape  # local QK heads, d_model, QK head width
        self.F = lorsa.W_V.shape[0]  # local OV heads
        self.group_size = self.F // self.h
        self.own_rows = (0, self.F)  # no sharding of the optimizer state over data ranks
        self.use_gate = cfg.sparsity_include_decoder_norm
        self.rotary = cfg.positional_embedding_type == "rotary"
        self.params = {"W_Q": lorsa.W_Q.data, "W_K": lorsa.W_K.data, "W_V": lorsa.W_V.data, "W_O": lorsa.W_O.data,
                       "b_Q": lorsa.b_Q.data, "b_K": lorsa.b_K.data, "b_V": lorsa.b_V.data}  # fmt: skip
        if cfg.use_decoder_bias:
            self.params["b_D"] = lorsa.b_D.data
        self.qk_norm = bool(cfg.use_post_qk_ln)
        if self.qk_norm:  # learned scales of the per-head RMS norms of Q and K
            self.params["ln_q.w"], self.params["ln_k.w"] = lorsa.ln_q.w.data, lorsa.ln_k.w.data
        assert all(p.dtype == torch.float32 and p.is_contiguous() for p in self.params.values())
        dev = lorsa.W_V.device
        self.state = {n: (torch.zeros_like(p), torch.zeros_like(p)) for n, p in self.params.items()}
        bf = lambda *s: torch.empty(*s, dtype=torch.bfloat16, device=dev)  # noqa: E731
        self.WQ16, self.WK16 = bf(self.h * self.dqk, self.d), bf(self.h * self.dqk, self.d)  # [head x channel, d]: rows of x W^T
        self.WV16, self.WO16 = bf(self.F, self.d), bf(self.F, self.d)
        self.dec_norm = torch.empty(self.F, dtype=torch.float32, device=dev)
        self.loss_sum = torch.zeros(1, dtype=torch.float32, device=dev)
        self.groups: K.FeatureGroups | None = None
        self.t = 0
        self.refresh()

    @staticmethod
    def supports(lorsa, trainer_cfg=None) -> tuple[bool, str]:
        from ..models.lorsa import LowRankSparseAttention

        cfg = lorsa.cfg
        if type(lorsa) is not LowRankSparseAttention:
            return False, "model is not a LowRankSparseAttention"
        checks = [
            (cfg.act_fn == "topk", "activation is not topk"),
            (lorsa.W_V.is_cuda or trainer_cfg is None, "not on a CUDA device"),
            (cfg.dtype == torch.float32, "parameters are not fp32"),
            (cfg.positional_embedding_type in ("rotary", "none"), "positional embedding"),
            (cfg.rotary_scale == 1, "rotary scale"),
            (not cfg.use_post_qk_ln or QK_NORM_ON_FUSED_PATH(), "QK layer norm (set LMSAE_FUSED_LORSA_QK_NORM=1)"),
            (cfg.d_model % 64 == 0 and cfg.d_qk_head % 8 == 0 and lorsa.W_V.shape[0] % 8 == 0, "d_model / head widths not aligned"),
            (lorsa.W_V.shape[0] % max(lorsa.W_Q.shape[0], 1) == 0 and (lorsa.W_V.shape[0] // max(lorsa.W_Q.shape[0], 1)) % 8 == 0,
             "OV group size not a multiple of 8"),
            (not any(hp.fwd_hooks or hp.bwd_hooks for hp in lorsa.hook_points()), "hooks are attached"),
        ]  # fmt: skip
        if trainer_cfg is not None:
            checks += [
                (trainer_cfg.sparsity_loss_type is None, "sparsity loss"),
                (not trainer_cfg.lp_coefficient, "lp loss"),
                (not trainer_cfg.auxk_coefficient, "aux-k loss"),
                (trainer_cfg.optimizer_class == "adam", "optimizer is not adam"),
                (trainer_cfg.amp_dtype == torch.bfloat16, "amp dtype is not bf16"),
                (trainer_cfg.gradient_accumulation_steps == 1, "gradient accumulation"),
                (not trainer_cfg.clip_grad_norm, "gradient clipping"),
            ]
        for ok, why in checks:
            if not ok:
                return False, why
        return True, ""

    # ---- shadows ---------------------------------------------------------------------------------
    def _refresh_qk(self) -> None:
        # parameters are [head, d, channel]; the GEMM wants the rows of W^T: [head x channel, d]
        self.WQ16.copy_(self.params["W_Q"].permute(0, 2, 1).reshape(self.h * self.dqk, self.d))
        self.WK16.copy_(self.params["W_K"].permute(0, 2, 1).reshape(self.h * self.dqk, self.d))

    def refresh(self) -> None:
        """Re-derive the bf16 shadows and decoder norms from the fp32 masters (after loading / editing weights)."""
        self._refresh_qk()
        K.row_norm_shadow(self.params["W_V"], None, self.WV16)
        K.row_norm_shadow(self.params["W_O"], self.dec_norm, self.WO16)

    def join(self) -> None:
        pass

    def sync_params(self) -> None:
        pass

    # ---- forward pieces -----------------------------------------------------------------------------
    def _project(self, X: torch.Tensor, b: int, s: int):
        """``X [tokens, d]`` bf16 -> rotated ``q, k [b, s, h, dqk]`` and ``v [b, s, h, group]`` (bf16 on CUDA)."""
        q, k, v = self._project_linear(X, b, s)
        if self.qk_norm:
            with torch.no_grad():
                q, k = self.m.ln_q(q), self.m.ln_k(k)
        return (*self._rotated(q, k), v)

    def _project_linear(self, X: torch.Tensor, b: int, s: int):
        q = K.encoder_hidden(X, self.WQ16, self.params["b_Q"].reshape(-1)).view(b, s, self.h, self.dqk)
        k = K.encoder_hidden(X, self.WK16, self.params["b_K"].reshape(-1)).view(b, s, self.h, self.dqk)
        v = K.encoder_hidden(X, self.WV16, self.params["b_V"]).view(b, s, self.h, self.group_size)
        return q, k, v

    def _rotated(self, q: torch.Tensor, k: torch.Tensor):
        if self.rotary:
            q, k = rotate_pair(q, k, self.m.rotary_cos, self.m.rotary_sin, self.m.cfg.rotary_adjacent_pairs)
        return q, k

    def _attention(self, q, k, v):
        """Library attention on ``[b, h, s, *]`` views; fp32 on CPU (the plain statement), bf16 on CUDA, where the backend is
        pinned (see ``library_attention_backends``)."""
        if not q.is_cuda:
            q, k, v = q.float(), k.float(), v.float()
            return F.scaled_dot_product_attention(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3),
                                                  scale=1.0 / self.m.attn_scale, is_causal=True)  # fmt: skip
        if self.attention == "tensor_core" and attention_kernels.supported(q, v):
            return attention_kernels.causal_attention(q, k, v, 1.0 / self.m.attn_scale).permute(0, 2, 1, 3)
        with library_attention_backends():
            return F.scaled_dot_product_attention(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3),
                                                  scale=1.0 / self.m.attn_scale, is_causal=True)  # fmt: skip

    def encode(self, x: torch.Tensor, k_top: int) -> tuple[torch.Tensor, torch.Tensor]:
        """``x [b, s, d]`` bf16 -> codes ``(idx, act) [tokens, k]`` over this rank's OV heads."""
        b, s, _ = x.shape
        with torch.no_grad():
            q, k, v = self._project(x.reshape(b * s, self.d).contiguous(), b, s)
            z = self._attention(q, k, v).permute(0, 2, 1, 3).reshape(b * s, self.F)
        return self._select(z, k_top)

    def _select(self, z: torch.Tensor, k_top: int) -> tuple[torch.Tensor, torch.Tensor]:
        gate = self.dec_norm if self.use_gate else None
        idx, act = K.row_topk(z.to(torch.bfloat16) if z.is_cuda else z.float(), k_top, gate, None)
        if self.tp > 1:
            idx, act = merge_codes_over_shards(idx, act, gate, k_top, self.tp, self.tp_rank, self.tp_group)
        return idx, act

    # ---- the step ---------------------------------------------------------------------------------
    def step(self, x: torch.Tensor, label: torch.Tensor, k_top: int, lr: float, row_weight: torch.Tensor | None = None) -> torch.Tensor:
        """``x [b, s, d]`` normalised bf16 inputs, ``label [b, s, d]`` bf16 targets (the attention layer's output). Returns
        the mean loss over tokens (0-d device tensor). ``row_weight [b x s]`` fp32 weighs every token's squared error
        (0 for masked tokens and ``tokens / valid tokens`` for the others gives the mean over valid tokens; masked
        tokens still serve as keys and values of later positions, as they do in the model's own forward pass)."""
        b, s, d = x.shape
        T_l = b * s  # this replica's tokens
        T = T_l * self.dp  # the step's tokens: every replica brings the same number of sequences
        X = x.reshape(T_l, d).contiguous()
        Y = label.reshape(T_l, d).contiguous()
        grad_scale = 2.0 / T
        norm_node = None
        if self.qk_norm:
            # a second small autograd node in front of the rotation: the per-head RMS norms of Q and K with their scales
            q0, k0, v = self._project_linear(X, b, s)
            q0, k0 = q0.detach().requires_grad_(True), k0.detach().requires_grad_(True)
            wq, wk = self.m.ln_q.w, self.m.ln_k.w
            with torch.enable_grad():
                qn, kn = self.m.ln_q(q0), self.m.ln_k(k0)
            norm_node = (qn, kn, q0, k0, wq, wk)
            q, k = self._rotated(qn.detach(), kn.detach())
        else:
            q, k, v = self._project(X, b, s)
        # the attention alone keeps an autograd node (its backward is the library's); everything around it is explicit
        ql, kl, vl = (t.detach().requires_grad_(True) for t in (q, k, v))
        with torch.enable_grad():
            out = self._attention(ql, kl, vl)  # [b, h, s, group]
        z = out.detach().permute(0, 2, 1, 3).reshape(T_l, self.F)
        idx, act = self._select(z, k_top)
        self.loss_sum.zero_()
        WO16 = self.WO16
        bD = self.params.get("b_D")
        if self.tp == 1:
            dxhat, dact, _ = K.sparse_decode_loss(idx, act, WO16, bD, Y, row_weight, grad_scale, self.loss_sum)
        else:
            xhat = K.sparse_decode(idx, act, WO16, None, torch.float32)
            dist.all_reduce(xhat, group=self.tp_group)
            dxhat = K.mse_loss_grad(xhat, Y, bD, row_weight, grad_scale, self.loss_sum)
            dact = K.sparse_dact(idx, WO16, dxhat)
        # d z: the activation passes the gradient where a head was selected (its value is the pre-activation itself)
        dz = torch.zeros(T_l, self.F + 8, dtype=z.dtype if z.is_cuda else torch.float32, device=x.device)
        dz.scatter_(1, torch.where(idx >= 0, idx, torch.full_like(idx, self.F)).long(), dact.to(dz.dtype))
        dz = dz[:, : self.F].reshape(b, s, self.h, self.group_size).permute(0, 2, 1, 3)
        dq, dk, dv = torch.autograd.grad(out, (ql, kl, vl), dz.to(out.dtype))
        if self.rotary:
            dq, dk = rotate_pair(dq, dk, self.m.rotary_cos, self.m.rotary_sin, self.m.cfg.rotary_adjacent_pairs, inverse=True)
        norm_grads = {}
        if norm_node is not None:
            qn, kn, q0, k0, wq, wk = norm_node
            dq, gwq = torch.autograd.grad(qn, (q0, wq), dq.to(qn.dtype))
            dk, gwk = torch.autograd.grad(kn, (k0, wk), dk.to(kn.dtype))
            norm_grads = {"ln_q.w": gwq.float(), "ln_k.w": gwk.float()}
        low = torch.bfloat16 if x.is_cuda else torch.float32
        dQ = dq.reshape(T_l, self.h * self.dqk).to(low)
        dK = dk.reshape(T_l, self.h * self.dqk).to(low)
        dV = dv.reshape(T_l, self.F).to(low)
        Xl = X.to(low)
        grads = {
            # [head x channel, d] -> the parameter's [head, d, channel]
            "W_Q": _mm_f32(dQ.t(), Xl).view(self.h, self.dqk, d).permute(0, 2, 1).contiguous(),
            "W_K": _mm_f32(dK.t(), Xl).view(self.h, self.dqk, d).permute(0, 2, 1).contiguous(),
            "W_V": _mm_f32(dV.t(), Xl),
            "b_Q": dQ.sum(0, dtype=torch.float32).view(self.h, self.dqk),
            "b_K": dK.sum(0, dtype=torch.float32).view(self.h, self.dqk),
            "b_V": dV.sum(0, dtype=torch.float32),
        }
        if bD is not None:
            grads["b_D"] = K.colsum_bf16(dxhat)
        grads.update(norm_grads)
        if self.dp > 1:
            # Replicas: the dense gradients (some 50 MB at 8192 heads) are summed in one collective on a flat buffer; for W_O the
            # codes and the output gradient of every replica (a few MB) are gathered and each replica rebuilds the same rows, so
            # that no dense [F, d] gradient exists here either. Every replica then applies the same update.
            names = list(grads)
            flat = torch.cat([grads[n].reshape(-1) for n in names])
            dist.all_reduce(flat, group=self.dp_group)
            off = 0
            for n in names:
                grads[n] = flat[off : off + grads[n].numel()].view(grads[n].shape)
                off += grads[n].numel()
            idx, act, dact, dxhat = (self._gather_rows(t) for t in (idx, act, dact, dxhat))
            dist.all_reduce(self.loss_sum, group=self.dp_group)
        self.t += 1
        b1, b2 = self.betas
        # W_O: rows rebuilt from the codes (act x d x_hat), Adam, bf16 shadow and row norms in one pass
        if self.groups is None or self.groups.entries.numel() < idx.numel():
            self.groups = K.FeatureGroups(self.F, idx.numel(), x.device)
        self.groups.build(idx)
        mO, vO = self.state["W_O"]
        K.sparse_grad_adam(self.groups, act, dact, dxhat, dxhat, self.params["W_O"], mO, vO, WO16, None, None, None, None, None, None, None,
                           self.dec_norm, None, None, lr, b1, b2, self.eps, self.t, True)  # fmt: skip
        for name, g in grads.items():
            m_, v_ = self.state[name]
            shadow = self.WV16.view(-1) if name == "W_V" else None
            K.adam_flat(self.params[name].view(-1), g.reshape(-1), m_.view(-1), v_.view(-1), lr, b1, b2, self.eps, self.t, shadow=shadow)
        self._refresh_qk()
        return (self.loss_sum / T).squeeze(0)

    def _gather_rows(self, t: torch.Tensor) -> torch.Tensor:
        """``[rows, n]`` of every replica stacked in rank order."""
        t = t.contiguous()
        out = torch.empty(self.dp * t.shape[0], *t.shape[1:], dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t, group=self.dp_group)
        return out

    # ---- optimizer state in the model's parameter shapes -------------------------------------------------
    def optimizer_state(self) -> dict:
        out = {"step": self.t}
        for name, (m_, v_) in self.state.items():
            out[name] = {"exp_avg": m_, "exp_avg_sq": v_}
        return out

    def load_optimizer_state(self, sd: dict) -> None:
        self.t = int(sd["step"])
        for name, (m_, v_) in self.state.items():
            if name in sd:
                m_.copy_(sd[name]["exp_avg"])
                v_.copy_(sd[name]["exp_avg_sq"])
