"""Cross-layer transcoder decoder fan-out on sparse codes: wrappers, torch oracles and the autograd entry point.

The decoder of a cross-layer transcoder sends the features of source layer ``s`` to every target layer ``t >= s``
(models/clt.py:629-709 of the reference project: one dense or CSR product per ``(s, t)`` pair, one all-reduce per target
layer). The kernels of ``csrc/clt_ops.cu`` work on one padded code list per token, ``c = s * F + f``:

* ``clt_decode``   every target layer in one launch, gathering only the decoder rows of active features;
* ``clt_dact``     gradient of the codes;
* ``clt_wgrad``    gradient of the decoders from by-feature lists (counting sort), written as rows of zero-filled dense
  tensors so that any optimizer can consume them.

Operands are bf16 with fp32 accumulation; the oracles below do the same math in plain torch (any device).
"""

from __future__ import annotations

from typing import Sequence

import torch

from . import sae_kernels as K
from .sparse_autograd import dense_to_padded_sparse


def _split(idx: torch.Tensor, F: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    valid = idx >= 0
    c = idx.clamp_min(0).long()
    return valid, c // F, c % F


def ref_clt_decode(idx: torch.Tensor, val: torch.Tensor, weights: Sequence[torch.Tensor], bias: torch.Tensor | None) -> torch.Tensor:
    """``[L, B, d]`` fp32: ``y[t, b] = bias[t] + sum_j [s_j <= t] val[b, j] * weights[t][s_j, f_j]``."""
    L = len(weights)
    F, d = weights[0].shape[1:]
    B, Kc = idx.shape
    valid, s, f = _split(idx, F)
    out = torch.zeros(L, B, d, dtype=torch.float32, device=idx.device)
    for t in range(L):
        use = valid & (s <= t)
        rows = weights[t].float()[s.clamp_max(t), f]  # [B, K, d]
        out[t] = (rows * (val * use).unsqueeze(-1)).sum(dim=1)
        if bias is not None:
            out[t] += bias[t].float()
    return out


def ref_clt_dact(idx: torch.Tensor, weights: Sequence[torch.Tensor], dy: torch.Tensor) -> torch.Tensor:
    L = len(weights)
    F = weights[0].shape[1]
    valid, s, f = _split(idx, F)
    out = torch.zeros(idx.shape, dtype=torch.float32, device=idx.device)
    for t in range(L):
        use = valid & (s <= t)
        rows = weights[t].float()[s.clamp_max(t), f]
        out += (rows * dy[t].float().unsqueeze(1)).sum(dim=-1) * use
    return out


def ref_clt_wgrad(idx: torch.Tensor, val: torch.Tensor, dy: torch.Tensor, L: int, F: int) -> list[torch.Tensor]:
    B, Kc = idx.shape
    d = dy.shape[-1]
    valid, s, f = _split(idx, F)
    grads = []
    rows_b = torch.arange(B, device=idx.device)[:, None].expand(B, Kc)
    for t in range(L):
        g = torch.zeros((t + 1) * F, d, dtype=torch.float32, device=idx.device)
        use = valid & (s <= t)
        contrib = val[use].unsqueeze(-1) * dy[t].float()[rows_b[use]]
        g.index_add_(0, idx[use].long(), contrib)
        grads.append(g.view(t + 1, F, d))
    return grads


def clt_decode(idx, val, weights16: Sequence[torch.Tensor], bias: torch.Tensor | None, out_dtype=torch.float32) -> torch.Tensor:
    L, (F, d) = len(weights16), weights16[0].shape[1:]
    if not idx.is_cuda:
        return ref_clt_decode(idx, val, weights16, bias).to(out_dtype)
    out = torch.empty(L, idx.shape[0], d, dtype=out_dtype, device=idx.device)
    K._ext().clt_decode(idx, val, list(weights16), None if bias is None else bias.float().contiguous(), out)
    return out


def clt_dact(idx, weights16: Sequence[torch.Tensor], dy16: torch.Tensor) -> torch.Tensor:
    if not idx.is_cuda:
        return ref_clt_dact(idx, weights16, dy16)
    dval = torch.empty(idx.shape, dtype=torch.float32, device=idx.device)
    K._ext().clt_dact(idx, list(weights16), dy16, dval)
    return dval


def clt_wgrad(idx, val, dy16: torch.Tensor, L: int, F: int) -> list[torch.Tensor]:
    if not idx.is_cuda:
        return ref_clt_wgrad(idx, val, dy16, L, F)
    B, Kc = idx.shape
    d = dy16.shape[-1]
    groups = K.FeatureGroups(L * F, idx.numel(), idx.device).build(idx)
    grads = [torch.zeros(t + 1, F, d, dtype=torch.float32, device=idx.device) for t in range(L)]
    K._ext().clt_wgrad(groups.offsets, groups.entries, val, dy16, grads, B, Kc)
    return grads


class CLTSparseDecode(torch.autograd.Function):
    """``acts [B, L, F]`` (sparse), ``bias [L, d]`` or None, ``W_D[0..L-1]`` -> ``[L, B, d]``; gradients for all."""

    @staticmethod
    def forward(ctx, acts: torch.Tensor, bias: torch.Tensor | None, *weights: torch.Tensor) -> torch.Tensor:
        B, L, F = acts.shape
        idx, val = dense_to_padded_sparse(acts.detach().reshape(B, L * F))
        w16 = [w.detach().to(torch.bfloat16).contiguous() for w in weights]
        out = clt_decode(idx, val, w16, None if bias is None else bias.detach(), torch.float32)
        ctx.save_for_backward(idx, val, *w16)
        ctx.meta = (B, L, F, acts.dtype, None if bias is None else bias.dtype, [w.dtype for w in weights])
        return out if acts.dtype == torch.float32 else out.to(acts.dtype)

    @staticmethod
    def backward(ctx, grad_out: torch.Tensor):
        idx, val, *w16 = ctx.saved_tensors
        B, L, F, act_dtype, bias_dtype, w_dtypes = ctx.meta
        g16 = grad_out.to(torch.bfloat16).contiguous()
        d_acts = d_bias = None
        d_w: list[torch.Tensor | None] = [None] * L
        if ctx.needs_input_grad[0]:
            dval = clt_dact(idx, w16, g16)
            flat = torch.zeros(B, L * F, dtype=torch.float32, device=grad_out.device)
            keep = idx >= 0
            rows = torch.arange(B, device=idx.device)[:, None].expand_as(idx)
            flat[rows[keep], idx[keep].long()] = dval[keep]
            d_acts = flat.view(B, L, F).to(act_dtype)
        if bias_dtype is not None and ctx.needs_input_grad[1]:
            d_bias = grad_out.float().sum(dim=1).to(bias_dtype)
        if any(ctx.needs_input_grad[2:]):
            d_w = [g.to(dt) for g, dt in zip(clt_wgrad(idx, val, g16, L, F), w_dtypes)]
        return (d_acts, d_bias, *d_w)


def clt_sparse_decode(acts: torch.Tensor, weights: Sequence[torch.Tensor], bias: torch.Tensor | None = None) -> torch.Tensor:
    """Differentiable fan-out decode. ``acts [..., L, F]`` -> ``[L, ..., d]``."""
    lead = acts.shape[:-2]
    out = CLTSparseDecode.apply(acts.reshape(-1, *acts.shape[-2:]), bias, *weights)
    return out.reshape(out.shape[0], *lead, out.shape[-1])
