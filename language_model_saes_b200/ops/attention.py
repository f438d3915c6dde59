"""Causal attention whose value width differs from the query/key width, on the sm_100a tensor cores.

A low-rank sparse attention dictionary runs one attention per QK head with the head's whole OV group as the value
(models/lorsa.py:642-661,864-904 of the reference project, which calls ``scaled_dot_product_attention``): ``q, k`` are
``[batch, seq, heads, d_qk]`` and ``v`` is ``[batch, seq, heads, d_v]`` with ``d_v`` a multiple of ``d_qk`` or unrelated
to it. ``csrc/attention.cu`` implements the forward pass with tcgen05 MMAs, accumulators in TMEM and TMA-fed operands;
``ref_causal_attention`` is the plain-torch oracle.
"""

from __future__ import annotations

import math

import torch

from . import sae_kernels as K


def library_attention_backends():
    """Context in which ``scaled_dot_product_attention`` may pick its memory-efficient or its plain backend only.

    A value width that differs from the query/key width rules the flash backend out, and the library then prefers its
    cuDNN backend on this architecture. With torch 2.11 / cuDNN 9 on sm_100 that backend's BACKWARD pass returned input
    gradients that depended on what the allocator's recycled memory held: correct in a fresh process, unrelated to the
    true gradient (cosine near 0) or NaN once freed blocks had been filled with a NaN pattern, for several stride layouts
    of the output gradient and at both a tiny and a training-size shape; its forward pass and both passes of the
    memory-efficient backend were correct in every such run. The backward pass follows the forward's choice, so the
    context is only needed around the forward call."""
    from torch.nn.attention import SDPBackend, sdpa_kernel

    return sdpa_kernel([SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH])


def ref_causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``(out [b, s, h, dv], lse [b, h, s])``."""
    s = q.shape[1]
    scores = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    mask = torch.ones(s, s, dtype=torch.bool, device=q.device).tril()
    scores = scores.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)
    out = torch.einsum("bhqk,bkhg->bqhg", torch.softmax(scores, dim=-1), v.float())
    return out, lse


def supported(q: torch.Tensor, v: torch.Tensor) -> bool:
    return (
        q.is_cuda and q.ndim == 4 and v.ndim == 4 and q.shape[-1] in (64, 128) and v.shape[-1] % 64 == 0
        and q.shape[1] % 8 == 0 and q.shape[0] <= 65535
    )  # fmt: skip


@torch.no_grad()
def causal_attention_fwd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None,
                         want_lse: bool = False) -> tuple[torch.Tensor, torch.Tensor | None]:  # fmt: skip
    """``q, k [b, s, h, d_qk]``, ``v [b, s, h, d_v]`` -> bf16 ``out [b, s, h, d_v]`` (and fp32 ``lse [b, h, s]``)."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    if not supported(q, v):
        out, lse = ref_causal_attention(q, k, v, scale)
        return out.to(torch.bfloat16), (lse if want_lse else None)
    b, s, h, _ = q.shape
    q16, k16 = q.to(torch.bfloat16).contiguous(), k.to(torch.bfloat16).contiguous()
    vt = v.to(torch.bfloat16).permute(0, 2, 3, 1).contiguous()  # [b, h, d_v, s]: keys contiguous for the P V product
    out = torch.empty(b, s, h, v.shape[-1], dtype=torch.bfloat16, device=q.device)
    lse = torch.empty(b, h, s, dtype=torch.float32, device=q.device) if want_lse else None
    K._ext().attn_fwd(q16, k16, vt, out, lse, float(scale), K.status_buffer(q.device))
    return out, lse


class CausalAttention(torch.autograd.Function):
    """Differentiable ``causal_attention_fwd``: three tcgen05 kernels (forward, dQ, dK/dV). Inputs of any float dtype are
    rounded to bf16 for the tensor cores; gradients are accumulated in fp32 and returned in the inputs' dtypes."""

    @staticmethod
    def forward(ctx, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, v_is_transposed: bool = False) -> torch.Tensor:
        q16, k16 = (t.detach().to(torch.bfloat16).contiguous() for t in (q, k))
        b, s, h, _ = q16.shape
        if v_is_transposed:  # the caller produced V^T [b, h, d_v, s] directly (no transpose pass in the forward)
            vt = v.detach().to(torch.bfloat16).contiguous()
            v16 = vt.permute(0, 3, 1, 2).contiguous()  # the backward kernels read V rows ([b, s, h, d_v])
        else:
            v16 = v.detach().to(torch.bfloat16).contiguous()
            vt = v16.permute(0, 2, 3, 1).contiguous()
        ctx.v_is_transposed = v_is_transposed
        out = torch.empty(b, s, h, v16.shape[-1], dtype=torch.bfloat16, device=q.device)
        lse = torch.empty(b, h, s, dtype=torch.float32, device=q.device)
        K._ext().attn_fwd(q16, k16, vt, out, lse, float(scale), K.status_buffer(q.device))
        ctx.save_for_backward(q16, k16, v16, out, lse)
        ctx.scale, ctx.dtypes = float(scale), (q.dtype, k.dtype, v.dtype)
        return out.to(v.dtype)

    @staticmethod
    def backward(ctx, dout: torch.Tensor):
        q16, k16, v16, out, lse = ctx.saved_tensors
        do16 = dout.to(torch.bfloat16).contiguous()
        delta = (do16.float() * out.float()).sum(dim=-1).permute(0, 2, 1).contiguous()  # [b, h, s]
        qt = q16.permute(0, 2, 3, 1).contiguous()
        kt = k16.permute(0, 2, 3, 1).contiguous()
        dot = do16.permute(0, 2, 3, 1).contiguous()
        dq = torch.empty(q16.shape, dtype=torch.float32, device=q16.device)
        dk = torch.empty_like(dq)
        dv = torch.empty(v16.shape, dtype=torch.float32, device=q16.device)
        ext = K._ext()
        ext.launches += 1  # two kernels in one entry point
        ext.attn_bwd(q16, k16, v16, do16, qt, kt, dot, lse, delta, dq, dk, dv, ctx.scale, K.status_buffer(q16.device))
        if ctx.v_is_transposed:
            dv = dv.permute(0, 2, 3, 1)
        return dq.to(ctx.dtypes[0]), dk.to(ctx.dtypes[1]), dv.to(ctx.dtypes[2]), None, None


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor | None = None, scale: float | None = None,
                     vt: torch.Tensor | None = None) -> torch.Tensor:  # fmt: skip
    """Differentiable causal attention ``[b, s, h, d_qk] x [b, s, h, d_v] -> [b, s, h, d_v]``; the tensor-core kernels
    when the shape is supported on a GPU, the torch oracle otherwise. The values may be given transposed instead, as
    ``vt [b, h, d_v, s]`` (what the forward kernel reads), which saves a transpose pass when the caller can produce
    that layout directly."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    if vt is not None:
        if supported(q, vt.permute(0, 3, 1, 2)):
            return CausalAttention.apply(q, k, vt, scale, True)
        v = vt.permute(0, 3, 1, 2)
    if not supported(q, v):
        return ref_causal_attention(q, k, v, scale)[0].to(v.dtype)
    return CausalAttention.apply(q, k, v, scale)
