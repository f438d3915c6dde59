"""Sparse decode of a mixture of linear transforms (MOLT) through the gather kernels of the sparse-dictionary steps.

The model's decode is ``out_b = sum_c a_bc U_c (V_c x_b)`` over transforms ``c`` of rank ``r`` (``U_c [d, r]``,
``V_c [r, d]``; models/molt.py:543-589 of the reference project, which runs it as two dense products over ALL
transforms of a rank group and multiplies by the sparse gate ``a`` in between: ``2 * 2 * B * n * r * d`` FLOPs). With a
sparse gate only the active (token, transform) pairs matter. Writing transform ``c`` as ``r`` rank-1 features
``(c, j)`` with encoder rows ``V_c[j, :]`` and decoder rows ``U_c[:, j]``:

    t_b,(c,j)  = V_c[j, :] . x_b                    a batched dot product over the active pairs   (``sparse_dact``)
    out_b      = sum_(c,j) (a_bc t_b,(c,j)) U_c[:, j]   a sparse decode over the expanded codes      (``sparse_decode``)

and the backward pass is the same two kernels with the roles of ``U`` and ``V`` swapped, plus the by-feature gradient
rows of ``sparse_grad_adam`` (its dense-output mode) for ``dU`` and ``dV``. Cost: ``~8 * B * L0 * r * d`` FLOPs of
gathers instead of the dense products. Operands are rounded to bf16 (fp32 accumulation), as under autocast.

Opt-in: ``MOLTConfig.use_triton_kernel`` (the reference's name for "use the sparse kernels"). The CPU runs the torch
statements of the same kernels.
"""

from __future__ import annotations

import torch

from . import sae_kernels as K
from .sparse_autograd import dense_to_padded_sparse, sparse_decoder_grad

_MAX_CODES = 8192  # codes per row and launch: the decode kernel stages a row's codes in shared memory


def _expand(idx: torch.Tensor, r: int) -> torch.Tensor:
    """Transform indices ``[B, K]`` (-1 = empty) -> indices of their ``r`` rank-1 features ``[B, K * r]``."""
    j = torch.arange(r, device=idx.device, dtype=idx.dtype)
    e = idx.unsqueeze(-1) * r + j
    return torch.where(idx.unsqueeze(-1) >= 0, e, torch.full_like(e, -1)).reshape(idx.shape[0], -1)


def _chunks(n: int):
    for lo in range(0, n, _MAX_CODES):
        yield slice(lo, min(n, lo + _MAX_CODES))


def _dots(idx_e: torch.Tensor, rows16: torch.Tensor, vec16: torch.Tensor) -> torch.Tensor:
    """``rows16[idx_e[b, q]] . vec16[b]`` for every code (0 at empty slots)."""
    return torch.cat([K.sparse_dact(idx_e[:, s].contiguous(), rows16, vec16) for s in _chunks(idx_e.shape[1])], dim=1)


def _decode(idx_e: torch.Tensor, vals: torch.Tensor, rows16: torch.Tensor) -> torch.Tensor:
    out = None
    for s in _chunks(idx_e.shape[1]):
        part = K.sparse_decode(idx_e[:, s].contiguous(), vals[:, s].contiguous(), rows16, None, torch.float32)
        out = part if out is None else out + part
    return out


class MoltGroupDecode(torch.autograd.Function):
    """``sum_c acts[b, c] U[c] (V[c] x[b])`` for one rank group: ``acts [B, n]`` (sparse), ``x [B, d]``, ``U [n, d, r]``,
    ``V [n, r, d]`` -> ``[B, d]`` fp32; gradients for all four."""

    @staticmethod
    def forward(ctx, acts: torch.Tensor, x: torch.Tensor, U: torch.Tensor, V: torch.Tensor) -> torch.Tensor:
        n, d, r = U.shape
        idx, val = dense_to_padded_sparse(acts.detach())
        idx_e = _expand(idx, r)
        x16 = x.detach().to(torch.bfloat16).contiguous()
        V16 = V.detach().to(torch.bfloat16).reshape(n * r, d).contiguous()  # row (c, j) = V[c, j, :]
        U16 = U.detach().to(torch.bfloat16).permute(0, 2, 1).reshape(n * r, d).contiguous()  # row (c, j) = U[c, :, j]
        t = _dots(idx_e, V16, x16)  # [B, K r]
        a_rep = val.repeat_interleave(r, dim=1)
        out = _decode(idx_e, a_rep * t, U16)
        ctx.save_for_backward(idx, idx_e, a_rep, t, x16, U16, V16)
        ctx.shape = (acts.shape, n, d, r)
        ctx.dtypes = (acts.dtype, x.dtype, U.dtype, V.dtype)
        return out

    @staticmethod
    def backward(ctx, grad_out: torch.Tensor):
        idx, idx_e, a_rep, t, x16, U16, V16 = ctx.saved_tensors
        (B, n_feat), n, d, r = ctx.shape
        g16 = grad_out.to(torch.bfloat16).contiguous()
        dvals = _dots(idx_e, U16, g16)  # d out / d (a t) at every code
        d_acts = d_x = d_U = d_V = None
        dt = dvals * a_rep
        if ctx.needs_input_grad[0]:
            da = (dvals * t).view(B, -1, r).sum(-1)  # [B, K]
            d_acts = torch.zeros(B, n_feat + 1, dtype=torch.float32, device=grad_out.device)
            d_acts.scatter_(1, torch.where(idx >= 0, idx, torch.full_like(idx, n_feat)).long(), da)
            d_acts = d_acts[:, :n_feat].to(ctx.dtypes[0])
        if ctx.needs_input_grad[1]:
            d_x = _decode(idx_e, dt, V16).to(ctx.dtypes[1])
        if ctx.needs_input_grad[2]:
            rows = sum(sparse_decoder_grad(idx_e[:, s].contiguous(), (a_rep * t)[:, s].contiguous(), g16, n * r) for s in _chunks(idx_e.shape[1]))
            d_U = rows.view(n, r, d).permute(0, 2, 1).to(ctx.dtypes[2])
        if ctx.needs_input_grad[3]:
            rows = sum(sparse_decoder_grad(idx_e[:, s].contiguous(), dt[:, s].contiguous(), x16, n * r) for s in _chunks(idx_e.shape[1]))
            d_V = rows.view(n, r, d).to(ctx.dtypes[3])
        return d_acts, d_x, d_U, d_V


def molt_group_decode(acts: torch.Tensor, x: torch.Tensor, U: torch.Tensor, V: torch.Tensor) -> torch.Tensor:
    """Differentiable sparse decode of one rank group; leading dimensions of ``acts`` / ``x`` are flattened."""
    lead = x.shape[:-1]
    out = MoltGroupDecode.apply(acts.reshape(-1, acts.shape[-1]), x.reshape(-1, x.shape[-1]), U, V)
    return out.reshape(*lead, U.shape[1])
