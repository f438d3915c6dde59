"""Autograd entry points to the sparse sm_100a kernels for the generic (autograd) training path.

Same role as the two ``torch.autograd.Function`` classes around the Triton kernels of the reference project
(kernels/kernels.py:228-325 and kernels/entrypoints.py:16-90): when the activations are sparse enough, decode with a
gather-GEMM over the non-zeros instead of a dense ``[batch, F] x [F, d]`` product, and form the weight gradient from the
non-zeros only. Here the kernels are the ones of the fused step: ``sparse_decode`` (forward), ``sparse_dact`` (gradient
of the activations) and the gradient-row rebuild of ``sparse_grad_adam`` with its dense output enabled (gradient of
the decoder), all on bf16 operands with fp32 accumulation.
"""

from __future__ import annotations

import torch

from . import sae_kernels as K


def dense_to_padded_sparse(acts: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``[B, F]`` -> ``(idx int32 [B, kmax], val fp32 [B, kmax])`` holding every non-zero of each row (``idx = -1`` in
    the padding), ``kmax`` = largest number of non-zeros in a row, rounded up to a multiple of 8."""
    if acts.is_cuda and acts.dtype in (torch.float32, torch.bfloat16):
        from .select_kernels import dense_rows_to_sparse  # one counting pass + one ordered compaction pass

        return dense_rows_to_sparse(acts)
    nz = acts != 0
    kmax = max(8, -(-int(nz.sum(dim=-1).max()) // 8) * 8)
    kmax = min(kmax, acts.shape[-1])
    score, idx = nz.to(torch.float32).topk(kmax, dim=-1)  # picks the non-zeros first (any order)
    val = torch.gather(acts, -1, idx).float()
    keep = score > 0
    return torch.where(keep, idx, torch.full_like(idx, -1)).to(torch.int32), torch.where(keep, val, torch.zeros_like(val))


class SparseDecode(torch.autograd.Function):
    """``acts [B, F] @ W_D [F, d]`` for sparse ``acts``; gradients for both."""

    @staticmethod
    def forward(ctx, acts: torch.Tensor, W_D: torch.Tensor) -> torch.Tensor:
        idx, val = dense_to_padded_sparse(acts.detach())
        W16 = W_D.detach().to(torch.bfloat16).contiguous()
        out = K.sparse_decode(idx, val, W16, None, torch.float32)
        ctx.save_for_backward(idx, val, W16)
        ctx.shape = acts.shape
        ctx.dtypes = (acts.dtype, W_D.dtype)
        return out.to(acts.dtype if acts.dtype != torch.float32 else torch.float32)

    @staticmethod
    def backward(ctx, grad_out: torch.Tensor):
        idx, val, W16 = ctx.saved_tensors
        B, F = ctx.shape
        g16 = grad_out.to(torch.bfloat16).contiguous()
        d_acts = d_W = None
        if ctx.needs_input_grad[0]:
            dval = K.sparse_dact(idx, W16, g16)
            d_acts = torch.zeros(B, F, dtype=torch.float32, device=grad_out.device)
            rows = torch.arange(B, device=idx.device)[:, None].expand_as(idx)
            keep = idx >= 0
            d_acts[rows[keep], idx[keep].long()] = dval[keep]
            d_acts = d_acts.to(ctx.dtypes[0])
        if ctx.needs_input_grad[1]:
            d_W = sparse_decoder_grad(idx, val, g16, F)
            d_W = d_W.to(ctx.dtypes[1])
        return d_acts, d_W


def sparse_decoder_grad(idx: torch.Tensor, val: torch.Tensor, grad_out_bf16: torch.Tensor, F: int) -> torch.Tensor:
    """``dW_D[f, :] = sum over the non-zeros (b, j) with idx[b, j] == f of val[b, j] * grad_out[b, :]`` as dense fp32
    ``[F, d]``: counting sort by feature, then one CTA per feature row rebuilds its gradient row (no atomics)."""
    d = grad_out_bf16.shape[1]
    if not grad_out_bf16.is_cuda:
        return K.ref_sparse_grads(idx.long(), val, torch.zeros_like(val), grad_out_bf16, grad_out_bf16, F)[0]
    groups = K.FeatureGroups(F, idx.numel(), idx.device)
    groups.build(idx)
    out = torch.empty(F, d, dtype=torch.float32, device=idx.device)
    none16 = torch.empty(0, dtype=torch.bfloat16, device=idx.device)  # no parameter, state or shadow is touched:
    K.sparse_grad_adam(groups, val, torch.zeros_like(val), grad_out_bf16, grad_out_bf16, out, out, out, none16, out, out, out,
                       none16, None, None, None, None, None, None, 0.0, 0.9, 0.999, 1e-8, 1, update=False,
                       grad_out=(out, None))  # fmt: skip  (update is off; `out` only stands in for the shape checks)
    return out


def sparse_decode(acts: torch.Tensor, W_D: torch.Tensor) -> torch.Tensor:
    """Differentiable ``acts @ W_D`` through the sparse kernels (2-D ``acts``; other shapes are flattened)."""
    lead = acts.shape[:-1]
    out = SparseDecode.apply(acts.reshape(-1, acts.shape[-1]), W_D)
    return out.reshape(*lead, W_D.shape[1])
