"""Top-k with straight-through gradient, and the geometric median.

topk() follows the semantics of utils/math.py:81-171 in the reference project: select over one or several
dimensions jointly, keep selected values (gradient passes through them unchanged), zero the rest, optional
selection by absolute value, optional threshold output.
"""

from __future__ import annotations

import torch


def topk(x: torch.Tensor, k: int, dim: int | tuple[int, ...] = -1, *, return_threshold: bool = False, abs: bool = False):
    dims = (dim,) if isinstance(dim, int) else tuple(dim)
    dims = tuple(d % x.ndim for d in dims)
    keep_dims = tuple(d for d in range(x.ndim) if d not in dims)
    perm = keep_dims + dims
    xp = x.permute(perm)
    lead_shape = xp.shape[: len(keep_dims)]
    tail_shape = xp.shape[len(keep_dims) :]
    flat = xp.reshape(*lead_shape, -1)
    with torch.no_grad():
        score = flat.abs() if abs else flat
        vals, idx = torch.topk(score, k=k, dim=-1, sorted=False)
        mask = torch.zeros_like(flat, dtype=torch.bool).scatter_(-1, idx, True)
        threshold = vals.min(dim=-1).values
    out = (flat * mask.to(flat.dtype)).reshape(*lead_shape, *tail_shape)
    inv = [0] * len(perm)
    for i, p in enumerate(perm):
        inv[p] = i
    out = out.permute(inv)
    return (out, threshold) if return_threshold else out


def compute_geometric_median(x: torch.Tensor, max_iter: int = 1000, tol: float = 1e-5) -> torch.Tensor:
    """Weiszfeld iteration for the point minimising the summed Euclidean distance to the rows of ``x``."""
    y = x.mean(dim=0)
    for _ in range(max_iter):
        dist = (x - y).norm(dim=1).clamp_min(1e-10)
        w = 1.0 / dist
        y_new = (w.unsqueeze(1) * x).sum(0) / w.sum()
        if (y_new - y).norm() < tol:
            return y_new
        y = y_new
    return y
