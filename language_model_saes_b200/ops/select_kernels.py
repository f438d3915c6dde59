"""Selection and compaction on the GPU: batch-level top-k thresholds by radix select, dense rows to padded sparse lists,
and masked row compaction with a dtype cast (kernels of ``csrc/select_ops.cu``), each with a plain-torch oracle.

* ``positive_topk(x, k, dims, group)`` keeps the ``k`` largest positive entries over ``dims`` (mask-multiply, straight-
  through gradient), the batch-level selection of BatchTopK dictionaries (models/sparse_dictionary.py:775-788 of the
  reference project) and of the cross-layer transcoder's ``batchtopk`` / ``batchlayertopk`` (models/clt.py:330-368 there).
  On a GPU the threshold is the exact k-th largest value found by a two-level histogram of the float bit patterns: two
  streaming passes over ``x`` instead of a sort; under feature or data sharding the ranks add their histograms (two
  all-reduces of at most 256 KB) where the reference bisects with one all-reduce per iteration
  (utils/distributed/ops.py:226-250 there). Entries equal to the threshold all pass, so ties keep more than ``k``.
* ``dense_rows_to_sparse`` turns ``[B, N]`` activations into ``(idx, val)`` lists in ascending column order.
* ``compact_rows`` drops masked-out token rows (and casts) in one pass: activation/processors/activation.py:277-285.
"""

from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist

from . import sae_kernels as K

_MAX_SEGMENTS = 64


def ref_positive_threshold(values: torch.Tensor, k: int) -> torch.Tensor:
    """k-th largest positive entry of a flat tensor (fp32 scalar); the smallest positive float if there are fewer."""
    pos = values[values > 0].float()
    if pos.numel() < k or k <= 0:
        return torch.tensor(1e-45, dtype=torch.float32, device=values.device)
    return torch.topk(pos, k).values[-1]


def _kernel_ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in (torch.float32, torch.bfloat16) and x.numel() > 0


@torch.no_grad()
def positive_thresholds(x3: torch.Tensor, k: int, group=None, return_remaining: bool = False, floor: torch.Tensor | None = None):
    """``x3``: contiguous ``[A, S, N]``. Returns fp32 ``[S]``: for every segment ``s`` the k-th largest positive value of
    ``x3[:, s, :]``, taken over the union of all ranks of ``group`` when one is given. ``return_remaining`` (GPU kernels
    only) also returns int64 ``[S]``: how many of the entries equal to the threshold the selection of ``k`` includes.

    ``floor`` (16-bit data, one segment, GPU kernels; fp32 one-element device tensor, the same on every rank): a guess of a
    lower bound of the result, e.g. a fraction of the previous batch's threshold. The histogram pass then counts only
    values of at least ``floor``, which removes nearly all of its shared-memory atomics. The result does not depend on
    the guess: when fewer than ``k`` values reach the floor, a second pass without it runs (decided on the device, the
    host launches both and reads nothing)."""
    A, S, N = x3.shape
    world = dist.get_world_size(group) if group is not None else 1
    if not _kernel_ok(x3):
        out = []
        for s in range(S):
            vals = x3[:, s, :].reshape(-1)
            if world > 1:
                kk = min(k, vals.numel())
                top = torch.topk(vals.float().clamp_min(0), kk).values
                parts = [torch.empty_like(top) for _ in range(world)]
                dist.all_gather(parts, top, group=group)
                vals = torch.cat(parts)
            out.append(ref_positive_threshold(vals, k))
        thr = torch.stack(out)
        if not return_remaining:
            return thr
        above = torch.stack([(x3[:, s, :].float() > thr[s]).sum() for s in range(S)]).to(torch.int64)
        if world > 1:
            dist.all_reduce(above, group=group)
        return thr, (k - above).clamp(min=0)
    ext = K._ext()
    dev = x3.device
    nhi = int(ext.radix_hi_bins())
    hist_hi = torch.empty(nhi, dtype=torch.int32, device=dev)
    hist_lo = torch.empty(65536, dtype=torch.int32, device=dev)
    sel0 = torch.zeros(4, dtype=torch.int64, device=dev)
    sel1 = torch.zeros(4, dtype=torch.int64, device=dev)
    thr = torch.empty(S, dtype=torch.float32, device=dev)
    remaining = torch.zeros(S, dtype=torch.int64, device=dev)
    half = x3.dtype == torch.bfloat16  # 16-bit data: the first level already resolves the value
    floored = floor is not None and half and S == 1
    for s in range(S):
        hist_hi.zero_()
        ext.radix_hist(x3, A, S, N, s, 0, None, hist_hi, floor.reshape(1).float() if floored else None, None)
        if world > 1:
            dist.all_reduce(hist_hi, group=group)
        ext.radix_pick(hist_hi, nhi, int(k), None, 0, sel0, thr[s : s + 1] if half else None, None)
        if floored:  # the repeat without the floor: both kernels return at once unless sel0[3] says the floor was too high
            hist_hi.zero_()
            ext.radix_hist(x3, A, S, N, s, 0, None, hist_hi, None, sel0)
            if world > 1:
                dist.all_reduce(hist_hi, group=group)
            ext.radix_pick(hist_hi, nhi, int(k), None, 0, sel0, thr[s : s + 1], sel0)
        if not half:
            hist_lo.zero_()
            ext.radix_hist(x3, A, S, N, s, 1, sel0, hist_lo, None, None)
            if world > 1:
                dist.all_reduce(hist_lo, group=group)
            ext.radix_pick(hist_lo, 65536, 0, sel0, 1, sel1, thr[s : s + 1], None)
        remaining[s : s + 1].copy_((sel0 if half else sel1)[1:2])
    return (thr, remaining) if return_remaining else thr


def _middle_block(ndim: int, dims: Sequence[int]) -> tuple[int, int] | None:
    """The kept dimensions must be one contiguous block ``[i, j)`` (possibly empty, anywhere): returns ``(i, j)``."""
    sel = sorted(d % ndim for d in dims)
    keep = [d for d in range(ndim) if d not in sel]
    if not keep:
        return (0, 0)
    if keep != list(range(keep[0], keep[-1] + 1)):
        return None
    return keep[0], keep[-1] + 1


def positive_topk(x: torch.Tensor, k: int, dims: Sequence[int], group=None) -> torch.Tensor | None:
    """``x * mask`` where ``mask`` marks the ``k`` largest positive entries over ``dims`` (separately for every index of
    the other dimensions). Returns None when the layout is not one this path handles (callers then use the sort-based
    implementation): the kept dimensions must be adjacent, with at most 64 index combinations, and the last dimension
    must be selected over."""
    blk = _middle_block(x.ndim, dims)
    if blk is None or not _kernel_ok(x) or (x.ndim - 1) not in {d % x.ndim for d in dims}:
        return None
    i, j = blk
    S = 1
    for s_ in x.shape[i:j]:
        S *= s_
    if S > _MAX_SEGMENTS:
        return None
    xc = x.contiguous()
    A = 1
    for a_ in x.shape[:i]:
        A *= a_
    N = xc.numel() // (A * S)
    thr = positive_thresholds(xc.detach().view(A, S, N), k, group)
    return _ThresholdMask.apply(xc, thr, A, S, N)


class _ThresholdMask(torch.autograd.Function):
    """``where(x >= thr[segment], x, 0)`` in one streaming pass; the gradient passes where the output is non-zero."""

    @staticmethod
    def forward(ctx, x, thr, A, S, N):
        out = K._ext().threshold_mask(x.detach(), thr, A, S, N)
        ctx.save_for_backward(out)
        return out

    @staticmethod
    def backward(ctx, grad):
        (out,) = ctx.saved_tensors
        return grad * (out != 0).to(grad.dtype), None, None, None, None


# ---- dense rows -> padded sparse ---------------------------------------------------------------------
def ref_dense_rows_to_sparse(acts: torch.Tensor, cap: int) -> tuple[torch.Tensor, torch.Tensor]:
    B, N = acts.shape
    idx = torch.full((B, cap), -1, dtype=torch.int32, device=acts.device)
    val = torch.zeros(B, cap, dtype=torch.float32, device=acts.device)
    for b in range(B):
        cols = torch.nonzero(acts[b], as_tuple=False).flatten()[:cap]
        idx[b, : cols.numel()] = cols.to(torch.int32)
        val[b, : cols.numel()] = acts[b, cols].float()
    return idx, val


@torch.no_grad()
def dense_rows_to_sparse(acts: torch.Tensor, cap: int | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """``[B, N]`` -> ``(idx int32 [B, cap], val fp32 [B, cap])``, ascending columns, ``-1`` / ``0`` padding. ``cap`` None:
    the largest row count, rounded up to a multiple of 8 (costs a counting pass and one host read)."""
    assert acts.ndim == 2
    if not _kernel_ok(acts):
        if cap is None:
            cap = max(8, -(-int((acts != 0).sum(-1).max()) // 8) * 8) if acts.numel() else 8
        return ref_dense_rows_to_sparse(acts, cap)
    acts = acts.contiguous()
    ext = K._ext()
    B = acts.shape[0]
    nnz = torch.empty(B, dtype=torch.int32, device=acts.device)
    seg = None
    if cap is None:
        seg = torch.empty(B, 8, 2, dtype=torch.int32, device=acts.device)  # the counting pass leaves them for the compaction
        ext.row_compact(acts, None, None, nnz, None, None, None, None, None, seg)
        cap = max(8, -(-int(nnz.max()) // 8) * 8)
    idx = torch.empty(B, cap, dtype=torch.int32, device=acts.device)
    val = torch.empty(B, cap, dtype=torch.float32, device=acts.device)
    ext.row_compact(acts, idx, val, nnz, None, None, None, None, None, seg)
    return idx, val


@torch.no_grad()
def threshold_rows_to_sparse(g: torch.Tensor, thr: torch.Tensor, col_div: torch.Tensor | None = None, width_group=None,
                             n_ties: torch.Tensor | None = None, tie_group=None, cap: int | None = None,
                             overflow: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:  # fmt: skip
    """Entries of ``g [B, N]`` that reach the (positive) threshold ``thr`` (one-element fp32 tensor) as padded sparse lists,
    values divided by ``col_div[column]`` when given: the codes of a batch-level top-k straight from the gated
    pre-activations, without a masked dense tensor in between.

    ``n_ties`` (one-element integer tensor: how many entries EQUAL to the threshold belong to the selection, as
    ``positive_thresholds(..., return_remaining=True)`` reports it) makes the number of codes exact when the threshold
    value repeats (16-bit data): ties are granted in (rank of ``tie_group``, row, column) order until the count is
    used up. Without it every tie is kept.

    ``cap``: fixed list width (a multiple of 8). Without it the width is the widest row's count, which costs one host
    read per call; with it nothing is read back: a row with more than ``cap`` selected entries keeps its first ``cap``
    (ascending column) and the number of such rows is added to ``overflow`` (one-element integer device tensor) for
    the caller to look at when it next synchronises anyway."""
    if not _kernel_ok(g):
        return _ref_threshold_rows_to_sparse(g, thr, col_div, width_group, n_ties, tie_group, cap, overflow)
    ext = K._ext()
    g = g.contiguous()
    B = g.shape[0]
    nnz = torch.empty(B, dtype=torch.int32, device=g.device)
    quota = seg = None
    if n_ties is None:
        if cap is None:
            ext.row_compact(g, None, None, nnz, thr, None, None, None, None, None)
            widest = nnz.max()
    else:
        ties = torch.empty(B, dtype=torch.int32, device=g.device)
        seg = torch.empty(B, 8, 2, dtype=torch.int32, device=g.device)  # per warp segment: the compaction pass starts from them
        ext.row_compact(g, None, None, nnz, thr, None, ties, None, None, seg)
        budget = n_ties.reshape(()).to(torch.int64)
        if tie_group is not None and dist.get_world_size(tie_group) > 1:
            mine = ties.sum(dtype=torch.int64).reshape(1)
            every = [torch.empty_like(mine) for _ in range(dist.get_world_size(tie_group))]
            dist.all_gather(every, mine, group=tie_group)
            budget = budget - torch.cat(every)[: dist.get_rank(tie_group)].sum()  # earlier ranks are served first
        before = torch.cumsum(ties, 0, dtype=torch.int64) - ties
        quota = (budget - before).clamp(min=0).minimum(ties.to(torch.int64)).to(torch.int32)
        if cap is None:
            widest = (nnz + quota).max()
    if cap is None:
        if width_group is not None and dist.get_world_size(width_group) > 1:
            dist.all_reduce(widest, op=dist.ReduceOp.MAX, group=width_group)  # ranks that exchange their lists need one width
        cap = max(8, -(-int(widest) // 8) * 8)
    assert cap % 8 == 0 and cap > 0
    idx = torch.empty(B, cap, dtype=torch.int32, device=g.device)
    val = torch.empty(B, cap, dtype=torch.float32, device=g.device)
    ext.row_compact(g, idx, val, nnz, thr, col_div, None, quota, None, seg)  # nnz: the row's full count, also beyond the list width
    if overflow is not None:
        overflow += (nnz > cap).sum()
    return idx, val


@torch.no_grad()
def column_threshold_rows_to_sparse(x: torch.Tensor, col_thr: torch.Tensor, cap: int,
                                    overflow: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Entries of ``x [B, N]`` above their column's threshold ``col_thr [N]`` as padded sparse lists of fixed width ``cap``
    (ascending columns, values unchanged): the JumpReLU selection of pre-activations against per-feature thresholds. Rows
    with more than ``cap`` such entries keep the first ones and are counted in ``overflow``."""
    assert x.ndim == 2 and cap % 8 == 0 and cap > 0
    B = x.shape[0]
    if not _kernel_ok(x):
        keep = x.float() > col_thr.float()
        if overflow is not None:
            overflow += (keep.sum(-1) > cap).sum()
        idx = torch.full((B, cap), -1, dtype=torch.int32, device=x.device)
        val = torch.zeros(B, cap, dtype=torch.float32, device=x.device)
        for b in range(B):
            cols = torch.nonzero(keep[b], as_tuple=False).flatten()[:cap]
            idx[b, : cols.numel()] = cols.to(torch.int32)
            val[b, : cols.numel()] = x[b, cols].float()
        return idx, val
    x = x.contiguous()
    idx = torch.empty(B, cap, dtype=torch.int32, device=x.device)
    val = torch.empty(B, cap, dtype=torch.float32, device=x.device)
    nnz = torch.empty(B, dtype=torch.int32, device=x.device)
    K._ext().row_compact(x, idx, val, nnz, None, None, None, None, col_thr.float().contiguous(), None)
    if overflow is not None:
        overflow += (nnz > cap).sum()
    return idx, val


def jumprelu_window_grad(G: torch.Tensor, S: torch.Tensor, n: torch.Tensor, theta: torch.Tensor, window: float,
                         dtheta: torch.Tensor, add_per_hit: float = 0.0) -> None:
    """``dtheta[f] += sum_b (G[b, f] / n[f] + add_per_hit) * (-theta[f] / window) * 1[|S n - theta| < window / 2 and S n > 0]``:
    the JumpReLU threshold gradient of a head from the dense reconstruction gradient ``G`` and the summed pre-activations
    ``S`` (both ``[B, F]`` bf16 on the GPU); ``add_per_hit`` is a loss derivative that is the same at every entry."""
    if not (G.is_cuda and G.dtype == torch.bfloat16 and S.dtype == torch.bfloat16 and G.shape[1] % 8 == 0):
        x = S.float() * n
        hit = ((x - theta).abs() < 0.5 * window) & (x > 0)
        total = torch.where(hit, G.float(), torch.zeros((), device=G.device)).sum(0) / n + add_per_hit * hit.sum(0)
        dtheta += total * (-theta / window)
        return
    K._ext().jumprelu_window_grad(G.contiguous(), S.contiguous(), n.contiguous(), theta.contiguous(), float(window),
                                  float(add_per_hit), dtheta)


def _ref_threshold_rows_to_sparse(g, thr, col_div, width_group, n_ties, tie_group, cap=None, overflow=None):
    """Plain-torch statement of ``threshold_rows_to_sparse`` (any device): same selection, same order."""
    gf = g.float()
    t = thr.reshape(()).float()
    keep = gf > t
    ties = gf == t
    if n_ties is None:
        keep = keep | ties
    else:
        budget = n_ties.reshape(()).to(torch.int64)
        if tie_group is not None and dist.get_world_size(tie_group) > 1:
            mine = ties.sum().to(torch.int64).reshape(1)
            every = [torch.empty_like(mine) for _ in range(dist.get_world_size(tie_group))]
            dist.all_gather(every, mine, group=tie_group)
            budget = budget - torch.cat(every)[: dist.get_rank(tie_group)].sum()
        rank_of_tie = torch.cumsum(ties.reshape(-1).to(torch.int64), 0).reshape(ties.shape) - 1  # row-major order
        keep = keep | (ties & (rank_of_tie < budget))
    if cap is None:
        widest = keep.sum(-1).max()
        if width_group is not None and dist.get_world_size(width_group) > 1:
            dist.all_reduce(widest, op=dist.ReduceOp.MAX, group=width_group)
        cap = max(8, -(-int(widest) // 8) * 8)
    elif overflow is not None:
        overflow += (keep.sum(-1) > cap).sum()
    vals = gf / col_div.float() if col_div is not None else gf
    B = g.shape[0]
    idx = torch.full((B, cap), -1, dtype=torch.int32, device=g.device)
    val = torch.zeros(B, cap, dtype=torch.float32, device=g.device)
    for b in range(B):
        cols = torch.nonzero(keep[b], as_tuple=False).flatten()[:cap]
        idx[b, : cols.numel()] = cols.to(torch.int32)
        val[b, : cols.numel()] = vals[b, cols]
    return idx, val


# ---- masked row compaction ---------------------------------------------------------------------------
@torch.no_grad()
def compact_rows(src: torch.Tensor, keep: torch.Tensor, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """Rows of ``src [n, d]`` whose ``keep [n]`` entry is set, in order, cast to ``out_dtype``."""
    out_dtype = out_dtype or src.dtype
    ok = (
        _kernel_ok(src) and src.ndim == 2 and src.shape[1] % 8 == 0 and out_dtype in (torch.float32, torch.bfloat16)
        and src.shape[0] < 2**31 - 1
    )  # fmt: skip
    if not ok:
        return src[keep.bool()].to(out_dtype)
    ext = K._ext()
    n = src.shape[0]
    keep32 = keep.to(torch.int32).contiguous()
    pos = torch.empty(n + 1, dtype=torch.int32, device=src.device)
    sums = torch.empty((n + 4095) // 4096, dtype=torch.int32, device=src.device)
    ext.exclusive_scan(keep32, pos, sums)
    m = int(pos[n])
    out = torch.empty(m, src.shape[1], dtype=out_dtype, device=src.device)
    ext.gather_rows_cast(src.contiguous(), keep32, pos, out)
    return out
