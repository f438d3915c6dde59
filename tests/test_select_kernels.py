"""Radix-select thresholds, dense-to-sparse row compaction and masked row compaction against plain torch."""

import math

import pytest
import torch

from language_model_saes_b200.ops import select_kernels as S
from language_model_saes_b200.utils.math import topk


def test_positive_threshold_oracle_and_layout_rule_cpu():
    x = torch.tensor([0.5, -1.0, 3.0, 0.0, 2.0, 2.0])
    assert S.ref_positive_threshold(x, 2) == 2.0 and S.ref_positive_threshold(x, 1) == 3.0
    assert 0 < S.ref_positive_threshold(x, 10) < 1e-30  # fewer than k positive values: everything positive passes
    thr = S.positive_thresholds(torch.tensor([[[1.0, 4.0], [2.0, 0.0]], [[3.0, -1.0], [5.0, 6.0]]]), 2)
    assert thr.tolist() == [3.0, 5.0]  # segment s covers x[:, s, :]
    assert S._middle_block(3, (0, 2)) == (1, 2) and S._middle_block(3, (0, 1, 2)) == (0, 0) and S._middle_block(4, (0, 1, 3)) == (2, 3)
    assert S._middle_block(4, (1, 3)) is None  # kept dims 0 and 2 are not adjacent
    assert S.positive_topk(torch.rand(4, 4), 3, (0, 1)) is None  # CPU tensors take the sort-based path of the callers


def test_compaction_oracles_cpu():
    a = torch.tensor([[0.0, 2.0, 0.0, 3.0], [0.0, 0.0, 0.0, 0.0], [1.0, 1.0, 1.0, 1.0]])
    idx, val = S.dense_rows_to_sparse(a)
    assert idx.shape == (3, 8) and idx[0, :3].tolist() == [1, 3, -1] and val[0, :2].tolist() == [2.0, 3.0]
    assert idx[1].eq(-1).all() and idx[2, :4].tolist() == [0, 1, 2, 3]
    src = torch.arange(12.0).view(4, 3)
    out = S.compact_rows(src, torch.tensor([True, False, True, True]), torch.bfloat16)
    assert out.dtype == torch.bfloat16 and torch.equal(out.float(), src[[0, 2, 3]])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,dims,k", [((256, 4096), (0, 1), 256 * 32), ((64, 3, 1000), (0, 2), 64 * 7), ((8, 16, 2, 515), (0, 1, 3), 900),
                                         ((33, 777), (0, 1), 1), ((16, 64), (0, 1), 5000)])  # fmt: skip
def test_radix_threshold_matches_sort(dtype, shape, dims, k):
    torch.manual_seed(0)
    x = torch.randn(*shape, device="cuda").to(dtype)
    x = x * (x > 0)
    got = S.positive_topk(x, k, dims)
    assert got is not None
    n_sel = 1
    for d_ in dims:
        n_sel *= shape[d_]
    want = topk(x.float(), k=min(k, n_sel), dim=dims)
    if dtype == torch.float32 and k <= n_sel // 2:
        assert torch.equal(got, want)  # continuous data: no ties, the selections coincide exactly
    else:
        # ties at the threshold (bf16 data repeats values) keep a few more than k; everything above the threshold agrees
        kept, ref_kept = got != 0, want != 0
        assert (ref_kept & ~kept).sum() == 0
        extra = kept & ~ref_kept
        if extra.any():
            i, j = S._middle_block(x.ndim, dims)
            A = math.prod(shape[:i])
            thr = S.positive_thresholds(x.contiguous().view(A, math.prod(shape[i:j]), -1), k)
            vshape = [shape[d_] if i <= d_ < j else 1 for d_ in range(x.ndim)]
            assert torch.equal(got[extra].float(), thr.view(vshape).expand(shape)[extra])  # the extras are ties


@pytest.mark.gpu
def test_radix_threshold_exact_value_fp32():
    torch.manual_seed(1)
    x = torch.rand(1 << 22, device="cuda") * torch.logspace(-6, 3, 1 << 22, device="cuda")
    x[::3] = 0
    for k in (1, 17, 100000, 1 << 20):
        thr = S.positive_thresholds(x.view(1, 1, -1), k)
        assert thr.item() == torch.topk(x, k).values[-1].item()


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(512, 8192), (37, 1003)])
def test_radix_threshold_with_a_floor_guess_does_not_depend_on_the_guess(shape):
    """16-bit data: a floor below the result skips most of the histogram, a floor above it triggers the repeat without a
    floor on the device; threshold and tie count equal the plain call's either way."""
    torch.manual_seed(2)
    x = torch.randn(*shape, device="cuda").to(torch.bfloat16).contiguous()
    k = shape[0] * 12
    thr0, rem0 = S.positive_thresholds(x.view(1, 1, -1), k, return_remaining=True)
    assert thr0.item() == torch.topk(x.float().reshape(-1), k).values[-1].item()
    for factor in (0.0, 0.5, 0.75, 1.0, 1.5, 100.0):
        floor = thr0 * factor
        thr, rem = S.positive_thresholds(x.view(1, 1, -1), k, return_remaining=True, floor=floor)
        assert thr.item() == thr0.item() and rem.item() == rem0.item(), factor


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B,N,k", [(64, 4096, 50), (7, 1000, 1), (300, 33000, 700), (4, 256, 0)])
def test_row_compaction_matches_nonzero(dtype, B, N, k):
    torch.manual_seed(2)
    x = torch.zeros(B, N, device="cuda")
    for b in range(B):
        cols = torch.randperm(N, device="cuda")[: max(0, k - b % 3)]
        x[b, cols] = torch.rand(cols.numel(), device="cuda") + 0.5
    x = x.to(dtype)
    idx, val = S.dense_rows_to_sparse(x)
    ridx, rval = S.ref_dense_rows_to_sparse(x, idx.shape[1])
    assert torch.equal(idx, ridx) and torch.equal(val, rval)
    idx2, val2 = S.dense_rows_to_sparse(x, cap=8)  # a cap below the row count truncates, never overruns
    r2 = S.ref_dense_rows_to_sparse(x, 8)
    assert torch.equal(idx2, r2[0]) and torch.equal(val2, r2[1])


@pytest.mark.gpu
@pytest.mark.parametrize("src_dtype,out_dtype", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16),
                                                 (torch.bfloat16, torch.float32), (torch.float32, torch.float32)])  # fmt: skip
def test_masked_row_compaction(src_dtype, out_dtype):
    torch.manual_seed(3)
    n, d = 10000, 768
    src = torch.randn(n, d, device="cuda").to(src_dtype)
    keep = torch.rand(n, device="cuda") > 0.3
    got = S.compact_rows(src, keep, out_dtype)
    assert torch.equal(got, src[keep].to(out_dtype))
    assert S.compact_rows(src, torch.zeros(n, dtype=torch.bool, device="cuda"), out_dtype).shape == (0, d)


@pytest.mark.gpu
def test_threshold_compaction_rations_ties_to_an_exact_count():
    torch.manual_seed(4)
    B, N, k = 64, 4096, 16
    g = torch.randn(B, N, device="cuda").relu_().to(torch.bfloat16)  # 16-bit data: the k-th largest value repeats
    thr, rem = S.positive_thresholds(g.view(1, 1, -1), k * B, return_remaining=True)
    n_above, n_equal = int((g.float() > thr).sum()), int((g.float() == thr).sum())
    assert n_equal > 1 and n_above < k * B <= n_above + n_equal and int(rem) == k * B - n_above
    idx_all, _ = S.threshold_rows_to_sparse(g, thr)
    assert int((idx_all >= 0).sum()) == n_above + n_equal  # without a budget every tie is kept
    div = torch.rand(N, device="cuda") + 0.5
    idx, val = S.threshold_rows_to_sparse(g, thr, div, n_ties=rem)
    assert int((idx >= 0).sum()) == k * B
    rows = torch.arange(B, device="cuda")[:, None].expand_as(idx)[idx >= 0]
    cols = idx[idx >= 0].long()
    assert bool((g[rows, cols].float() >= thr).all())
    assert torch.allclose(val[idx >= 0], g[rows, cols].float() / div[cols])
    strict = g.float() > thr
    got = torch.zeros_like(strict)
    got[rows, cols] = True
    assert bool((got | ~strict).all())  # everything above the threshold is there; the rest of the budget went to ties
    for r in range(B):  # ascending columns within a row
        c = idx[r][idx[r] >= 0]
        assert bool((c[1:] > c[:-1]).all())
