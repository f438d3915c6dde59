"""``batch_index`` / ``multi_batch_index`` on sharded tensors (2 gloo ranks) against plain indexing of the full tensor,
over the cases that tests/distributed/test_batched_index.py of the reference project walks through: no batch dimension,
leading batch dimensions, index tuples shorter than the tensor's rank, the split on an indexed / a batch / a trailing
dimension, three-dimensional tensors, and results in index order or grouped by owner."""

import itertools

import torch
import torch.distributed as dist

from language_model_saes_b200.parallel.dist_ops import Sharded, batch_index, multi_batch_index
from language_model_saes_b200.testing import distributed_test


def _full_index(X: torch.Tensor, idx: torch.Tensor, n_batch: int) -> torch.Tensor:
    """X[(:,) * n_batch, idx[:, 0], idx[:, 1], ...] with the picked rows stacked along dimension ``n_batch``."""
    lead = (slice(None),) * n_batch
    return X[lead + tuple(idx[:, j] for j in range(idx.shape[1]))]


def _grouped_by_owner(idx: torch.Tensor, col: int, size: int) -> torch.Tensor:
    """Order in which an unordered result lists the rows: by the rank that owns them, input order inside a rank."""
    return torch.argsort(torch.div(idx[:, col], size, rounding_mode="floor"), stable=True)


@distributed_test(nproc_per_node=2, backend="gloo")
def test_batch_index_on_every_split_dimension():
    r, g = dist.get_rank(), dist.group.WORLD
    gen = torch.Generator().manual_seed(0)
    checked = 0
    for shape, n_batch, n_idx in [((8, 6), 0, 2), ((8, 6), 0, 1), ((4, 8, 6), 1, 2), ((4, 8, 6), 1, 1), ((8, 6, 4), 0, 3),
                                  ((8, 6, 4), 0, 2), ((2, 4, 6, 8), 2, 2), ((2, 4, 6, 8), 1, 2)]:  # fmt: skip
        X = torch.randn(*shape, generator=gen)
        n = 11
        idx = torch.stack([torch.randint(0, shape[n_batch + j], (n,), generator=gen) for j in range(n_idx)], dim=1)
        want = _full_index(X, idx, n_batch)
        for dim in range(len(shape)):
            if shape[dim] % 2:
                continue
            xs = Sharded(X.chunk(2, dim)[r].contiguous(), dim, g)
            got = batch_index(xs, idx, n_batch_dims=n_batch, preserve_order=True)
            assert got.shape == want.shape and torch.equal(got, want), (shape, n_batch, n_idx, dim)
            un = batch_index(xs, idx, n_batch_dims=n_batch)
            col = dim - n_batch
            if 0 <= col < n_idx:  # the split dimension is indexed: rows come grouped by owner
                order = _grouped_by_owner(idx, col, shape[dim] // 2)
                assert torch.equal(un, want.index_select(n_batch, order)), (shape, n_batch, n_idx, dim)
            else:  # batch or trailing dimension: nothing is regrouped
                assert torch.equal(un, want), (shape, n_batch, n_idx, dim)
            checked += 1
    assert checked >= 20
    # replicated inputs and empty index lists
    X = torch.randn(6, 4, generator=gen)
    idx = torch.tensor([[5, 0], [1, 3]])
    assert torch.equal(batch_index(Sharded(X), idx), X[idx[:, 0], idx[:, 1]]) and torch.equal(batch_index(X, idx), X[idx[:, 0], idx[:, 1]])
    xs = Sharded(X.chunk(2, 0)[r].contiguous(), 0, g)
    none = batch_index(xs, torch.empty(0, 2, dtype=torch.long), preserve_order=True)
    assert none.shape == (0,)
    only_rank0 = batch_index(xs, torch.tensor([[0, 1], [2, 2]]), preserve_order=True)  # every row lives on rank 0
    assert torch.equal(only_rank0, X[torch.tensor([0, 2]), torch.tensor([1, 2])])
    dup = batch_index(xs, torch.tensor([[4, 1], [4, 1], [0, 0]]), preserve_order=True)  # repeated index rows
    assert torch.equal(dup, torch.stack([X[4, 1], X[4, 1], X[0, 0]]))


@distributed_test(nproc_per_node=2, backend="gloo")
def test_multi_batch_index_shares_exchanges_and_keeps_every_result():
    r, g = dist.get_rank(), dist.group.WORLD
    gen = torch.Generator().manual_seed(1)
    A, B, C = torch.randn(8, 5, generator=gen), torch.randn(8, 5, generator=gen), torch.randn(8, 6, 3, generator=gen)
    D = torch.randint(0, 100, (8, 5), generator=gen)  # another dtype: its own exchange
    ia = torch.tensor([[7], [0], [3], [3], [4]])
    ib = torch.tensor([[1], [6]])
    ic = torch.tensor([[2, 5], [7, 0], [4, 4]])

    def shard(t, dim=0):
        return Sharded(t.chunk(2, dim)[r].contiguous(), dim, g)

    for preserve, n_calls in itertools.product((True, False), (1, 2)):
        for _ in range(n_calls):  # (a second call reuses nothing from the first)
            ra, rb, rc, rd, re_, rf = multi_batch_index(
                [(shard(A), ia), (shard(B), ib), (shard(C), ic), (shard(D), ia), (A, ia), (shard(C, 1), ic)], preserve_order=preserve)  # fmt: skip
            if preserve:
                assert torch.equal(ra, A[ia[:, 0]]) and torch.equal(rb, B[ib[:, 0]]) and torch.equal(rd, D[ia[:, 0]])
                assert torch.equal(rc, C[ic[:, 0], ic[:, 1]]) and torch.equal(rf, C[ic[:, 0], ic[:, 1]])
            else:
                assert torch.equal(ra, A[ia[:, 0]][_grouped_by_owner(ia, 0, 4)]) and torch.equal(rb, B[ib[:, 0]][_grouped_by_owner(ib, 0, 4)])
                assert torch.equal(rc, C[ic[:, 0], ic[:, 1]][_grouped_by_owner(ic, 0, 4)])
                assert torch.equal(rf, C[ic[:, 0], ic[:, 1]][_grouped_by_owner(ic, 1, 3)])
            assert torch.equal(re_, A[ia[:, 0]])  # a plain tensor passes through ordinary indexing
    # leading batch dimensions fall back to one exchange per tensor, same values
    E = torch.randn(3, 8, 4, generator=gen)
    ie = torch.tensor([[6], [1], [1]])
    (re2,) = multi_batch_index([(shard(E, 1), ie)], n_batch_dims=1, preserve_order=True)
    assert torch.equal(re2, E[:, ie[:, 0]])
    assert multi_batch_index([]) == []
