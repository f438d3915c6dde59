"""Sharding-aware tensor ops on 2 gloo ranks against the same op on the full tensor (the reference project checks its
DTensor ops the same way: tests/unit/utils/test_distributed_ops.py)."""

import torch
import torch.distributed as dist

from language_model_saes_b200.parallel.dist_ops import (
    Sharded,
    all_gather_dict,
    all_gather_list,
    batch_index,
    broadcast_object,
    full_tensor,
    item,
    masked_fill,
    maybe_local_map,
    multi_batch_index,
    nonzero,
    searchsorted,
    slice_fill,
)
from language_model_saes_b200.testing import distributed_test
from language_model_saes_b200.utils.discrete import DiscreteMapper, KeyedDiscreteMapper


def test_plain_tensors_are_ordinary_ops():
    x = torch.arange(24.0).view(4, 6)
    idx = torch.tensor([[3, 1], [0, 5]])
    assert torch.equal(batch_index(x, idx), x[idx[:, 0], idx[:, 1]])
    assert torch.equal(batch_index(x, idx[:, :1], n_batch_dims=1), x[:, idx[:, 0]])
    assert torch.equal(nonzero(x > 20), (x > 20).nonzero())
    assert torch.equal(masked_fill(x, x > 3, 0.0), x.masked_fill(x > 3, 0.0))
    assert item(torch.tensor(3.0)) == 3.0
    assert torch.equal(full_tensor(x), x)
    assert torch.equal(slice_fill(x.clone(), (slice(None), 0), 7.0)[:, 0], torch.full((4,), 7.0))
    assert searchsorted(torch.tensor([1.0, 2.0, 3.0]), torch.tensor([2.5])).item() == 2
    assert [r.tolist() for r in multi_batch_index([(x, idx)])] == [x[idx[:, 0], idx[:, 1]].tolist()]


def test_discrete_mapper_roundtrip():
    m = DiscreteMapper()
    assert m.encode(["a", "b", "a"]) == [0, 1, 0]
    assert m.decode([1, 0]) == ["b", "a"]
    assert m.get_mapping() == {"a": 0, "b": 1}
    k = KeyedDiscreteMapper()
    assert k.encode("ds", ["x", "y"]) == [0, 1] and k.encode("m", ["y"]) == [0]
    assert k.decode("ds", [1]) == ["y"] and sorted(k.keys()) == ["ds", "m"]


@distributed_test(nproc_per_node=2, backend="gloo")
def test_sharded_ops_match_full_tensor():
    r, g = dist.get_rank(), dist.group.WORLD
    torch.manual_seed(0)
    X = torch.randn(8, 6, 4)
    idx = torch.tensor([[7, 1], [0, 2], [5, 5], [3, 0], [4, 4]])
    for dim in (0, 1, 2):
        xs = Sharded(X.chunk(2, dim)[r].contiguous(), dim, g)
        assert xs.shape == X.shape
        assert torch.equal(xs.full(), X)
        assert torch.equal(batch_index(xs, idx, preserve_order=True), X[idx[:, 0], idx[:, 1]])
    # unordered result: same multiset of rows, grouped by owner
    xs = Sharded(X.chunk(2, 0)[r].contiguous(), 0, g)
    un = batch_index(xs, idx)
    assert torch.equal(un, X[torch.tensor([0, 3, 7, 5, 4]), torch.tensor([2, 0, 1, 5, 4])])
    xs1 = Sharded(X.chunk(2, 1)[r].contiguous(), 1, g)
    assert torch.equal(batch_index(xs1, idx[:, 1:2], n_batch_dims=1, preserve_order=True), X[:, idx[:, 1]])
    M = X[..., 0] > 0.5
    assert torch.equal(nonzero(Sharded(M.chunk(2, 0)[r].contiguous(), 0, g)), M.nonzero())
    a, b = nonzero(Sharded(M.chunk(2, 0)[r].contiguous(), 0, g), as_tuple=True)
    assert torch.equal(torch.stack([a, b], 1), M.nonzero())
    Y, Z = torch.randn(8, 3), torch.randn(8, 3)
    i2 = torch.tensor([[6], [1], [2], [6]])
    ya, za = multi_batch_index(
        [(Sharded(Y.chunk(2, 0)[r].contiguous(), 0, g), i2), (Sharded(Z.chunk(2, 0)[r].contiguous(), 0, g), i2)], preserve_order=True
    )
    assert torch.equal(ya, Y[i2[:, 0]]) and torch.equal(za, Z[i2[:, 0]])
    mf = masked_fill(xs, Sharded((X > 0).chunk(2, 0)[r], 0, g), -1.0)
    assert torch.equal(mf.full(), X.masked_fill(X > 0, -1.0))
    doubled = maybe_local_map(lambda t: t * 2)(xs)
    assert isinstance(doubled, Sharded) and torch.equal(doubled.full(), X * 2)
    assert item(Sharded(torch.tensor(5.0))) == 5.0


@distributed_test(nproc_per_node=2, backend="gloo")
def test_object_collectives_and_mapper():
    r, g = dist.get_rank(), dist.group.WORLD
    d = all_gather_dict({"t": torch.arange(r + 1), "o": f"r{r}"}, g)
    assert d[1]["t"].tolist() == [0, 1] and d[0]["t"].tolist() == [0] and d[0]["o"] == "r0" and d[1]["o"] == "r1"
    assert all_gather_list([r], g) == [0, 1]
    assert all_gather_list([r], g, flatten=False) == [[0], [1]]
    assert broadcast_object("hello" if r == 0 else None, 0, g) == "hello"
    m = DiscreteMapper()
    enc = m.encode(["b", "a"] if r == 0 else ["c", "a"], group=g)
    tables: list = [None, None]
    dist.all_gather_object(tables, m.get_mapping(), group=g)
    assert tables[0] == tables[1] == {"a": 0, "b": 1, "c": 2}
    assert enc == ([1, 0] if r == 0 else [2, 0])
