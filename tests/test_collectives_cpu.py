"""The autograd-aware collectives and the cross-shard top-k, two gloo ranks against one process: what each one does to values
and to gradients, and that the sharded selection is the same set as ``torch.topk`` on the whole feature axis (the role of
utils/distributed/ops.py:158-266 of the reference project)."""

import torch
import torch.distributed as dist

from language_model_saes_b200.parallel.collectives import (
    all_gather_cat,
    all_reduce_sum,
    all_reduce_sum_both,
    copy_to_group,
    distributed_threshold,
    distributed_topk,
)
from language_model_saes_b200.testing import distributed_test


def test_without_a_group_everything_is_the_identity_and_topk_is_plain():
    x = torch.randn(4, 10, requires_grad=True)
    assert all_reduce_sum(x, None) is x and copy_to_group(x, None) is x and all_reduce_sum_both(x, None) is x and all_gather_cat(x, None) is x
    out = distributed_topk(x, 3, None)
    want = torch.zeros_like(x).scatter(-1, x.topk(3).indices, x.topk(3).values) * (x > 0)
    assert torch.equal(out, want)
    out.sum().backward()
    assert torch.equal(x.grad, (out != 0).float())  # the gradient passes where a value was kept
    # negative entries may be selected when asked to
    y = -torch.rand(2, 6) - 0.1
    assert (distributed_topk(y, 2, None, positive_only=False) != 0).sum() == 4
    assert (distributed_topk(y, 2, None) != 0).sum() == 0
    # several axes at once: the k largest of the whole batch
    z = torch.rand(5, 8)
    kept = distributed_topk(z, 7, None, dim=(-2, -1))
    assert (kept != 0).sum() == 7 and kept.max() == z.max() and torch.equal(kept[kept != 0].sort().values, z.flatten().topk(7).values.sort().values)
    assert distributed_threshold(z, 3, None).shape == (5, 1)


@distributed_test(nproc_per_node=2)
def test_values_and_gradients_of_each_collective_on_two_ranks():
    rank, g = dist.get_rank(), dist.group.WORLD
    mine = torch.full((3,), float(rank + 1), requires_grad=True)
    # sum forward, identity backward: a partial result that enters a sum
    out = all_reduce_sum(mine, g)
    assert out.tolist() == [3.0] * 3
    (out * (rank + 1)).sum().backward()
    assert mine.grad.tolist() == [float(rank + 1)] * 3
    # identity forward, sum backward: a replicated value that every rank uses in its own shard
    rep = torch.ones(3, requires_grad=True)
    (copy_to_group(rep, g) * (rank + 1)).sum().backward()
    assert rep.grad.tolist() == [3.0] * 3
    # sum both ways
    both = torch.full((3,), float(rank + 1), requires_grad=True)
    out = all_reduce_sum_both(both, g)
    assert out.tolist() == [3.0] * 3
    (out * (rank + 1)).sum().backward()
    assert both.grad.tolist() == [3.0] * 3
    # gather in rank order along any axis
    piece = torch.full((2, 2), float(rank))
    assert all_gather_cat(piece, g, dim=1).tolist() == [[0.0, 0.0, 1.0, 1.0]] * 2
    assert all_gather_cat(piece, g, dim=0)[:, 0].tolist() == [0.0, 0.0, 1.0, 1.0]


@distributed_test(nproc_per_node=2)
def test_sharded_topk_selects_what_topk_on_the_whole_axis_selects():
    rank, g = dist.get_rank(), dist.group.WORLD
    gen = torch.Generator().manual_seed(0)  # the same full tensor on both ranks
    full = torch.randn(6, 40, generator=gen)
    full[0] = -full[0].abs()  # a row without a positive entry
    full[1, 3:] = -1.0  # a row with fewer positive entries than k
    full[1, :3] = torch.tensor([0.5, 0.7, 0.9])
    full[2, :30] = 0.25  # ties at the threshold keep every tied entry, on whichever shard it is
    full[2, 30:] = -1.0
    local = full[:, rank * 20 : (rank + 1) * 20].clone().requires_grad_()
    k = 5
    out = distributed_topk(local, k, g)
    kept = all_gather_cat(out.detach(), g, dim=-1)
    assert (kept[0] != 0).sum() == 0
    assert kept[1].nonzero().flatten().tolist() == [0, 1, 2]
    assert (kept[2] != 0).sum() == 30
    for r in (3, 4, 5):
        want = torch.zeros(40).scatter(0, full[r].topk(k).indices, full[r].topk(k).values)
        want = want * (want > 0)
        assert torch.equal(kept[r], want)
    out.sum().backward()
    assert torch.equal(local.grad, (out != 0).float())
    thr = distributed_threshold(full[3:, rank * 20 : (rank + 1) * 20], k, g)
    assert torch.equal(thr[:, 0], full[3:].topk(k).values[:, -1])
    # more wanted than one shard holds: the other shard's candidates fill in
    few = full[3:, rank * 2 : (rank + 1) * 2]
    thr = distributed_threshold(few, 3, g)
    assert torch.equal(thr[:, 0], full[3:, :4].topk(3).values[:, -1])
    # the k largest of the whole batch, feature axis sharded
    batch = distributed_topk(full[3:, rank * 20 : (rank + 1) * 20].abs(), 9, g, dim=(-2, -1))
    got = all_gather_cat(batch, g, dim=-1)
    assert (got != 0).sum() == 9
    assert torch.equal(got[got != 0].sort().values, full[3:].abs().flatten().topk(9).values.sort().values)
