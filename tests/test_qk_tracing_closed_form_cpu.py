"""``compute_qk_tracing`` against closed forms. Queries and keys are LINEAR in one shared source vector,
``q = A v`` and ``k = B v``, so the attention score ``q . k = sum_ij v_i v_j (A[:, i] . B[:, j])`` splits exactly into

* pair terms        ``T[i, j] = v_i v_j (A[:, i] . B[:, j])``   (source i through the query, source j through the key),
* query marginals   ``a_Q[i]  = v_i (k . A[:, i]) = sum_j T[i, j]``,
* key marginals     ``a_K[j]  = v_j (q . B[:, j]) = sum_i T[i, j]``,

which is what the function's three outputs must contain (the reference project checks the same identities in
tests/unit/test_compute_qk_tracing.py). Layout contract: the forward batch holds ``topk`` identical rows per slot
(attention feature), row ``s * topk + r`` being slot ``s``."""

import pytest
import torch

from language_model_saes_b200.circuits.attribution import NodeRefs, QKTracingResult, compute_qk_tracing


def _setup(A: torch.Tensor, B: torch.Tensor, v: torch.Tensor, topk: int):
    """``A, B [slots, d_qk, n_src]``, ``v [slots, n_src]`` -> (q_targets, k_targets, sources)."""
    n_slots, _, n_src = A.shape
    src = v.repeat_interleave(topk, dim=0).clone().requires_grad_(True)  # [slots * topk, n_src]
    q = torch.stack([src @ A[s].T for s in range(n_slots)], dim=1)  # [rows, slots, d_qk]
    k = torch.stack([src @ B[s].T for s in range(n_slots)], dim=1)
    slots = torch.arange(n_slots).unsqueeze(-1)
    return (NodeRefs.from_nodes_and_refs([("q_vectors", slots, q)]), NodeRefs.from_nodes_and_refs([("k_vectors", slots, k)]),
            NodeRefs.from_nodes_and_refs([("src", torch.arange(n_src).unsqueeze(-1), src)]))  # fmt: skip


def _closed_forms(A, B, v):
    T = v[:, None] * v[None, :] * (A.T @ B)
    return T, T.sum(1), T.sum(0)


def _index(node) -> int:
    return int(node.indices[0, 0])


@pytest.mark.parametrize("n_slots,topk,n_src,d_qk,seed", [(3, 4, 6, 5, 0), (1, 3, 7, 2, 1), (4, 2, 3, 8, 2)])
def test_pairs_and_marginals_equal_their_closed_forms(n_slots, topk, n_src, d_qk, seed):
    g = torch.Generator().manual_seed(seed)
    A, B, v = torch.randn(n_slots, d_qk, n_src, generator=g), torch.randn(n_slots, d_qk, n_src, generator=g), torch.randn(n_slots, n_src, generator=g)
    res = compute_qk_tracing(*_setup(A, B, v, topk), topk=topk)
    assert isinstance(res, QKTracingResult) and len(res.pairs.value) == len(res.q_marginal.value) == len(res.k_marginal.value) == n_slots
    assert res.pairs.dimensions[0].keys == ["q_vectors"]
    for s in range(n_slots):
        T, aq, ak = _closed_forms(A[s], B[s], v[s])
        pairs = res.pairs.value[s]
        qn, kn = list(pairs.dimensions[0]), list(pairs.dimensions[1])
        assert 0 < len(pairs.value) <= topk * topk and len(qn) == len(kn) == len(pairs.value)
        seen = set()
        for a, b, val in zip(qn, kn, pairs.value):
            assert a.key == b.key == "src"
            i, j = _index(a), _index(b)  # dimension 0 is the query-side source, dimension 1 the key-side source
            assert torch.allclose(val, T[i, j], atol=1e-5), (s, i, j, float(val), float(T[i, j]))
            assert (i, j) not in seen  # a pair reached from both sides is listed once
            seen.add((i, j))
        for marg, want in ((res.q_marginal.value[s], aq), (res.k_marginal.value[s], ak)):
            nodes = list(marg.dimensions[0])
            assert 0 < len(nodes) <= topk
            for node, val in zip(nodes, marg.value):
                assert torch.allclose(val, want[_index(node)], atol=1e-5)
            # the listed sources are the strongest ones of that side, in descending order
            assert torch.allclose(marg.value, want.topk(len(nodes)).values, atol=1e-5)


def test_marginals_cover_every_source_when_topk_is_the_source_count():
    g = torch.Generator().manual_seed(7)
    n_src = 5
    A, B, v = torch.randn(2, 4, n_src, generator=g), torch.randn(2, 4, n_src, generator=g), torch.randn(2, n_src, generator=g)
    res = compute_qk_tracing(*_setup(A, B, v, n_src), topk=n_src)
    for s in range(2):
        _, aq, ak = _closed_forms(A[s], B[s], v[s])
        for marg, want in ((res.q_marginal.value[s], aq), (res.k_marginal.value[s], ak)):
            got = torch.zeros(n_src)
            for node, val in zip(marg.dimensions[0], marg.value):
                got[_index(node)] = val
            assert torch.allclose(got, want, atol=1e-5)
            # the marginals of a side add up to the attention score itself
            assert torch.allclose(got.sum(), (A[s] @ v[s]) @ (B[s] @ v[s]), atol=1e-4)


def test_the_globally_strongest_pair_is_found():
    """One pair term is made to dominate everything else; whichever side picks it up first, it must be in the list with
    its exact value, query-side source first."""
    g = torch.Generator().manual_seed(3)
    n_src, d_qk, topk = 8, 4, 3
    A, B = 0.05 * torch.randn(1, d_qk, n_src, generator=g), 0.05 * torch.randn(1, d_qk, n_src, generator=g)
    A[0, :, 2] = torch.tensor([3.0, 0.0, 0.0, 0.0])
    B[0, :, 6] = torch.tensor([2.0, 0.0, 0.0, 0.0])
    v = torch.ones(1, n_src)
    res = compute_qk_tracing(*_setup(A, B, v, topk), topk=topk)
    T, _, _ = _closed_forms(A[0], B[0], v[0])
    assert (T.abs().argmax() // n_src, T.abs().argmax() % n_src) == (2, 6)
    pairs = res.pairs.value[0]
    listed = {(_index(a), _index(b)): float(val) for a, b, val in zip(pairs.dimensions[0], pairs.dimensions[1], pairs.value)}
    assert (2, 6) in listed and abs(listed[(2, 6)] - float(T[2, 6])) < 1e-5
    assert (6, 2) not in listed or abs(listed[(6, 2)] - float(T[6, 2])) < 1e-5  # roles are positional, not symmetric


def test_a_pair_that_only_the_key_side_ranks_high_is_still_found():
    """Source 1 matters through the key only (its query column is zero) and source 4 through the query only: the pair
    (4, 1) must be listed as (query source 4, key source 1) whichever first-order list led to it."""
    n_src, d_qk, topk = 6, 3, 2
    A, B = torch.zeros(1, d_qk, n_src), torch.zeros(1, d_qk, n_src)
    A[0, 0, 4] = 2.0
    B[0, 0, 1] = 5.0
    A[0, 1, 0], B[0, 1, 0] = 0.1, 0.1  # a weak distractor present on both sides
    v = torch.ones(1, n_src)
    res = compute_qk_tracing(*_setup(A, B, v, topk), topk=topk)
    pairs = res.pairs.value[0]
    listed = {(_index(a), _index(b)): float(val) for a, b, val in zip(pairs.dimensions[0], pairs.dimensions[1], pairs.value)}
    assert abs(listed[(4, 1)] - 10.0) < 1e-5 and (1, 4) not in listed
    q_nodes = {_index(n) for n in res.q_marginal.value[0].dimensions[0]}
    k_nodes = {_index(n) for n in res.k_marginal.value[0].dimensions[0]}
    assert 4 in q_nodes and 1 not in q_nodes and 1 in k_nodes and 4 not in k_nodes
