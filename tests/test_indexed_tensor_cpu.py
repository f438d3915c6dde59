"""Node-indexed tensor algebra (``circuits/indexed_tensor.py``), case by case: construction, the two lookups and their
duality, set difference and union, element access by nodes, growth along an axis, top-k and the products. The cases
follow the behaviours that tests/unit/test_node_indexed_tensor.py of the reference project pins down (offsets of
registered nodes, -1 for anything not registered, order of the result = order of the query, exact values)."""

import pytest
import torch

from language_model_saes_b200.circuits.indexed_tensor import (
    NodeDimension,
    NodeIndexed,
    NodeIndexedMatrix,
    NodeIndexedTensor,
    NodeIndexedVector,
    NodeInfo,
)
from language_model_saes_b200.core.serialize import dumps, loads


def dim(*infos) -> NodeDimension:
    return NodeDimension.from_node_infos([NodeInfo(k, torch.tensor(i)) for k, i in infos])


def nodes(d: NodeDimension) -> list[tuple]:
    return [(n.key, n.indices.tolist()) for n in d.node_infos]


# two one-dimensional nodes: "a" with elements 0..2 (offsets 0..2), "b" with elements 10, 11 (offsets 3, 4)
@pytest.fixture
def ab():
    return dim(("a", [[0], [1], [2]]), ("b", [[10], [11]]))


# one node with (position, feature) pairs and one with single indices
@pytest.fixture
def feat_err():
    return dim(("feat", [[0, 5], [0, 7], [1, 5], [2, 9]]), ("err", [[0], [1], [2]]))


# ---- construction ---------------------------------------------------------------------------------------------------
def test_from_dimensions_allocates_zeros(ab):
    v = NodeIndexedVector.from_dimensions((ab,))
    assert v.data.shape == (5,) and v.data.abs().sum() == 0 and v.data.dtype == torch.float32
    m = NodeIndexedMatrix.from_dimensions((ab, dim(("c", [[0]]))), dtype=torch.float64)
    assert m.data.shape == (5, 1) and m.data.dtype == torch.float64


def test_from_data_keeps_values_and_checks_lengths(ab):
    data = torch.arange(5.0)
    v = NodeIndexedVector.from_data(data, (ab,))
    assert v.data is data or torch.equal(v.data, data)
    with pytest.raises(AssertionError):
        NodeIndexedVector.from_data(torch.zeros(4), (ab,))


def test_construction_from_node_info_lists_equals_prebuilt_dimension(ab):
    infos = [NodeInfo("a", torch.tensor([[0], [1], [2]])), NodeInfo("b", torch.tensor([[10], [11]]))]
    v = NodeIndexedVector.from_data(torch.arange(5.0), (infos,))
    assert v.dimensions[0] == ab
    z = NodeIndexedVector.from_dimensions((infos,))
    assert z.dimensions[0] == ab


def test_node_mappings_hold_offsets_and_indices(ab):
    m = ab.node_mappings
    assert list(m) == ["a", "b"]
    assert m["a"].indices.tolist() == [[0], [1], [2]] and m["b"].indices.tolist() == [[10], [11]]
    assert ab.offsets_of_key("a").tolist() == [0, 1, 2] and ab.offsets_of_key("b").tolist() == [3, 4]


def test_empty_dimension_needs_a_device():
    with pytest.raises(ValueError):
        NodeDimension.from_node_infos([])
    assert len(NodeDimension.from_node_infos([], device="cpu")) == 0


def test_same_key_given_twice_is_one_key_with_both_groups():
    d = dim(("a", [[0]]), ("b", [[5]]), ("a", [[3]]))
    assert d.keys == ["a", "b"] and len(d) == 3
    assert d.offsets_of_key("a").tolist() == [0, 2]
    assert d.node_mappings["a"].indices.tolist() == [[0], [3]]


# ---- nodes -> offsets -----------------------------------------------------------------------------------------------
@pytest.mark.parametrize(
    "query,want",
    [
        ((("a", [[0], [1], [2]]),), [0, 1, 2]),  # a whole node
        ((("b", [[10], [11]]),), [3, 4]),
        ((("a", [[1]]),), [1]),  # part of a node
        ((("b", [[11]]),), [4]),
        ((("b", [[11]]), ("a", [[2], [0]])), [4, 2, 0]),  # across nodes, in the order of the query
        ((("zzz", [[0]]),), [-1]),  # unknown key
        ((("a", [[99]]),), [-1]),  # index outside everything registered
        ((("b", [[0]]),), [-1]),  # an index that exists under another key only
        ((("a", [[1]]), ("q", [[1]]), ("b", [[10]]), ("a", [[7]])), [1, -1, 3, -1]),  # found and missing mixed
    ],
)
def test_nodes_to_offsets(ab, query, want):
    assert ab.nodes_to_offsets(dim(*query)).tolist() == want


def test_nodes_to_offsets_is_cached_per_query_dimension(ab):
    """The cache key is the identity of the query's tensors (a cheap hash, as in the reference): the same dimension
    object hits, an equal one built anew is looked up again with the same result."""
    q = dim(("b", [[11]]), ("a", [[0]]))
    first = ab.nodes_to_offsets(q)
    assert hash(q) in ab._n2o_cache and ab.nodes_to_offsets(q) is first
    again = ab.nodes_to_offsets(dim(("b", [[11]]), ("a", [[0]])))
    assert first.tolist() == again.tolist() == [4, 0]


def test_nodes_to_offsets_after_merging_a_key(ab):
    merged = ab + dim(("a", [[7]]))
    assert merged.nodes_to_offsets(dim(("a", [[7], [0]]), ("b", [[10]]))).tolist() == [5, 0, 3]


@pytest.mark.parametrize(
    "query,want",
    [
        ((("feat", [[0, 5], [0, 7], [1, 5], [2, 9]]),), [0, 1, 2, 3]),
        ((("feat", [[1, 5]]),), [2]),
        ((("err", [[2]]), ("feat", [[0, 7]])), [6, 1]),
        ((("feat", [[0, 9]]),), [-1]),  # both coordinates occur, the pair does not
        ((("feat", [[5, 0]]),), [-1]),  # the pair reversed
        ((("err", [[3]]),), [-1]),
    ],
)
def test_nodes_to_offsets_with_index_pairs(feat_err, query, want):
    assert feat_err.nodes_to_offsets(dim(*query)).tolist() == want


# ---- offsets -> nodes and the duality -------------------------------------------------------------------------------
@pytest.mark.parametrize(
    "offsets,want",
    [
        ([0, 1, 2], [("a", [[0], [1], [2]])]),
        ([3, 4], [("b", [[10], [11]])]),
        ([4], [("b", [[11]])]),
        ([2, 3], [("a", [[2]]), ("b", [[10]])]),
    ],
)
def test_offsets_to_nodes(ab, offsets, want):
    assert nodes(ab.offsets_to_nodes(torch.tensor(offsets))) == want


def test_offsets_to_nodes_with_index_pairs(feat_err):
    assert nodes(feat_err.offsets_to_nodes(torch.tensor([1, 3]))) == [("feat", [[0, 7], [2, 9]])]
    assert nodes(feat_err.offsets_to_nodes(torch.tensor([4, 5, 6]))) == [("err", [[0], [1], [2]])]
    assert nodes(feat_err.offsets_to_nodes(torch.tensor([5, 0]))) == [("err", [[1]]), ("feat", [[0, 5]])]


@pytest.mark.parametrize("offsets", [[0, 1, 2, 3, 4], [4, 0], [3], [2, 2, 1]])
def test_offsets_to_nodes_then_back(ab, offsets):
    assert ab.nodes_to_offsets(ab.offsets_to_nodes(torch.tensor(offsets))).tolist() == offsets


def test_nodes_to_offsets_then_back(ab, feat_err):
    q = dim(("b", [[11]]), ("a", [[1], [0]]))
    assert ab.offsets_to_nodes(ab.nodes_to_offsets(q)) == q
    q2 = dim(("err", [[1]]), ("feat", [[2, 9], [0, 5]]))
    assert feat_err.offsets_to_nodes(feat_err.nodes_to_offsets(q2)) == q2
    merged = ab + dim(("a", [[7]]))
    q3 = dim(("a", [[7], [2]]))
    assert merged.offsets_to_nodes(merged.nodes_to_offsets(q3)) == q3


# ---- difference and union -------------------------------------------------------------------------------------------
def test_sub_removes_part_of_a_node(ab):
    assert nodes(ab - dim(("a", [[1]]))) == [("a", [[0], [2]]), ("b", [[10], [11]])]


def test_sub_removes_a_whole_node(ab):
    rest = ab - dim(("a", [[0], [1], [2]]))
    assert nodes(rest) == [("b", [[10], [11]])] and rest.keys == ["b"]


def test_sub_ignores_what_is_not_there(ab):
    assert ab - dim(("a", [[50]]), ("c", [[0]])) == ab


def test_sub_across_nodes_leaves_contiguous_offsets(ab):
    rest = ab - dim(("a", [[0]]), ("b", [[11]]))
    assert nodes(rest) == [("a", [[1], [2]]), ("b", [[10]])]
    assert rest.nodes_to_offsets(dim(("a", [[1], [2]]), ("b", [[10]]))).tolist() == [0, 1, 2]


def test_sub_of_everything_is_empty(ab):
    assert len(ab - ab) == 0 and (ab - ab).keys == []


def test_sub_with_index_pairs(feat_err):
    rest = feat_err - dim(("feat", [[0, 7], [2, 9]]), ("err", [[1]]))
    assert nodes(rest) == [("feat", [[0, 5], [1, 5]]), ("err", [[0], [2]])]


def test_sub_undoes_add_of_disjoint_pieces(ab):
    extra = dim(("c", [[0], [1]]), ("a", [[9]]))
    assert (ab + extra) - extra == ab


def test_add_with_empty_sides(ab):
    e = NodeDimension.empty("cpu")
    assert ab + e == ab and e + ab == ab


def test_add_rejects_a_key_whose_index_rank_differs(ab):
    with pytest.raises(AssertionError):
        ab + dim(("a", [[0, 0]]))


# ---- element access -------------------------------------------------------------------------------------------------
def test_getitem_by_nodes(ab):
    v = NodeIndexedVector.from_data(torch.tensor([10.0, 11.0, 12.0, 20.0, 21.0]), (ab,))
    assert v[dim(("a", [[0], [1], [2]]))].data.tolist() == [10.0, 11.0, 12.0]
    assert v[dim(("b", [[10], [11]]))].data.tolist() == [20.0, 21.0]
    assert v[dim(("b", [[11]]), ("a", [[0]]))].data.tolist() == [21.0, 10.0]  # reordered, across nodes
    assert v[dim(("a", [[1]]))].data.tolist() == [11.0]
    assert v[None].data.tolist() == v.data.tolist()


def test_getitem_result_carries_the_query_dimension(ab):
    v = NodeIndexedVector.from_data(torch.arange(5.0), (ab,))
    q = dim(("b", [[10]]), ("a", [[2]]))
    out = v[q]
    assert isinstance(out, NodeIndexedVector) and out.dimensions[0] == q


def test_getitem_wants_one_selector_per_axis(ab):
    m = NodeIndexedMatrix.from_dimensions((ab, ab))
    with pytest.raises(ValueError):
        m[ab]


def test_setitem_by_nodes(ab):
    v = NodeIndexedVector.from_dimensions((ab,))
    v[dim(("a", [[0], [1], [2]]))] = torch.tensor([1.0, 2.0, 3.0])
    assert v.data.tolist() == [1.0, 2.0, 3.0, 0.0, 0.0]
    v[dim(("b", [[11]]))] = 9.0
    assert v.data.tolist() == [1.0, 2.0, 3.0, 0.0, 9.0]  # the rest of the node is untouched
    v[None] = 4.0
    assert v.data.tolist() == [4.0] * 5
    q = dim(("b", [[10]]), ("a", [[1]]))
    v[q] = torch.tensor([7.0, 8.0])
    assert v[q].data.tolist() == [7.0, 8.0]
    w = NodeIndexedVector.from_data(torch.tensor([5.0, 6.0]), (q,))
    v[q] = w  # a node-indexed value on the right-hand side
    assert v[q].data.tolist() == [5.0, 6.0]


def test_access_with_index_pairs(feat_err):
    v = NodeIndexedVector.from_data(torch.arange(7.0), (feat_err,))
    assert v[dim(("feat", [[2, 9], [0, 5]]), ("err", [[1]]))].data.tolist() == [3.0, 0.0, 5.0]
    v[dim(("feat", [[1, 5]]))] = -1.0
    assert v.data.tolist() == [0.0, 1.0, -1.0, 3.0, 4.0, 5.0, 6.0]
    vals, where = v.topk(2)
    assert vals.tolist() == [6.0, 5.0] and nodes(where) == [("err", [[2], [1]])]


# ---- growth ---------------------------------------------------------------------------------------------------------
def test_add_nodes_extends_size_keeps_values_and_is_addressable(ab):
    v = NodeIndexedVector.from_data(torch.arange(5.0), (ab,))
    v.add_nodes(dim(("c", [[0], [1]])))
    assert v.data.tolist() == [0.0, 1.0, 2.0, 3.0, 4.0, 0.0, 0.0]
    assert v.dimensions[0].offsets_of_key("c").tolist() == [5, 6]
    v[dim(("c", [[1]]))] = 3.5
    assert v.data[6] == 3.5
    v.add_nodes(dim(("a", [[8]])), torch.tensor([2.5]))  # an existing key grows, with data
    assert v.dimensions[0].keys == ["a", "b", "c"] and v[dim(("a", [[8]]))].data.tolist() == [2.5]
    with pytest.raises(AssertionError):
        v.add_nodes(dim(("d", [[0]])), torch.zeros(2))


# ---- matrices -------------------------------------------------------------------------------------------------------
@pytest.fixture
def mat(ab):
    cols = dim(("x", [[0], [1]]), ("y", [[0]]))
    return NodeIndexedMatrix.from_data(torch.arange(15.0).view(5, 3), (ab, cols))


def test_matrix_slices(mat):
    assert mat.data.shape == (5, 3)
    assert mat[dim(("b", [[10], [11]])), None].data.tolist() == [[9.0, 10.0, 11.0], [12.0, 13.0, 14.0]]
    assert mat[None, dim(("y", [[0]]))].data.tolist() == [[2.0], [5.0], [8.0], [11.0], [14.0]]
    assert mat[dim(("a", [[2]]), ("b", [[10]])), dim(("y", [[0]]), ("x", [[0]]))].data.tolist() == [[8.0, 6.0], [11.0, 9.0]]
    assert torch.equal(mat[None, None].data, mat.data)


def test_matrix_assignment(mat):
    mat[dim(("a", [[0]])), dim(("x", [[1]]), ("y", [[0]]))] = torch.tensor([[-1.0, -2.0]])
    assert mat.data[0].tolist() == [0.0, -1.0, -2.0]
    sel = (dim(("b", [[11]]), ("a", [[1]])), dim(("x", [[0]])))
    mat[sel] = torch.tensor([[70.0], [80.0]])
    assert mat[sel].data.tolist() == [[70.0], [80.0]] and mat.data[4, 0] == 70.0 and mat.data[1, 0] == 80.0


def test_matrix_growth(mat):
    mat.add_targets(dim(("t", [[0]])))
    assert mat.data.shape == (6, 3) and mat.data[5].abs().sum() == 0
    mat[dim(("t", [[0]])), None] = 1.0
    assert mat.data[5].tolist() == [1.0, 1.0, 1.0]
    mat.add_sources(dim(("z", [[4]])), torch.full((6, 1), 2.0))
    assert mat.data.shape == (6, 4) and mat[None, dim(("z", [[4]]))].data.squeeze(1).tolist() == [2.0] * 6


def test_matrix_reductions_and_fills(mat):
    hit = (mat.map(lambda t: t > 12.0)).any(0)
    assert isinstance(hit, NodeIndexedVector) and hit.data.tolist() == [False, True, True] and hit.dimensions[0] == mat.dimensions[1]
    rows = NodeIndexedVector.from_data(torch.tensor([True, False]), (dim(("b", [[10], [11]])),))
    mat.masked_fill_dim_(0, rows, 0.0)
    assert mat.data[3].abs().sum() == 0 and mat.data[4].abs().sum() > 0
    mask = mat.map(lambda t: t == 14.0)
    mat.masked_fill_(mask, -5.0)
    assert mat.data[4, 2] == -5.0
    both = mask & mask
    assert both.data.sum() == 1 and (~both).data.sum() == 14


def test_flat_topk_and_edge_lists(mat):
    top = mat.flat_topk(3)
    assert isinstance(top, NodeIndexed) and top.value.tolist() == [14.0, 13.0, 12.0] and len(top) == 3
    assert nodes(top.dimensions[0]) == [("b", [[11], [11], [11]])]
    assert [n.key for n in top.dimensions[1]] == ["y", "x", "x"]
    picked = top[dim(("y", [[0]])), 1]  # entries whose source node is y[0]
    assert picked.value.tolist() == [14.0]
    assert mat.flat_topk(100).value.numel() == 15 and mat.flat_topk(0).value.numel() == 0
    entries = list(top)
    assert float(entries[0][0]) == 14.0 and entries[0][1].key == "b" and entries[0][2].key == "y"


# ---- products -------------------------------------------------------------------------------------------------------
def test_vector_times_matrix(ab, mat):
    v = NodeIndexedVector.from_data(torch.tensor([1.0, 0.0, -1.0, 2.0, 0.5]), (ab,))
    out = v.matmul(mat)
    assert isinstance(out, NodeIndexedVector) and out.dimensions[0] == mat.dimensions[1]
    assert torch.allclose(out.data, v.data @ mat.data)
    assert torch.equal((v @ mat).data, out.data)


def test_vector_times_vector(ab):
    v = NodeIndexedVector.from_data(torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0]), (ab,))
    w = NodeIndexedVector.from_data(torch.tensor([1.0, 0.0, 0.0, 0.0, 2.0]), (ab,))
    assert v @ w == 11.0
    u = NodeIndexedVector.from_data(torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0]), (ab,))
    assert v.matmul(u) == 0.0


def test_matrix_times_vector_and_matrix(ab, mat):
    cols = mat.dimensions[1]
    c = NodeIndexedVector.from_data(torch.tensor([1.0, -1.0, 0.5]), (cols,))
    out = mat @ c
    assert isinstance(out, NodeIndexedVector) and out.dimensions[0] == ab and torch.allclose(out.data, mat.data @ c.data)
    right = NodeIndexedMatrix.from_data(torch.arange(6.0).view(3, 2), (cols, dim(("o", [[0], [1]]))))
    prod = mat.matmul(right)
    assert isinstance(prod, NodeIndexedMatrix) and prod.dimensions == (ab, right.dimensions[1])
    assert torch.allclose(prod.data, mat.data @ right.data)
    eye = NodeIndexedMatrix.from_data(torch.eye(3), (cols, cols))
    assert torch.equal((mat @ eye).data, mat.data)
    with pytest.raises(ValueError):
        mat.matmul(torch.zeros(3))  # type: ignore[arg-type]


def test_products_check_the_contracted_nodes_only_on_request(ab, mat):
    other_rows = dim(("p", [[0], [1], [2], [3], [4]]))
    v = NodeIndexedVector.from_data(torch.ones(5), (other_rows,))
    assert torch.allclose(v.matmul(mat).data, mat.data.sum(0))  # same length, different nodes: allowed by default
    with pytest.raises(AssertionError):
        v.matmul(mat, _check_node_matching=True)
    same = NodeIndexedVector.from_data(torch.ones(5), (ab,))
    assert torch.allclose(same.matmul(mat, _check_node_matching=True).data, mat.data.sum(0))
    c = NodeIndexedVector.from_data(torch.ones(3), (dim(("w", [[0], [1], [2]])),))
    assert torch.allclose(mat.matmul(c).data, mat.data.sum(1))
    with pytest.raises(AssertionError):
        mat.matmul(c, _check_node_matching=True)


# ---- other ----------------------------------------------------------------------------------------------------------
def test_topk_can_ignore_nodes(ab):
    v = NodeIndexedVector.from_data(torch.tensor([5.0, 1.0, 4.0, 9.0, 3.0]), (ab,))
    vals, where = v.topk(2)
    assert vals.tolist() == [9.0, 5.0] and nodes(where) == [("b", [[10]]), ("a", [[0]])]
    vals, where = v.topk(2, ignore_dimension=dim(("b", [[10]]), ("zz", [[0]])))  # unknown nodes in the list do no harm
    assert vals.tolist() == [5.0, 4.0] and nodes(where) == [("a", [[0], [2]])]
    assert v.data.tolist() == [5.0, 1.0, 4.0, 9.0, 3.0]  # the vector itself is untouched


def test_nonzero_lists_values_with_their_nodes(ab):
    v = NodeIndexedVector.from_data(torch.tensor([0.0, 2.0, 0.0, 0.0, 7.0]), (ab,))
    vals, (where,) = v.nonzero()
    assert vals.tolist() == [2.0, 7.0] and nodes(where) == [("a", [[1]]), ("b", [[11]])]


def test_sum_clone_and_serialisation(ab, mat):
    v = NodeIndexedVector.from_data(torch.arange(5.0), (ab,))
    w = v.clone()
    w.data[0] = 100.0
    assert v.data[0] == 0.0 and (v + w).data.tolist() == [100.0, 2.0, 4.0, 6.0, 8.0]
    back = loads(dumps(mat), NodeIndexedMatrix)
    assert torch.equal(back.data, mat.data) and back.dimensions == mat.dimensions
    generic = NodeIndexedTensor.from_data(torch.zeros(5, 3, 5), (ab, mat.dimensions[1], ab))
    assert generic.n_dims == 3 and generic[None, dim(("y", [[0]])), dim(("a", [[1]]))].data.shape == (5, 1, 1)
