"""Serialisation of attribution results (``core/serialize.py`` + ``circuits/attribution.py``): every field survives a
dump / load cycle, optional fields may be absent, and blobs written before the QK tracing result had marginals (format
version 1: ``qk_trace_results`` is the bare list of pairs) still load, with empty marginals filled in. The cases follow
tests/unit/test_serialize.py of the reference project."""

import pickle

import torch

from language_model_saes_b200.circuits.attribution import AttributionResult, QKTracingResult
from language_model_saes_b200.circuits.indexed_tensor import NodeDimension, NodeIndexed, NodeIndexedMatrix, NodeIndexedVector, NodeInfo
from language_model_saes_b200.core import serialize
from language_model_saes_b200.core.serialize import dump, dumps, load, loads, unstructure


def _dim(key: str, n: int, width: int = 1) -> NodeDimension:
    idx = torch.arange(n * width).view(n, width)
    return NodeDimension.from_node_infos([NodeInfo(key=key, indices=idx)])


def _pairs() -> NodeIndexed:
    return NodeIndexed(
        value=[NodeIndexed(value=torch.tensor([1.5, 2.5]), dimensions=(_dim("q", 2), _dim("k", 2))),
               NodeIndexed(value=torch.tensor([3.5]), dimensions=(_dim("q", 1), _dim("k", 1)))],
        dimensions=(_dim("target", 2),),
    )  # fmt: skip


def _result(with_qk: bool) -> AttributionResult:
    torch.manual_seed(0)
    targets, sources = _dim("layer_0", 3), _dim("layer_1", 4, width=2)
    qk = None
    if with_qk:
        marg = lambda side: NodeIndexed(value=[NodeIndexed(value=torch.tensor([0.25, 0.75]), dimensions=(_dim(side, 2),)),
                                               NodeIndexed(value=torch.tensor([1.0]), dimensions=(_dim(side, 1),))],
                                        dimensions=(_dim("target", 2),))  # noqa: E731  # fmt: skip
        qk = QKTracingResult(q_marginal=marg("q"), k_marginal=marg("k"), pairs=_pairs())
    return AttributionResult(
        activations=NodeIndexedVector.from_data(torch.randn(3), (targets,)),
        attribution=NodeIndexedMatrix.from_data(torch.randn(3, 4), (targets, sources)),
        targets=targets, logits=torch.randn(5), probs=torch.softmax(torch.randn(5), dim=0), prompt_token_ids=[1, 2, 3],
        prompt_tokens=["<bos>", "a", "b"], logit_token_ids=[4, 5], logit_tokens=["c", "d"], qk_trace_results=qk,
    )  # fmt: skip


def _same(a: AttributionResult, b: AttributionResult) -> None:
    assert torch.equal(a.activations.data, b.activations.data) and a.activations.dimensions == b.activations.dimensions
    assert torch.equal(a.attribution.data, b.attribution.data) and a.attribution.dimensions == b.attribution.dimensions
    assert torch.equal(a.logits, b.logits) and torch.equal(a.probs, b.probs) and a.targets == b.targets
    assert a.prompt_token_ids == b.prompt_token_ids and a.prompt_tokens == b.prompt_tokens
    assert a.logit_token_ids == b.logit_token_ids and a.logit_tokens == b.logit_tokens


def test_dump_is_a_versioned_plain_structure():
    blob = dump(_result(with_qk=True))
    assert set(blob) == {"_version", "data"} and blob["_version"] == serialize.FORMAT_VERSION
    data = blob["data"]
    assert isinstance(data, dict) and {"activations", "attribution", "logits", "prompt_tokens", "qk_trace_results"} <= set(data)
    assert isinstance(data["logits"], torch.Tensor) and data["prompt_tokens"] == ["<bos>", "a", "b"]
    assert set(data["qk_trace_results"]) == {"q_marginal", "k_marginal", "pairs"}
    pickle.loads(pickle.dumps(blob))  # nothing but containers, tensors and scalars: a database can store it


def test_load_restores_every_field():
    res = _result(with_qk=True)
    again = load(dump(res), AttributionResult)
    assert isinstance(again, AttributionResult) and isinstance(again.attribution, NodeIndexedMatrix) and isinstance(again.activations, NodeIndexedVector)
    _same(res, again)
    qk = again.qk_trace_results
    assert isinstance(qk, QKTracingResult) and len(qk.pairs.value) == 2
    assert torch.equal(qk.pairs.value[0].value, torch.tensor([1.5, 2.5])) and torch.equal(qk.q_marginal.value[1].value, torch.tensor([1.0]))
    assert qk.pairs.value[0].dimensions[1] == _dim("k", 2) and qk.pairs.dimensions[0] == _dim("target", 2)
    _same(res, loads(dumps(res), AttributionResult))  # the byte form too


def test_optional_fields_may_be_absent():
    res = _result(with_qk=False)
    res.logit_token_ids = res.logit_tokens = None
    again = loads(dumps(res), AttributionResult)
    assert again.qk_trace_results is None and again.logit_token_ids is None and again.logit_tokens is None
    _same(res, again)


def test_legacy_blob_with_bare_qk_pairs_still_loads():
    res = _result(with_qk=False)
    legacy = {
        "_version": "1",
        "data": {
            "activations": unstructure(res.activations), "attribution": unstructure(res.attribution), "logits": res.logits, "probs": res.probs,
            "prompt_token_ids": [1, 2, 3], "prompt_tokens": ["<bos>", "a", "b"], "logit_token_ids": [4, 5], "logit_tokens": ["c", "d"],
            "qk_trace_results": unstructure(_pairs()),  # the shape before the marginals existed
        },
    }  # fmt: skip
    got = load(legacy, AttributionResult)
    qk = got.qk_trace_results
    assert isinstance(qk, QKTracingResult)
    assert len(qk.pairs.value) == 2 and torch.equal(qk.pairs.value[0].value, torch.tensor([1.5, 2.5])) and torch.equal(qk.pairs.value[1].value, torch.tensor([3.5]))
    # the marginals are filled in: one zero vector per target over the pair's q / k nodes
    assert len(qk.q_marginal.value) == 2 and len(qk.k_marginal.value) == 2
    assert torch.equal(qk.q_marginal.value[0].value, torch.zeros(2)) and torch.equal(qk.k_marginal.value[1].value, torch.zeros(1))
    assert qk.q_marginal.value[0].dimensions[0] == _dim("q", 2) and qk.k_marginal.value[0].dimensions[0] == _dim("k", 2)
    assert qk.q_marginal.dimensions[0] == _dim("target", 2)
    assert got.targets is None and torch.equal(got.attribution.data, res.attribution.data)
    # a blob of the current version is NOT migrated: the same payload under version 2 must fail to structure
    try:
        load({**legacy, "_version": serialize.FORMAT_VERSION}, AttributionResult)
        raise AssertionError("a bare pair list is not a current QKTracingResult")
    except AssertionError:
        raise
    except Exception:  # noqa: BLE001
        pass
