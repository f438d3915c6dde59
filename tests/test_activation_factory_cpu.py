"""``ActivationFactory`` end to end on a stand-in model: every target level, batching, several weighted sources, cached
activations as a source, the interceptor hook and the refusals. The expected behaviour is the reference project's
(tests/integration/test_activation_factory.py there; activation/factory.py:37-330)."""

import json

import pytest
import torch
from datasets import Dataset
from safetensors.torch import save_file

from language_model_saes_b200 import (
    ActivationFactoryActivationsSource,
    ActivationFactoryConfig,
    ActivationFactoryDatasetSource,
    ActivationFactoryTarget,
)
from language_model_saes_b200.activation.factory import ActivationFactory


class CountingModel:
    """Every text becomes three tokens (1 = eos, 2 = bos, 3) of which the mask keeps the last, with activations that name
    their hook point and position."""

    eos_token_id, pad_token_id, bos_token_id = 1, 0, 2

    def __init__(self):
        self.calls = []

    def to_activations(self, raw, hook_points, **kwargs):
        assert "text" in raw
        self.calls.append((list(raw["text"]), tuple(hook_points)))
        n = len(raw["text"])
        out = {hp: (torch.arange(9.0) + 9 * i).reshape(1, 3, 3).repeat(n, 1, 1) for i, hp in enumerate(hook_points)}
        out["tokens"] = (torch.arange(3) + 1).reshape(1, 3).repeat(n, 1)
        out["mask"] = ~torch.isin(out["tokens"], torch.tensor([self.eos_token_id, self.pad_token_id, self.bos_token_id]))
        return out

    def preprocess_raw_data(self, raw):
        return raw


@pytest.fixture
def texts():
    return Dataset.from_dict({"text": ["Hello world", "Test text", "Another example"]})


def config(**over):
    base = dict(sources=[ActivationFactoryDatasetSource(name="ds", prepend_bos=True, sample_weights=1.0)], target=ActivationFactoryTarget.ACTIVATIONS_1D,
                hook_points=["h0", "h1"], context_size=4, num_workers=0, model_batch_size=1, batch_size=None, buffer_size=None)  # fmt: skip
    base.update(over)
    return ActivationFactoryConfig(**base)


def run(cfg, texts, model=None, **kw):
    return list(ActivationFactory(cfg, **kw).process(model=model or CountingModel(), model_name="m", datasets={s.name: (texts, None) for s in cfg.sources}))


def test_factory_is_assembled_from_its_config():
    cfg = config()
    f = ActivationFactory(cfg)
    assert f.cfg == cfg and len(f.pre_aggregation_processors) == 1
    assert callable(f.post_aggregation_processor) and callable(f.aggregator)
    two = ActivationFactory(config(sources=[ActivationFactoryDatasetSource(name="a", sample_weights=0.5), ActivationFactoryDatasetSource(name="b", sample_weights=0.5)]))
    assert len(two.pre_aggregation_processors) == 2


def test_two_dimensional_target_keeps_the_context_axis_and_the_sample_info(texts):
    out = run(config(target=ActivationFactoryTarget.ACTIVATIONS_2D), texts)
    assert len(out) == 3  # one record per text
    assert out[0]["h0"].shape == (1, 3, 3) and torch.equal(out[0]["h0"], torch.arange(9.0).reshape(1, 3, 3))
    assert torch.equal(out[0]["h1"], torch.arange(9.0, 18.0).reshape(1, 3, 3))
    assert out[0]["meta"][0]["dataset_name"] == "ds" and out[2]["meta"][0]["context_idx"] == 2


def test_one_dimensional_target_drops_pad_eos_and_bos_positions(texts):
    out = run(config(), texts)
    # tokens 1 (eos) and 2 (bos) are filtered: only the third position of every text is left
    assert len(out) == 3 and out[0]["h0"].shape == (1, 3)
    assert torch.equal(out[0]["h0"], torch.tensor([[6.0, 7.0, 8.0]])) and torch.equal(out[0]["h1"], torch.tensor([[15.0, 16.0, 17.0]]))
    assert torch.equal(out[0]["tokens"].reshape(-1), torch.tensor([3]))


def test_a_list_of_ignored_token_ids_replaces_the_mask(texts):
    out = run(config(ignore_token_ids=[3]), texts)
    assert len(out) == 3 and torch.equal(out[0]["tokens"], torch.tensor([1, 2]))  # eos and bos stay, only id 3 goes
    assert torch.equal(out[0]["h0"], torch.arange(6.0).reshape(2, 3))


def test_batching_of_token_rows_regroups_them_and_forgets_the_sample_info(texts):
    out = run(config(batch_size=2), texts)
    assert [o["h0"].shape[0] for o in out] == [2, 1]
    assert torch.equal(out[0]["h0"], torch.tensor([[6.0, 7.0, 8.0]] * 2)) and torch.equal(out[1]["h0"], torch.tensor([[6.0, 7.0, 8.0]]))
    assert "meta" not in out[0]


def test_batching_of_sequences_keeps_the_sample_info(texts):
    out = run(config(target=ActivationFactoryTarget.ACTIVATIONS_2D, batch_size=2), texts)
    assert [tuple(o["h0"].shape) for o in out] == [(2, 3, 3), (1, 3, 3)]
    assert torch.equal(out[0]["h0"], torch.arange(9.0).reshape(1, 3, 3).repeat(2, 1, 1))
    assert out[0]["meta"][0]["dataset_name"] == "ds" and len(out[0]["meta"]) == 2


def test_lower_targets_stop_before_the_model(texts):
    model = CountingModel()
    raw = run(config(target=ActivationFactoryTarget.TOKENS), texts, model=model)
    assert len(raw) == 3 and "h0" not in raw[0]
    assert model.calls == []  # activations were never asked for


def test_the_model_is_asked_in_batches_of_model_batch_size(texts):
    model = CountingModel()
    out = run(config(target=ActivationFactoryTarget.ACTIVATIONS_2D, model_batch_size=2), texts, model=model)
    assert [len(t) for t, _ in model.calls] == [2, 1] and all(h == ("h0", "h1") for _, h in model.calls)
    assert sum(o["h0"].shape[0] for o in out) == 3


def test_several_sources_are_interleaved_until_all_are_exhausted(texts):
    torch.manual_seed(0)
    cfg = config(target=ActivationFactoryTarget.ACTIVATIONS_2D, sources=[ActivationFactoryDatasetSource(name="a", prepend_bos=True, sample_weights=0.7),
                                                                        ActivationFactoryDatasetSource(name="b", prepend_bos=False, sample_weights=0.3)])  # fmt: skip
    out = run(cfg, texts)
    names = [o["meta"][0]["dataset_name"] for o in out]
    assert sorted(names) == ["a"] * 3 + ["b"] * 3
    for src in ("a", "b"):  # every source keeps its own order
        assert [o["meta"][0]["context_idx"] for o in out if o["meta"][0]["dataset_name"] == src] == [0, 1, 2]


def test_missing_inputs_are_named(texts):
    f = ActivationFactory(config())
    with pytest.raises(AssertionError, match="Dataset ds not found in `datasets`"):
        list(f.process(model=CountingModel(), model_name="m", datasets={}))
    with pytest.raises(AssertionError, match="`model` must be provided for dataset sources"):
        list(f.process(datasets={"ds": (texts, None)}))
    with pytest.raises(AssertionError, match="`model_name` must be provided for dataset sources"):
        list(f.process(model=CountingModel(), datasets={"ds": (texts, None)}))


def _write_cache(root, hook, chunks=2, n=2, ctx=3, d=4):
    (root / hook).mkdir()
    g = torch.Generator().manual_seed(len(hook))
    tokens = torch.randint(3, 1000, (n, ctx), generator=g)
    for i in range(chunks):
        save_file({"activation": torch.randn(n, ctx, d, generator=g), "tokens": tokens, "mask": torch.ones(n, ctx, dtype=torch.bool),
                   "attention_mask": torch.ones(n, ctx, dtype=torch.bool)}, str(root / hook / f"chunk-{i}.safetensors"))  # fmt: skip
        (root / hook / f"chunk-{i}.meta.json").write_text(json.dumps([{"context_id": f"ctx_{j}"} for j in range(n)]))
    return tokens


def test_cached_activations_as_a_source(tmp_path):
    tokens = _write_cache(tmp_path, "h0")
    src = ActivationFactoryActivationsSource(name="cache", path=str(tmp_path), sample_weights=1.0, device="cpu", dtype=None, num_workers=0, prefetch=None)
    out = list(ActivationFactory(config(sources=[src], target=ActivationFactoryTarget.ACTIVATIONS_2D, hook_points=["h0"])).process())
    assert len(out) == 2  # one record per chunk
    for o in out:
        assert o["h0"].shape == (2, 3, 4) and torch.equal(o["tokens"], tokens)
        assert [m["context_id"] for m in o["meta"]] == ["ctx_0", "ctx_1"]
    flat = list(ActivationFactory(config(sources=[src], target=ActivationFactoryTarget.ACTIVATIONS_1D, hook_points=["h0"], batch_size=4)).process())
    assert [o["h0"].shape for o in flat] == [(4, 4), (4, 4), (4, 4)]  # 2 chunks x 2 samples x 3 tokens, regrouped by four


def test_cached_activations_cannot_feed_a_target_below_activations():
    src = ActivationFactoryActivationsSource(name="cache", path="nowhere", sample_weights=1.0, device="cpu", dtype=None, num_workers=0, prefetch=2)
    with pytest.raises(ValueError, match="Activations sources are only supported for target >= ACTIVATIONS_2D"):
        ActivationFactory(config(sources=[src], target=ActivationFactoryTarget.TOKENS))


def test_interceptor_sees_every_record_with_the_index_of_its_source(texts):
    seen = []

    def tag(record, source_idx):
        seen.append(source_idx)
        record["source_idx"] = source_idx
        return record

    cfg = config(target=ActivationFactoryTarget.ACTIVATIONS_2D, sources=[ActivationFactoryDatasetSource(name="a", sample_weights=0.5),
                                                                        ActivationFactoryDatasetSource(name="b", sample_weights=0.5)])  # fmt: skip
    out = run(cfg, texts, before_aggregation_interceptor=tag)
    assert len(out) == 6 and sorted(seen) == [0, 0, 0, 1, 1, 1]
    assert all(o["source_idx"] == (0 if o["meta"][0]["dataset_name"] == "a" else 1) for o in out)


def test_override_dtype_casts_the_activations_only(texts):
    out = run(config(target=ActivationFactoryTarget.ACTIVATIONS_2D, override_dtype=torch.bfloat16), texts)
    assert out[0]["h0"].dtype == torch.bfloat16 and out[0]["tokens"].dtype == torch.int64
