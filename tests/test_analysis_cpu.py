"""Feature analysis, samples and auto-interpretation on CPU with tiny models and a fake chat client.
The selection logic is checked against a brute-force restatement over the whole stream."""

import asyncio
import json

import numpy as np
import pytest
import torch

from language_model_saes_b200.analysis import FeatureAnalyzer, FeatureAnalyzerConfig, Segment, TokenizedSample
from language_model_saes_b200.analysis.autointerp import AutoInterpConfig, FeatureInterpreter, ScorerType
from language_model_saes_b200.analysis.autointerp.feature_interpreter import _binary_metrics, parse_json_reply
from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder


class _FakeFactory:
    """Stands in for the activation factory: replays a fixed list of 2-D batches."""

    def __init__(self, batches):
        self.batches = batches

    def process(self, **kwargs):
        return iter(self.batches)


def _stream(n_batches=4, batch=3, ctx=8, d=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    out, c = [], 0
    for _ in range(n_batches):
        out.append({
            "h": torch.randn(batch, ctx, d, generator=g),
            "tokens": torch.randint(1, 50, (batch, ctx), generator=g),
            "meta": [{"context_idx": c + i, "dataset_name": "ds" if (c + i) % 2 == 0 else "other", "model_name": "m"} for i in range(batch)],
        })  # fmt: skip
        c += batch
    return out


def _sae(d=16, f=32):
    torch.manual_seed(1)
    cfg = SAEConfig(hook_point_in="h", hook_point_out="h", d_model=d, expansion_factor=f // d, act_fn="relu", device="cpu", dtype=torch.float32)
    sae = SparseAutoEncoder(cfg)
    sae.init_parameters(encoder_uniform_bound=0.5, decoder_uniform_bound=0.5)
    return sae


def test_feature_analyzer_matches_bruteforce():
    sae, batches = _sae(), _stream()
    cfg = FeatureAnalyzerConfig(total_analyzing_tokens=10**6, ignore_token_ids=[], subsamples={
        "top_activations": {"proportion": 1.0, "n_samples": 4}, "non_activating": {"proportion": 0.3, "n_samples": 2}})  # fmt: skip
    res = FeatureAnalyzer(cfg).analyze_chunk(_FakeFactory(batches), sae)
    assert len(res) == sae.cfg.d_sae
    acts = torch.cat([sae.encode(b["h"]) for b in batches]).detach()  # [contexts, ctx, F]
    peak = acts.amax(dim=1)
    for f in (0, 5, 17, 31):
        r = res[f]
        assert r["act_times"] == int((acts[..., f] > 0).sum())
        assert r["n_analyzed_tokens"] == acts.shape[0] * acts.shape[1]
        assert abs(r["max_feature_acts"] - float(acts[..., f].max())) < 1e-6
        top = next(s for s in r["samplings"] if s["name"] == "top_activations")
        want = torch.argsort(peak[:, f], descending=True, stable=True)[:4]
        want = [int(i) for i in want if peak[i, f] > -1]
        assert list(top["context_idx"]) == want
        assert top["dataset_name"] == ["ds" if i % 2 == 0 else "other" for i in want]
        dense = np.zeros((len(want), acts.shape[1]), dtype=np.float32)
        idx = top["feature_acts_indices"].astype(int)
        dense[idx[0], idx[1]] = top["feature_acts_values"]
        np.testing.assert_allclose(dense, acts[want, :, f].numpy(), rtol=1e-6)
        assert list(top["shard_idx"]) == [0] * len(want) and list(top["n_shards"]) == [1] * len(want)


def test_feature_analyzer_respects_ignore_tokens_and_token_budget():
    sae, batches = _sae(), _stream()
    cfg = FeatureAnalyzerConfig(total_analyzing_tokens=3 * 8 * 2, ignore_token_ids=list(range(1, 25)))
    res = FeatureAnalyzer(cfg).analyze_chunk(_FakeFactory(batches), sae)
    toks = torch.cat([b["tokens"] for b in batches[:2]])
    assert res[0]["n_analyzed_tokens"] == int((toks >= 25).sum())
    acts = torch.cat([sae.encode(b["h"]) for b in batches[:2]]).detach() * (toks >= 25)[..., None]
    assert res[3]["act_times"] == int((acts[..., 3] > 0).sum())


def test_mask_is_used_when_no_ignore_list():
    sae, batches = _sae(), _stream(n_batches=1)
    batches[0]["mask"] = torch.zeros(3, 8, dtype=torch.bool)
    batches[0]["mask"][:, :2] = True
    res = FeatureAnalyzer(FeatureAnalyzerConfig(total_analyzing_tokens=100)).analyze_chunk(_FakeFactory(batches), sae)
    assert res[0]["n_analyzed_tokens"] == 6


def test_tokenized_sample_segments_and_displays():
    text = "The cat sat"
    origins = [{"key": "text", "range": (0, 3)}, {"key": "text", "range": (3, 7)}, None, {"key": "text", "range": (7, 11)}]
    s = TokenizedSample.construct(text, torch.tensor([0.1, 2.0, 9.0, 0.5]), origins, max_activation=2.0)
    assert [seg.text for seg in s.segments] == ["The", " cat", " sat"]
    assert [seg.activation for seg in s.segments] == pytest.approx([0.1, 2.0, 0.5])
    assert s.display_highlighted(0.7) == "The<< cat>> sat"
    assert s.display_plain() == text
    assert s.display_max(0.7) == "(The)  cat\n"
    assert s.display_next(0.7) == " sat\n"
    assert s.sample_max_activation == 2.0
    assert len(s.to_max_activation_surrounding(1).segments) == 2
    s.add_z_pattern_data(torch.tensor([[1, 1], [0, 1]]), torch.tensor([0.9, 0.1]), origins)
    assert s.z_pattern_data[1].contributing_indices == [0, 1] and s.z_pattern_data[1].max_contribution == pytest.approx(0.9)
    assert s.display_max(0.7).startswith("[() The] => ")
    assert Segment("a\n", 1.0).display_max(0.5) == "a\n\n"


def test_parse_json_reply_and_metrics():
    assert parse_json_reply('{"a": 1}') == {"a": 1}
    assert parse_json_reply('Here you go:\n```json\n{"evaluation_results": [true, false]}\n```') == {"evaluation_results": [True, False]}
    with pytest.raises(ValueError):
        parse_json_reply("no json here")
    m = _binary_metrics([True, True, False, False], [True, False, False, True])
    assert m["accuracy"] == 0.5 and m["precision"] == 0.5 and m["recall"] == 0.5 and m["balanced_accuracy"] == 0.5


class _FakeChat:
    """``client.chat.completions.create`` of the OpenAI async interface; answers depend on the system prompt."""

    def __init__(self):
        self.calls = []
        self.chat = self
        self.completions = self

    async def create(self, model, messages, **kwargs):
        self.calls.append(messages)
        system, user = messages[0]["content"], messages[1]["content"]
        if "evaluation_results" in system:
            n = user.count("Example ")
            # detection: say true when the plain text has the word cat; fuzzing: true when cat is highlighted
            lines = [ln for ln in user.splitlines() if ln.startswith("Example ")]
            if "<<" in system:
                res = ["<< cat>>" in ln for ln in lines]
            else:
                res = [" cat" in ln for ln in lines]
            assert len(res) == n
            content = json.dumps({"steps": [], "evaluation_results": res})
        else:
            content = json.dumps({"steps": [{"thought": "t"}], "final_explanation": "the word cat", "activation_consistency": 5, "complexity": 1})
        msg = type("M", (), {"content": content})
        return type("R", (), {"choices": [type("C", (), {"message": msg})]})


def _cat_sample(active: bool):
    words = ["The", " cat" if active else " dog", " sat", " on", " a", " mat"]
    return TokenizedSample([Segment(w, 3.0 if w == " cat" else 0.0) for w in words], 3.0)


def test_interpreter_explains_and_scores_with_fake_client():
    chat = _FakeChat()
    cfg = AutoInterpConfig(scorer_type=[ScorerType.DETECTION, ScorerType.FUZZING], fuzzing_decile_correct=3, fuzzing_decile_incorrect=2)
    it = FeatureInterpreter(cfg, mongo_client=None, client=chat)
    pos = [_cat_sample(True) for _ in range(6)]
    neg = [_cat_sample(False) for _ in range(6)]
    out = asyncio.run(it.interpret_single_feature(pos, neg))
    assert out["explanation"] == "the word cat" and out["complexity"] == 1 and out["consistency"] == 5
    det, fuzz = out["evaluations"]
    assert det["method"] == "detection" and det["metrics"]["balanced_accuracy"] == 1.0 and det["passed"]
    assert fuzz["method"] == "fuzzing" and fuzz["metrics"]["accuracy"] == 1.0 and fuzz["passed"]
    assert out["passed"] and len(chat.calls) == 3
    bad = it._create_incorrectly_marked_example(pos[0])
    assert sum(seg.activation > 0 for seg in bad.segments) == 3 and bad.segments[1].activation == 0


def test_interpreter_too_few_examples_gives_empty_evaluation():
    it = FeatureInterpreter(AutoInterpConfig(), mongo_client=None, client=_FakeChat())
    out = asyncio.run(it.evaluate_explanation_fuzzing({"final_explanation": "x"}, [_cat_sample(True)]))
    assert out["passed"] is False and out["ground_truth"] == []
