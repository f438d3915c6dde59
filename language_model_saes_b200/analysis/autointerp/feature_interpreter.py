"""Explain features with a chat model and score the explanations
(analysis/autointerp/feature_interpreter.py:47-838 of the reference project).

The chat client is any object with ``await client.chat.completions.create(model=, messages=, ...)`` returning
``.choices[0].message.content`` (the ``openai.AsyncOpenAI`` interface); tests inject a fake one. JSON answers are
parsed leniently: the first balanced ``{...}`` block of the reply is used when the reply is not pure JSON.
"""

from __future__ import annotations

import asyncio
import json
import random
import time
import traceback
from typing import Any, AsyncGenerator, Callable, Literal, Optional

import numpy as np
import torch
from pydantic import BaseModel

from ...backend.language_model import LanguageModel
from ...utils.logging import get_logger
from ..samples import Segment, TokenizedSample
from .autointerp_base import AutoInterpConfig, ExplainerType, ScorerType
from .evaluation_prompts import generate_detection_prompt, generate_fuzzing_prompt
from .explanation_prompts import generate_explanation_prompt, generate_explanation_prompt_neuronpedia

logger = get_logger("analysis.autointerp")


class Step(BaseModel):
    thought: str


class AutoInterpExplanation(BaseModel):
    steps: list[Step]
    final_explanation: str
    activation_consistency: Literal[1, 2, 3, 4, 5]
    complexity: Literal[1, 2, 3, 4, 5]


class AutoInterpEvaluation(BaseModel):
    steps: list[Step]
    evaluation_results: list[bool]


def parse_json_reply(text: str) -> dict[str, Any]:
    """Parse a model reply that should be a JSON object but may be wrapped in prose or a code fence."""
    try:
        out = json.loads(text)
        if isinstance(out, dict):
            return out
    except json.JSONDecodeError:
        pass
    start = text.find("{")
    while start != -1:
        depth, in_str, esc = 0, False, False
        for i in range(start, len(text)):
            c = text[i]
            if in_str:
                esc = (c == "\\") and not esc
                if c == '"' and not esc:
                    in_str = False
                continue
            if c == '"':
                in_str = True
            elif c == "{":
                depth += 1
            elif c == "}":
                depth -= 1
                if depth == 0:
                    try:
                        out = json.loads(text[start : i + 1])
                        if isinstance(out, dict):
                            return out
                    except json.JSONDecodeError:
                        pass
                    break
        start = text.find("{", start + 1)
    raise ValueError(f"no JSON object in reply: {text[:200]!r}")


def _dense_acts(indices, values, n_rows: int | None = None) -> torch.Tensor:
    idx = torch.as_tensor(np.asarray(indices)).long()
    val = torch.as_tensor(np.asarray(values)).float()
    if idx.numel() == 0:
        return torch.zeros(n_rows or 0, 1)
    rows = n_rows if n_rows is not None else int(idx[0].max()) + 1
    out = torch.zeros(rows, int(idx[1].max()) + 1)
    out[idx[0], idx[1]] = val
    return out


def _sampling_rows(sampling):
    n = len(sampling.context_idx)
    shard = sampling.shard_idx if sampling.shard_idx is not None else [0] * n
    n_shards = sampling.n_shards if sampling.n_shards is not None else [1] * n
    return zip(range(n), sampling.dataset_name, shard, n_shards, sampling.context_idx)


def generate_activating_examples(feature, model: LanguageModel, datasets: Callable[[str, int, int], Any], analysis,
                                 n: int = 10, max_length: int = 50) -> list[TokenizedSample]:  # fmt: skip
    """The first sampling's contexts, each cut to ``max_length`` tokens centred on its strongest token."""
    samples: list[TokenizedSample] = []
    if n == 0 or not analysis.samplings:
        return samples
    sampling = analysis.samplings[0]
    acts = _dense_acts(sampling.feature_acts_indices, sampling.feature_acts_values, len(sampling.context_idx))
    z_idx = torch.as_tensor(np.asarray(sampling.z_pattern_indices)).long() if sampling.z_pattern_indices is not None else None
    z_val = torch.as_tensor(np.asarray(sampling.z_pattern_values)).float() if sampling.z_pattern_values is not None else None
    for i, ds_name, shard, n_shards, ctx in _sampling_rows(sampling):
        data = datasets(ds_name, int(shard), int(n_shards))[int(ctx)]
        try:
            origins = model.trace({k: [v] for k, v in data.items()})[0]
        except Exception:  # noqa: BLE001 - a sample that cannot be traced is skipped
            continue
        row = acts[i]
        peak = int(row.argmax())
        lo, hi = max(0, peak - max_length // 2), min(len(origins), peak + max_length // 2)
        row = torch.nn.functional.pad(row, (0, max(0, hi - row.numel())))
        sample = TokenizedSample.construct(data["text"], row[lo:hi], origins[lo:hi], analysis.max_feature_acts)
        if z_idx is not None and z_val is not None:
            sel = z_idx[0] == i
            qk = z_idx[1:, sel]
            inside = (qk < hi).all(dim=0) & (qk >= lo).all(dim=0)
            sample.add_z_pattern_data(qk[:, inside] - lo, z_val[sel][inside], origins[lo:hi])
        samples.append(sample)
        if len(samples) >= n:
            break
    return samples


def generate_non_activating_examples(feature, model: LanguageModel, datasets: Callable[[str, int, int], Any], analysis,
                                     n: int = 10, max_length: int = 50) -> list[TokenizedSample]:  # fmt: skip
    """Contexts of the ``non_activating`` sampling, cut to their first ``max_length`` tokens."""
    samples: list[TokenizedSample] = []
    sampling = next((s for s in analysis.samplings if s.name == "non_activating"), None)
    if n == 0 or sampling is None:
        return samples
    acts = _dense_acts(sampling.feature_acts_indices, sampling.feature_acts_values, len(sampling.context_idx))
    for i, ds_name, shard, n_shards, ctx in _sampling_rows(sampling):
        try:
            data = datasets(ds_name, int(shard), int(n_shards))[int(ctx)]
            origins = model.trace({k: [v] for k, v in data.items()})[0]
            row = torch.nn.functional.pad(acts[i], (0, max(0, max_length - acts[i].numel())))
            samples.append(TokenizedSample.construct(data["text"], row[:max_length], origins[:max_length], analysis.max_feature_acts))
        except Exception as e:  # noqa: BLE001
            logger.error(f"Error processing non-activating examples of feature {feature.index}: {e}")
            continue
        if len(samples) >= n:
            break
    return samples


def _binary_metrics(truth: list[bool], pred: list[bool]) -> dict[str, float]:
    tp = sum(t and p for t, p in zip(truth, pred))
    tn = sum((not t) and (not p) for t, p in zip(truth, pred))
    fp = sum((not t) and p for t, p in zip(truth, pred))
    fn = sum(t and (not p) for t, p in zip(truth, pred))
    div = lambda a, b: a / b if b > 0 else 0  # noqa: E731
    precision, recall = div(tp, tp + fp), div(tp, tp + fn)
    return {
        "accuracy": div(tp + tn, len(truth)),
        "precision": precision,
        "recall": recall,
        "f1": div(2 * precision * recall, precision + recall),
        "balanced_accuracy": (recall + div(tn, tn + fp)) / 2,
    }


def _empty_evaluation(method: str) -> dict[str, Any]:
    return {"method": method, "prompt": "", "response": "", "ground_truth": [], "predictions": [],
            "metrics": {"accuracy": 0, "precision": 0, "recall": 0, "f1": 0, "balanced_accuracy": 0}, "passed": False, "time": 0}  # fmt: skip


class FeatureInterpreter:
    pass_threshold: float = 0.7
    """Balanced accuracy from which an evaluation counts as passed."""

    def __init__(self, cfg: AutoInterpConfig, mongo_client, client: Any | None = None):
        self.cfg = cfg
        self.mongo_client = mongo_client
        self.explainer_client = client if client is not None else self._setup_llm_clients()

    def _setup_llm_clients(self):
        try:
            from openai import AsyncOpenAI
        except ImportError as e:
            raise ImportError("the openai package is needed for automatic interpretation") from e
        http_client = None
        if self.cfg.openai_proxy:
            import httpx

            http_client = httpx.AsyncClient(proxy=self.cfg.openai_proxy)
        return AsyncOpenAI(base_url=self.cfg.openai_base_url, api_key=self.cfg.openai_api_key or "unset", http_client=http_client)

    async def _chat(self, system: str, user: str, as_json: bool) -> tuple[str, float]:
        t0 = time.time()
        kwargs = {"response_format": {"type": "json_object"}} if as_json else {"stream": False}
        resp = await self.explainer_client.chat.completions.create(
            model=self.cfg.openai_model, messages=[{"role": "system", "content": system}, {"role": "user", "content": user}], **kwargs
        )
        content = resp.choices[0].message.content
        assert content is not None, f"No reply from the chat model\n\nsystem_prompt: {system}\n\nuser_prompt: {user}"
        return content, time.time() - t0

    def get_feature_examples(self, feature, model: LanguageModel, datasets, analysis_name: str = "default", max_length: int = 50):
        analysis = next((a for a in feature.analyses if a.name == analysis_name), None)
        if analysis is None:
            raise ValueError(f"Analysis {analysis_name} not found for feature {feature.index}")
        if analysis.max_feature_acts == 0:
            raise ValueError(f"Feature {feature.index} has no activation. Skipping interpretation.")
        act = generate_activating_examples(feature, model, datasets, analysis, self.cfg.n_activating_examples, max_length)
        non = generate_non_activating_examples(feature, model, datasets, analysis, self.cfg.n_non_activating_examples, max_length)
        return act, non

    async def generate_explanation(self, activating_examples: list[TokenizedSample], top_logits=None) -> dict[str, Any]:
        if self.cfg.explainer_type is ExplainerType.OPENAI:
            system, user = generate_explanation_prompt(self.cfg, activating_examples)
            content, dt = await self._chat(system, user, as_json=True)
            explanation = parse_json_reply(content)
        else:
            system, user = generate_explanation_prompt_neuronpedia(self.cfg, activating_examples, top_logits)
            content, dt = await self._chat(system, user, as_json=False)
            explanation = {"final_explanation": content, "activation_consistency": 5, "complexity": 5}
        return {"user_prompt": user, "system_prompt": system, "response": explanation, "time": dt}

    async def _evaluate(self, method: str, system: str, user: str, truth: list[bool], prompt_for_record: str) -> dict[str, Any]:
        content, dt = await self._chat(system, user, as_json=True)
        reply = parse_json_reply(content)
        pred = [bool(p) for p in reply.get("evaluation_results", [])][: len(truth)]
        pred += [False] * (len(truth) - len(pred))
        metrics = _binary_metrics(truth, pred)
        return {"method": method, "prompt": prompt_for_record, "response": reply, "ground_truth": [int(t) for t in truth] if method == "detection" else truth,
                "predictions": pred, "metrics": metrics, "passed": metrics["balanced_accuracy"] >= self.pass_threshold, "time": dt}  # fmt: skip

    async def evaluate_explanation_detection(self, explanation, activating_examples, non_activating_examples) -> dict[str, Any]:
        n = self.cfg.detection_n_examples
        pos = random.sample(activating_examples, min(n, len(activating_examples)))
        neg = random.sample(non_activating_examples, min(n, len(non_activating_examples)))
        if len(pos) + len(neg) < n:
            return _empty_evaluation("detection")
        labelled = [(ex, True) for ex in pos] + [(ex, False) for ex in neg]
        random.shuffle(labelled)
        system, user = generate_detection_prompt(self.cfg, explanation, [ex for ex, _ in labelled])
        return await self._evaluate("detection", system, user, [t for _, t in labelled], system + "\n\n" + user)

    def _create_incorrectly_marked_example(self, sample: TokenizedSample) -> TokenizedSample:
        """Same text, but as many (at least 3) randomly chosen non-firing tokens are marked as firing instead."""
        cut = self.cfg.activation_threshold * sample.max_activation
        n_marked = max(3, sum(seg.activation > cut for seg in sample.segments))
        quiet = [i for i, seg in enumerate(sample.segments) if seg.activation < cut]
        chosen = set(random.sample(quiet, min(n_marked, len(quiet))))
        return TokenizedSample([Segment(seg.text, sample.max_activation if i in chosen else 0) for i, seg in enumerate(sample.segments)],
                               sample.max_activation)  # fmt: skip

    async def evaluate_explanation_fuzzing(self, explanation, activating_examples) -> dict[str, Any]:
        if len(activating_examples) < self.cfg.fuzzing_n_examples:
            return _empty_evaluation("fuzzing")
        n_ok, n_bad = self.cfg.fuzzing_decile_correct, self.cfg.fuzzing_decile_incorrect
        drawn = random.sample(activating_examples, min(n_ok + n_bad, len(activating_examples)))
        labelled = [(ex, True) for ex in drawn[:n_ok]] + [(self._create_incorrectly_marked_example(ex), False) for ex in drawn[n_ok:]]
        random.shuffle(labelled)
        system, user = generate_fuzzing_prompt(self.cfg, explanation, labelled)
        return await self._evaluate("fuzzing", system, user, [t for _, t in labelled], user)

    async def interpret_single_feature(self, activating_examples, non_activating_examples, top_logits=None) -> dict[str, Any]:
        t0 = time.time()
        exp = await self.generate_explanation(activating_examples, top_logits)
        explanation = exp["response"]
        evaluations = []
        if ScorerType.DETECTION in self.cfg.scorer_type:
            evaluations.append(await self.evaluate_explanation_detection(explanation, activating_examples, non_activating_examples))
        if ScorerType.FUZZING in self.cfg.scorer_type:
            evaluations.append(await self.evaluate_explanation_fuzzing(explanation, activating_examples))
        return {
            "explanation": explanation.get("final_explanation"),
            "complexity": explanation.get("complexity"),
            "consistency": explanation.get("activation_consistency"),
            "explanation_details": exp,
            "evaluations": evaluations,
            "passed": any(e["passed"] for e in evaluations),
            "time": {"total": time.time() - t0, "response": exp["time"] + sum(e["time"] for e in evaluations)},
        }

    async def interpret_features(self, sae_name: str, sae_series: str, model: LanguageModel, datasets, analysis_name: str = "default",
                                 feature_indices: Optional[list[int]] = None, max_concurrent: int = 10,
                                 progress_callback: Optional[Callable[[int, int, int], None]] = None) -> AsyncGenerator[dict[str, Any], None]:  # fmt: skip
        """Yield one result per interpreted feature, at most ``max_concurrent`` requests in flight. Features that have
        an interpretation (unless ``overwrite_existing``) or never fired are skipped; errors are logged and counted."""
        if feature_indices is None:
            rec = self.mongo_client.get_sae(sae_name, sae_series)
            assert rec is not None, f"SAE {sae_name} {sae_series} not found"
            feature_indices = list(range(rec.cfg.d_sae))
        gate = asyncio.Semaphore(max_concurrent)

        async def one(idx: int):
            async with gate:
                try:
                    feature = self.mongo_client.get_feature(sae_name, sae_series, idx)
                    todo = (
                        feature is not None
                        and (self.cfg.overwrite_existing or feature.interpretation is None or feature.interpretation.get("text") is None)
                        and len(feature.analyses) > 0
                        and feature.analyses[0].act_times > 0
                    )
                    if not todo:
                        return None, idx, "skipped"
                    act, non = self.get_feature_examples(feature, model, datasets, analysis_name, self.cfg.max_length)
                    res = await self.interpret_single_feature(act, non, feature.logits)
                    return {"feature_index": feature.index, "sae_name": sae_name, "sae_series": sae_series} | res, idx, "done"
                except Exception as e:  # noqa: BLE001
                    logger.error(f"Error interpreting feature {idx}:\n{e}\n{traceback.format_exc()}")
                    return None, idx, "failed"

        counts = {"done": 0, "skipped": 0, "failed": 0}
        for fut in asyncio.as_completed([one(i) for i in feature_indices]):
            res, idx, status = await fut
            counts[status] += 1
            if status == "done":
                yield res
            if progress_callback is not None:
                progress_callback(sum(counts.values()), len(feature_indices), idx)
        logger.info(f"Interpretation complete: {counts['done']} completed, {counts['skipped']} skipped, {counts['failed']} failed "
                    f"out of {len(feature_indices)} total")  # fmt: skip
