"""``/dictionaries``: browse dictionaries, features, samples; run inference on text; interpretations and bookmarks
(server/routers/dictionaries.py of the reference project; same paths and payloads, msgpack for the large ones)."""

from __future__ import annotations

import json
from typing import Any, Optional

import numpy as np
import torch
from fastapi import APIRouter, Response
from pydantic import BaseModel

from .. import config as C
from ..common import make_serializable, natural_sort_key, packed
from ..loaders import get_model, get_sae
from ..samples import cached_extract_samples, list_feature_data

router = APIRouter(prefix="/dictionaries", tags=["dictionaries"])


def _filters(raw: str | None):
    if not raw:
        return None, None
    try:
        return json.loads(raw), None
    except (json.JSONDecodeError, TypeError):
        return None, Response(content=f"Invalid metric_filters format: {raw}", status_code=400)


def _analysis(feature, name: str | None):
    return next((a for a in feature.analyses if name is None or a.name == name), None)


@router.get("")
def list_dictionaries():
    return sorted(C.client.list_saes(sae_series=C.sae_series, has_analyses=True), key=natural_sort_key)


@router.get("/{name}/metrics")
def get_available_metrics(name: str):
    return {"metrics": C.client.get_available_metrics(name, sae_series=C.sae_series)}


@router.get("/{name}/features/count")
def count_features_with_filters(name: str, feature_analysis_name: str | None = None, metric_filters: str | None = None):
    parsed, err = _filters(metric_filters)
    if err is not None:
        return err
    return {"count": C.client.count_features_with_filters(sae_name=name, sae_series=C.sae_series, name=feature_analysis_name, metric_filters=parsed)}


@router.get("/{name}/features/{feature_index}")
def get_feature(name: str, feature_index: str, feature_analysis_name: str | None = None, metric_filters: str | None = None, no_samplings: bool = False):
    """``feature_index`` is an integer or ``random`` (a random feature that fired, honouring the filters)."""
    parsed, err = _filters(metric_filters)
    if err is not None:
        return err
    if feature_index == "random":
        feature = C.client.get_random_alive_feature(sae_name=name, sae_series=C.sae_series, name=feature_analysis_name or "default", metric_filters=parsed)
    else:
        try:
            feature = C.client.get_feature(sae_name=name, sae_series=C.sae_series, index=int(feature_index))
        except ValueError:
            return Response(content=f"Feature index {feature_index} is not a valid integer", status_code=400)
    if feature is None:
        return Response(content=f"Feature {feature_index} not found in SAE {name}", status_code=404)
    analysis = _analysis(feature, feature_analysis_name)
    if analysis is None:
        msg = f"Feature analysis {feature_analysis_name} not found in SAE {name}" if feature_analysis_name else f"No feature analysis found in SAE {name}"
        return Response(content=msg, status_code=404)
    groups = None if no_samplings else [
        {"analysis_name": s.name, "samples": cached_extract_samples(name, C.sae_series, feature.index, s.name, 0, len(s.context_idx))}
        for s in analysis.samplings
    ]  # fmt: skip
    return packed({
        "feature_index": feature.index, "analysis_name": analysis.name, "interpretation": feature.interpretation,
        "dictionary_name": feature.sae_name, "logits": feature.logits, "decoder_norms": analysis.decoder_norms,
        "decoder_similarity_matrix": analysis.decoder_similarity_matrices, "decoder_inner_product_matrix": analysis.decoder_inner_product_matrices,
        "act_times": analysis.act_times, "max_feature_act": analysis.max_feature_acts, "n_analyzed_tokens": analysis.n_analyzed_tokens,
        "sample_groups": groups, "is_bookmarked": C.client.is_bookmarked(sae_name=name, sae_series=C.sae_series, feature_index=feature.index),
    })  # fmt: skip


@router.get("/{name}/features")
def list_features(name: str, start: int, end: int, analysis_name: str | None = None, sample_length: int = 1, visible_range: int | None = None):
    out = []
    for feature in C.client.list_features(sae_name=name, sae_series=C.sae_series, indices=list(range(start, end))):
        analysis = _analysis(feature, analysis_name)
        if analysis is None:
            out.append(None)
            continue
        sampling = next((s for s in analysis.samplings if s.name == "top_activations"), None)
        samples = cached_extract_samples(name, C.sae_series, feature.index, sampling.name, 0, sample_length, visible_range=visible_range) if sampling else None
        out.append({"feature_index": feature.index, "analysis_name": analysis.name, "interpretation": feature.interpretation,
                    "dictionary_name": feature.sae_name, "act_times": analysis.act_times, "max_feature_act": analysis.max_feature_acts,
                    "n_analyzed_tokens": analysis.n_analyzed_tokens, "samples": samples})  # fmt: skip
    return make_serializable(out)


@router.get("/{name}/features/{feature_index}/samplings")
def get_samplings(name: str, feature_index: int, analysis_name: str | None = None):
    feature = C.client.get_feature(sae_name=name, sae_series=C.sae_series, index=feature_index)
    if feature is None:
        return Response(content=f"Feature {feature_index} not found in SAE {name}", status_code=404)
    analysis = _analysis(feature, analysis_name)
    if analysis is None:
        return Response(content=f"Analysis {analysis_name} not found in SAE {name}", status_code=404)
    return [{"name": s.name, "length": len(s.context_idx)} for s in analysis.samplings]


@router.get("/{name}/features/{feature_index}/sampling/{sampling_name}")
def get_samples(name: str, feature_index: int, sampling_name: str, analysis_name: str | None = None, start: int = 0,
                length: int | None = None, visible_range: int | None = None):  # fmt: skip
    return packed(cached_extract_samples(name, C.sae_series, feature_index, sampling_name, start, None if length is None else start + length,
                                         visible_range=visible_range))  # fmt: skip


def activation_histogram(act_times: dict[int, int], bins: int = 100) -> dict[str, Any]:
    """log10 activation-count histogram as a plotly-style trace (plain JSON, no plotting library needed)."""
    x = np.log10(np.maximum(np.asarray(list(act_times.values()), dtype=np.float64), 1e-12))
    counts, edges = np.histogram(x, bins=bins) if x.size else (np.zeros(0), np.zeros(1))
    return {"type": "bar", "x": ((edges[:-1] + edges[1:]) / 2).tolist(), "y": counts.tolist(), "marker": {"color": "#636EFA"},
            "hovertemplate": "Count: %{y}<br>Range: %{x}<extra></extra>", "showlegend": False}  # fmt: skip


@router.get("/{name}")
def get_dictionary(name: str):
    times = C.client.get_feature_act_times(name, sae_series=C.sae_series)
    if times is None:
        return Response(content=f"Dictionary {name} not found", status_code=404)
    alive = C.client.get_alive_feature_count(name, sae_series=C.sae_series)
    if alive is None:
        return Response(content=f"SAE {name} not found", status_code=404)
    return packed({"dictionary_name": name, "feature_activation_times_histogram": [activation_histogram(times)], "alive_feature_count": alive})


@router.get("/{name}/analyses")
def get_analyses(name: str):
    return C.client.list_analyses(name, C.sae_series)


def _encode_text(name: str, text: str):
    model_name = C.client.get_sae_model_name(name, C.sae_series)
    assert model_name is not None, f"SAE {name} not found or no model name is associated with it"
    model, sae = get_model(name=model_name), get_sae(name=name)
    with torch.no_grad():
        acts = sae.normalize_activations(model.to_activations({"text": [text]}, hook_points=sae.cfg.associated_hook_points))
        x, kwargs, _ = sae.prepare_input(acts)
        feature_acts = sae.encode(x, **kwargs)
    return model, feature_acts


@router.post("/{name}/features/{feature_index}/infer")
def infer_feature(name: str, feature_index: int, text: str):
    """Activations of one feature on a given text."""
    model, feature_acts = _encode_text(name, text)
    row = feature_acts[0, :, feature_index].float()
    pos = row.nonzero().squeeze(-1)
    return packed({"text": text, "origins": model.trace({"text": [text]})[0], "feature_acts_indices": pos, "feature_acts_values": row[pos]})


class UpdateInterpretationRequest(BaseModel):
    text: str


@router.put("/{name}/features/{feature_index}/interpretation")
def update_interpretation(name: str, feature_index: int, request: UpdateInterpretationRequest):
    interpretation = {"text": request.text}
    try:
        C.client.update_feature(sae_name=name, sae_series=C.sae_series, feature_index=feature_index, update_data={"interpretation": interpretation})
    except ValueError:
        return Response(content=f"Feature {feature_index} not found in SAE {name}", status_code=404)
    return {"message": "Interpretation updated successfully", "interpretation": interpretation}


@router.post("/{name}/features/{feature_index}/bookmark")
def add_bookmark(name: str, feature_index: int):
    try:
        if C.client.add_bookmark(sae_name=name, sae_series=C.sae_series, feature_index=feature_index):
            return {"message": "Bookmark added successfully"}
        return Response(content="Feature is already bookmarked", status_code=409)
    except ValueError as e:
        return Response(content=str(e), status_code=404)


@router.delete("/{name}/features/{feature_index}/bookmark")
def remove_bookmark(name: str, feature_index: int):
    if C.client.remove_bookmark(sae_name=name, sae_series=C.sae_series, feature_index=feature_index):
        return {"message": "Bookmark removed successfully"}
    return Response(content="Bookmark not found", status_code=404)


@router.get("/{name}/features/{feature_index}/bookmark")
def check_bookmark(name: str, feature_index: int):
    return {"is_bookmarked": C.client.is_bookmarked(sae_name=name, sae_series=C.sae_series, feature_index=feature_index)}


@router.put("/{name}/features/{feature_index}/bookmark")
def update_bookmark(name: str, feature_index: int, tags: Optional[list[str]] = None, notes: Optional[str] = None):
    if C.client.update_bookmark(sae_name=name, sae_series=C.sae_series, feature_index=feature_index, tags=tags, notes=notes):
        return {"message": "Bookmark updated successfully"}
    return Response(content="Bookmark not found", status_code=404)


@router.post("/{name}/inference")
def inference(name: str, text: str, max_features: int = 10):
    """The features that fire most (summed over the text) with their per-token activations and stored records."""
    model, feature_acts = _encode_text(name, text)
    weight = feature_acts[0].float().sum(dim=0)
    k = min(max_features, int((weight > 0).sum()))
    top_w, top_i = torch.topk(weight, k) if k > 0 else (weight[:0], weight[:0].long())
    origins = model.trace({"text": [text]})[0]
    records = list_feature_data(sae_name=name, indices=top_i.tolist(), with_samplings=True, sampling_size=5)
    out = []
    for i in top_i.tolist():
        rec = records.get((name, i))
        if rec is None:
            continue
        row = feature_acts[0, :, i].float()
        pos = row.nonzero().squeeze(-1)
        out.append({**rec, "inference": {"text": text, "origins": origins, "feature_acts_indices": pos, "feature_acts_values": row[pos]}})
    return packed(out)
