"""Turn stored samplings into displayable samples: text, token origins, sparse activations
(server/logic/samples.py of the reference project)."""

from __future__ import annotations

from functools import lru_cache
from typing import Any

import numpy as np

from . import config as C
from .loaders import get_dataset, get_model


def _rows_of(indices: np.ndarray, values: np.ndarray, i: int) -> tuple[np.ndarray, np.ndarray]:
    """Entries of sample ``i`` of a COO block whose first index row is the sample."""
    sel = indices[0] == i
    return indices[1:, sel], values[sel]


def extract_samples(sampling, start: int | None = None, end: int | None = None, visible_range: int | None = None) -> list[dict[str, Any]]:
    """Samples ``start..end`` of a sampling. With ``visible_range`` only the tokens within that distance of the strongest
    token are kept (``token_offset`` / ``text_offset`` tell where the window starts)."""
    n = len(sampling.context_idx)
    start, end = start or 0, n if end is None else min(end, n)
    fa_idx, fa_val = np.asarray(sampling.feature_acts_indices).astype(np.int64), np.asarray(sampling.feature_acts_values)
    zp = sampling.z_pattern_indices is not None and sampling.z_pattern_values is not None
    zp_idx = np.asarray(sampling.z_pattern_indices).astype(np.int64) if zp else None
    zp_val = np.asarray(sampling.z_pattern_values) if zp else None
    shard = sampling.shard_idx if sampling.shard_idx is not None else [0] * n
    n_shards = sampling.n_shards if sampling.n_shards is not None else [1] * n
    out = []
    for i in range(start, end):
        model = get_model(name=sampling.model_name[i])
        data = dict(get_dataset(name=sampling.dataset_name[i], shard_idx=int(shard[i]), n_shards=int(n_shards[i]))[int(sampling.context_idx[i])])
        origins = model.trace({k: [v] for k, v in data.items()})[0]
        (pos,), val = _rows_of(fa_idx, fa_val, i)
        z_i, z_v = _rows_of(zp_idx, zp_val, i) if zp else (None, None)
        token_offset, text_offset = 0, None
        if visible_range is not None:
            peak = int(pos[np.argmax(val)]) if len(pos) else 0
            keep = (pos > peak - visible_range) & (pos < peak + visible_range)
            pos, val = pos[keep], val[keep]
            if zp:
                zk = ((z_i > peak - visible_range) & (z_i < peak + visible_range)).all(axis=0)
                z_i, z_v = z_i[:, zk], z_v[zk]
            token_offset = max(0, peak - visible_range)
            origins = origins[token_offset : peak + visible_range]
        if "text" in data:
            ranges = [o["range"] for o in origins if o is not None and o["key"] == "text"]
            if ranges:
                data["text"] = data["text"][: max(r[1] for r in ranges)]
                if visible_range is not None:
                    text_offset = min(r[0] for r in ranges)
                    data["text"] = data["text"][text_offset:]
        out.append({**data, "token_offset": token_offset, "text_offset": text_offset, "origins": origins,
                    "feature_acts_indices": pos, "feature_acts_values": val, "z_pattern_indices": z_i, "z_pattern_values": z_v})  # fmt: skip
    return out


@lru_cache(maxsize=C.LRU_CACHE_SIZE_SAMPLES)
def cached_extract_samples(sae_name: str, sae_series: str, feature_index: int, sampling_name: str, start: int | None = None,
                           end: int | None = None, visible_range: int | None = None) -> list[dict[str, Any]]:  # fmt: skip
    feature = C.client.get_feature(sae_name=sae_name, sae_series=sae_series, index=feature_index)
    if feature is None:
        return []
    for analysis in feature.analyses:
        sampling = next((s for s in analysis.samplings if s.name == sampling_name), None)
        if sampling is not None:
            return extract_samples(sampling, start, end, visible_range)
    return []


def pick_analysis(feature, name: str | None = None):
    """The named analysis; without a name ``"default"`` if present, else the first."""
    if name is not None:
        return next((a for a in feature.analyses if a.name == name), None)
    return next((a for a in feature.analyses if a.name == "default"), None) or next(iter(feature.analyses), None)


def list_feature_data(sae_name: str, indices: list[int], with_samplings: bool = True, sampling_size: int = 1,
                      sampling_visible_range: int = 10, with_logits: bool = True) -> dict[tuple[str, int], dict[str, Any]]:  # fmt: skip
    out: dict[tuple[str, int], dict[str, Any]] = {}
    for feature in C.client.list_features(sae_name=sae_name, sae_series=C.sae_series, indices=indices):
        analysis = pick_analysis(feature)
        if analysis is None:
            continue
        data = {"feature_index": feature.index, "analysis_name": analysis.name, "interpretation": feature.interpretation,
                "dictionary_name": feature.sae_name, "act_times": analysis.act_times, "max_feature_act": analysis.max_feature_acts,
                "n_analyzed_tokens": analysis.n_analyzed_tokens}  # fmt: skip
        if with_logits:
            data["logits"] = feature.logits
        if with_samplings:
            sampling = next((s for s in analysis.samplings if s.name == "top_activations"), None)
            data["samples"] = (cached_extract_samples(sae_name, C.sae_series, feature.index, sampling.name, 0, sampling_size,
                                                      visible_range=sampling_visible_range) if sampling is not None else [])  # fmt: skip
        out[(sae_name, feature.index)] = data
    return out
