"""Turn the analyser's tensors into one record per feature; dictionary types add their own fields through a
registry (analysis/post_analysis/base.py:24-187 of the reference project)."""

from __future__ import annotations

from abc import ABC
from typing import Any

import numpy as np
import torch

from ...models.sparse_dictionary import SparseDictionary
from ...utils.discrete import KeyedDiscreteMapper
from ...utils.logging import get_logger

logger = get_logger("analysis.post_analysis")


class PostAnalysisProcessor(ABC):
    @torch.no_grad()  # records are measurements: nothing here is differentiated, whatever mode the caller is in
    def process(self, sae: SparseDictionary, act_times: torch.Tensor, n_analyzed_tokens: int, max_feature_acts: torch.Tensor,
                sample_result: dict[str, dict[str, torch.Tensor]], mapper: KeyedDiscreteMapper, device_mesh=None,
                activation_factory=None, activation_factory_process_kwargs: dict[str, Any] | None = None,
                clt_layer: int | None = None) -> list[dict[str, Any]]:  # fmt: skip
        sample_result, extra = self._process_tensors(
            sae, act_times, n_analyzed_tokens, max_feature_acts, sample_result, mapper, device_mesh, activation_factory,
            activation_factory_process_kwargs=activation_factory_process_kwargs or {}, clt_layer=clt_layer,
        )  # fmt: skip
        sample_result = {k: v for k, v in sample_result.items() if v is not None}
        # one device->host copy per tensor, then pure numpy per feature (no per-feature synchronisation)
        host = {
            name: {k: (v.float().cpu().numpy() if isinstance(v, torch.Tensor) and v.is_floating_point() else
                       v.cpu().numpy() if isinstance(v, torch.Tensor) else v) for k, v in sub.items()}
            for name, sub in sample_result.items()
        }  # fmt: skip
        times = act_times.cpu().tolist()
        peaks = max_feature_acts.float().cpu().tolist()
        results = []
        for i in range(len(times)):
            results.append({
                "act_times": times[i],
                "n_analyzed_tokens": n_analyzed_tokens,
                "max_feature_acts": peaks[i],
                **(extra[i] if extra is not None else {}),
                "samplings": [
                    {
                        "name": name,
                        **self._sparsify_feature_acts(sub["feature_acts"][:, i]),
                        **self._extra_info(sub, i),
                        **{k: mapper.decode(k, sub[k][:, i].tolist()) for k in mapper.keys()},
                    }
                    for name, sub in host.items()
                ],
            })  # fmt: skip
        return results

    def _sparsify_feature_acts(self, feature_acts: np.ndarray) -> dict[str, Any]:
        """COO form of a ``[n_samples, ctx]`` block: ``indices [2, nnz]`` (float32, as stored by the reference), ``values``."""
        rows, cols = np.nonzero(feature_acts)
        return {
            "feature_acts_indices": np.stack([rows, cols]).astype(np.float32),
            "feature_acts_values": feature_acts[rows, cols].astype(np.float32),
        }

    def _extra_info(self, sampling_data: dict[str, Any], i: int) -> dict[str, Any]:
        ctx = np.asarray(sampling_data["context_idx"][:, i])
        return {
            "context_idx": ctx,
            "shard_idx": np.asarray(sampling_data["shard_idx"][:, i]) if "shard_idx" in sampling_data else np.zeros_like(ctx, dtype=np.int64),
            "n_shards": np.asarray(sampling_data["n_shards"][:, i]) if "n_shards" in sampling_data else np.ones_like(ctx, dtype=np.int64),
        }

    def _process_tensors(self, sae, act_times, n_analyzed_tokens, max_feature_acts, sample_result, mapper, device_mesh=None,
                         activation_factory=None, activation_factory_process_kwargs: dict[str, Any] | None = None,
                         clt_layer: int | None = None) -> tuple[dict[str, dict[str, Any]], list[dict[str, Any]] | None]:  # fmt: skip
        """Hook for dictionary-specific additions: may add keys to ``sample_result`` and return per-feature dicts."""
        return sample_result, None


_registry: dict[str, type[PostAnalysisProcessor]] = {}


def register_post_analysis_processor(sae_type: str, processor_class: type[PostAnalysisProcessor]) -> None:
    _registry[sae_type] = processor_class


def get_post_analysis_processor(sae_type: str) -> PostAnalysisProcessor:
    if sae_type not in _registry:
        raise KeyError(f"No post-analysis processor registered for SAE type: {sae_type}")
    return _registry[sae_type]()
