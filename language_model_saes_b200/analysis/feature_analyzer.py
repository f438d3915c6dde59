"""Streaming per-feature statistics and sample selection.

For every feature: how often it fired, its largest activation, and for each configured subsample the ``n_samples``
contexts with the largest peak activation among those whose peak is at most ``proportion`` x (largest activation so
far), with the whole per-token activation row of the context and its metadata. Same outputs as
analysis/feature_analyzer.py:52-359 of the reference project.

Every rank of the ``"model"`` mesh dimension analyses its own feature shard end to end; nothing is exchanged while
streaming (the batch is replicated, the encoder output is already feature-sharded), so state is a set of local tensors:
``elt [n, F_local]``, ``feature_acts [n, F_local, ctx]`` and one ``[n, F_local]`` tensor per metadata key. A batch is
merged by a per-feature ``topk`` over the ``n + batch`` candidates and one gather per tensor, not by a full sort.
"""

from __future__ import annotations

import warnings
from functools import partial
from typing import Any, Mapping, Optional

import torch
from pydantic import ConfigDict, Field
from tqdm import tqdm

from ..config import BaseConfig
from ..models.clt import CrossLayerTranscoder
from ..models.crosscoder import Crosscoder
from ..models.sparse_dictionary import SparseDictionary
from ..parallel.mesh import is_primary_rank, mesh_dim_size
from ..utils.discrete import KeyedDiscreteMapper
from ..utils.tensor_dict import concat_dict_of_tensor, topk_dict_of_tensor
from .post_analysis import PostAnalysisProcessor, get_post_analysis_processor


class FeatureAnalyzerConfig(BaseConfig):
    model_config = ConfigDict(arbitrary_types_allowed=True)
    total_analyzing_tokens: int
    ignore_token_ids: list[int] | None = None
    subsamples: dict[str, dict[str, int | float]] = Field(
        default_factory=lambda: {
            "top_activations": {"proportion": 1.0, "n_samples": 10},
            "non_activating": {"proportion": 0.3, "n_samples": 20, "max_length": 50},
        }
    )
    """name -> {proportion: fraction of the feature's max activation a context may reach, n_samples, max_length}"""
    clt_layer: int | None = None
    """Source layer to analyse; given exactly when the dictionary is a cross-layer transcoder."""


class FeatureAnalyzer:
    def __init__(self, cfg: FeatureAnalyzerConfig):
        self.cfg = cfg

    def _process_batch(self, feature_acts: torch.Tensor, discrete_meta: Mapping[str, torch.Tensor],
                       sample_result: Mapping[str, Mapping[str, torch.Tensor] | None], max_feature_acts: torch.Tensor,
                       device_mesh=None) -> dict[str, Mapping[str, torch.Tensor] | None]:  # fmt: skip
        """Merge one batch (``feature_acts [batch, ctx, F_local]``, ``discrete_meta[k] [batch, F_local]``) into the
        running selections."""
        peak = feature_acts.max(dim=1).values
        elt = peak.clamp(min=0.0)
        acts_t = feature_acts.transpose(1, 2)  # [batch, F, ctx]; gathered rows become contiguous below
        out = dict(sample_result)
        for name, spec in self.cfg.subsamples.items():
            elt_cur = elt.masked_fill(peak > max_feature_acts[None] * spec["proportion"], -torch.inf)
            cur = sample_result[name]
            batch_data = {"elt": elt_cur, "feature_acts": acts_t, **discrete_meta}
            n_keep = int(spec["n_samples"])
            if cur is None:
                merged = batch_data
            else:
                full = cur["elt"].shape[0] >= n_keep
                if full and not bool((elt_cur.max(dim=0).values > cur["elt"][-1]).any()):
                    continue  # no context of this batch displaces a kept one
                merged = concat_dict_of_tensor(dict(cur), batch_data)
            merged = topk_dict_of_tensor(merged, n_keep, sort_key="elt")
            # rows that are -inf for every feature carry nothing
            n_valid = int((merged["elt"] != -torch.inf).any(dim=1).sum())
            out[name] = {k: v[:n_valid].contiguous() for k, v in merged.items()}
        return out

    def compute_ignore_token_masks(self, tokens: torch.Tensor, ignore_token_ids: Optional[list[int]] = None) -> torch.Tensor:
        if ignore_token_ids is None:
            warnings.warn(
                "ignore_token_ids are not provided. No tokens (including pad tokens) will be filtered out. If this is "
                "intentional, set ignore_token_ids explicitly to an empty list to avoid this warning.",
                UserWarning, stacklevel=2,
            )  # fmt: skip
            ignore_token_ids = []
        if not ignore_token_ids:
            return torch.ones_like(tokens, dtype=torch.bool)
        return ~torch.isin(tokens, torch.tensor(ignore_token_ids, device=tokens.device, dtype=tokens.dtype))

    def get_post_analysis_func(self, sae_type: str) -> PostAnalysisProcessor:
        try:
            return get_post_analysis_processor(sae_type)
        except KeyError:
            return get_post_analysis_processor("generic")

    @torch.no_grad()
    def analyze_chunk(self, activation_factory, sae: SparseDictionary, device_mesh=None,
                      activation_factory_process_kwargs: dict[str, Any] | None = None) -> list[dict[str, Any]]:  # fmt: skip
        """Analyse this rank's feature shard; returns one dict per local feature."""
        kwargs = activation_factory_process_kwargs or {}
        stream = activation_factory.process(**kwargs)
        tp = mesh_dim_size(device_mesh, "model")
        f_local = sae.cfg.d_sae // tp
        dev = next(sae.parameters()).device
        act_times = torch.zeros(f_local, dtype=torch.long, device=dev)
        max_feature_acts = torch.zeros(f_local, dtype=sae.cfg.dtype, device=dev)
        sample_result: dict[str, Any] = {k: None for k in self.cfg.subsamples}
        mapper = KeyedDiscreteMapper()
        n_tokens = n_analyzed = 0
        bar = tqdm(total=self.cfg.total_analyzing_tokens, desc="Analyzing SAE", smoothing=0.01, disable=not is_primary_rank(device_mesh))

        encode, prepare_input = sae.encode, sae.prepare_input
        if isinstance(sae, CrossLayerTranscoder):
            assert self.cfg.clt_layer is not None, "clt_layer is required to analyse a cross-layer transcoder"
            encode = partial(sae.encode_single_layer, layer=self.cfg.clt_layer)
            prepare_input = partial(sae.prepare_input_single_layer, layer=self.cfg.clt_layer)
            sae.keep_only_decoders_for_layer_from(self.cfg.clt_layer)

        for batch in stream:
            meta = {k: [m[k] for m in batch["meta"]] for k in batch["meta"][0].keys()}
            x, enc_kwargs, _ = prepare_input(batch)
            tokens = batch["tokens"].to(dev)
            feature_acts = encode(x.to(dev), **enc_kwargs)
            if isinstance(sae, Crosscoder):
                feature_acts = feature_acts.amax(dim=-2)
            assert feature_acts.shape == (tokens.shape[0], tokens.shape[1], f_local), (
                f"feature_acts.shape: {tuple(feature_acts.shape)}, expected: {(tokens.shape[0], tokens.shape[1], f_local)}"
            )
            if self.cfg.ignore_token_ids is None and batch.get("mask") is not None:
                keep = batch["mask"].to(dev).bool()
            else:
                keep = self.compute_ignore_token_masks(tokens, self.cfg.ignore_token_ids)
            feature_acts = feature_acts * keep[..., None]

            act_times += feature_acts.gt(0.0).sum(dim=(0, 1))
            max_feature_acts = torch.maximum(max_feature_acts, feature_acts.amax(dim=(0, 1)))

            discrete_meta = {}
            for k, v in meta.items():
                if all(isinstance(i, str) for i in v):
                    row = torch.tensor(mapper.encode(k, v), device=dev, dtype=torch.int32)
                else:
                    row = torch.as_tensor(v, device=dev)
                discrete_meta[k] = row[:, None].expand(-1, f_local)
            sample_result = self._process_batch(feature_acts, discrete_meta, sample_result, max_feature_acts, device_mesh)

            n_tokens += tokens.numel()
            n_analyzed += int(keep.sum())
            bar.update(tokens.numel())
            if n_tokens >= self.cfg.total_analyzing_tokens:
                break
        bar.close()

        sample_result = {k: v for k, v in sample_result.items() if v is not None}
        return self.get_post_analysis_func(sae.cfg.sae_type).process(
            sae=sae, act_times=act_times, n_analyzed_tokens=n_analyzed, max_feature_acts=max_feature_acts,
            sample_result=sample_result, mapper=mapper, device_mesh=device_mesh, activation_factory=activation_factory,
            activation_factory_process_kwargs=kwargs, clt_layer=self.cfg.clt_layer,
        )  # fmt: skip
