"""Evaluate a dictionary on a stream: the training metrics without gradients, plus the downstream language-model
loss when a hooked model is given (evaluator.py:31-87 of the reference project)."""

from __future__ import annotations

from typing import Iterable

import torch
from tqdm import tqdm

from .config import BaseConfig
from .metrics import (
    DownstreamMetric,
    ExplainedVarianceMetric,
    FrequencyMetric,
    L0Metric,
    L2NormErrorMetric,
    LossMetric,
    MeanFeatureActMetric,
    Metric,
    ModelSpecificMetric,
)
from .models.sparse_dictionary import SparseDictionary
from .utils.logging import get_distributed_logger, log_metrics

logger = get_distributed_logger("evaluator")


class EvalConfig(BaseConfig):
    total_eval_tokens: int = 1000000


class Evaluator:
    def __init__(self, cfg: EvalConfig):
        self.cfg = cfg

    @torch.no_grad()
    def evaluate(self, sae: SparseDictionary, data_stream: Iterable[dict[str, torch.Tensor]], wandb_logger=None, model=None) -> dict[str, float]:
        from .models.lorsa import LowRankSparseAttention
        from .models.sae import SparseAutoEncoder

        metrics: list[Metric] = [FrequencyMetric(sae), LossMetric(sae), MeanFeatureActMetric(sae), ExplainedVarianceMetric(sae),
                                 L0Metric(sae), L2NormErrorMetric(sae), ModelSpecificMetric(sae)]  # fmt: skip
        if model is not None and isinstance(sae, (SparseAutoEncoder, LowRankSparseAttention)):
            logger.info("Downstream metrics available.")
            metrics.append(DownstreamMetric(sae, model))
        total = 0
        bar = tqdm(total=self.cfg.total_eval_tokens)
        dev = next(sae.parameters()).device
        for batch in data_stream:
            batch = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
            raw = batch
            batch = sae.normalize_activations(batch)
            ctx = sae.compute_loss(batch, return_aux_data=True)
            ctx["tokens"] = raw.get("tokens")
            for m in metrics:
                if isinstance(m, DownstreamMetric) and (raw.get("tokens") is None or raw["tokens"].ndim != 2):
                    continue
                ctx = {**ctx, **m.update(ctx)}
            n = batch["tokens"].numel() if batch.get("mask") is None else int(batch["mask"].sum())
            total += n
            bar.update(n)
            if total >= self.cfg.total_eval_tokens:
                break
        bar.close()
        results: dict[str, float] = {}
        for m in metrics:
            try:
                results.update(m.compute())
            except AssertionError:
                pass  # a metric that never saw a batch (e.g. downstream loss on 1-D activations)
        log_metrics(logger.logger, results, title="Evaluation Metrics")
        if wandb_logger is not None:
            wandb_logger.log(results)
        return results
