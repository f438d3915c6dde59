"""Training / evaluation metrics.

Same metric classes and logged keys as metrics.py of the reference project (Record :23, GradientNormMetric
:78, FrequencyMetric :102, LossMetric :149, MeanFeatureActMetric :185, ExplainedVarianceMetric :203,
L0Metric :254, L2NormErrorMetric :286, ModelSpecificMetric :313, DownstreamMetric :331). Differences:
``update`` only accumulates device tensors (no host synchronisation per step); cross-rank reductions (sum
over feature shards, mean over data ranks) and the device-to-host reads happen in ``compute``, i.e. once per
logging interval.
"""

from __future__ import annotations

from abc import ABC
from typing import Any

import torch
import torch.distributed as dist
from torch import Tensor

from .optim import compute_grad_norm
from .parallel.mesh import mesh_dim_size, mesh_group
from .utils.logging import get_distributed_logger
from .utils.tensor_specs import apply_token_mask, reduce

logger = get_distributed_logger("metrics")


def _num(v) -> float:
    return float(v.item()) if isinstance(v, Tensor) else float(v)


class Record:
    """Running sum / max / min with a count; ``compute`` returns the reduced value and resets."""

    def __init__(self, reduction: str = "mean"):
        assert reduction in ("mean", "sum", "max", "min"), f"Invalid reduction: {reduction}"
        self.value: Any = None
        self.count: Any = 0
        self.reduction = reduction

    def update(self, value, count: Tensor | int = 1):
        if isinstance(value, Tensor):
            value = value.detach()
            if value.dtype in (torch.bfloat16, torch.float16):
                value = value.float()
        self.count = self.count + count
        if self.value is None:
            self.value = value
        elif self.reduction in ("mean", "sum"):
            self.value = self.value + value
        elif self.reduction == "max":
            self.value = torch.maximum(self.value, value) if isinstance(value, Tensor) else max(self.value, value)
        else:
            self.value = torch.minimum(self.value, value) if isinstance(value, Tensor) else min(self.value, value)

    def compute(self):
        assert self.value is not None, "Record must be updated before computing"
        out = self.value / self.count if self.reduction == "mean" else self.value
        self.value, self.count = None, 0
        return out


class Metric(ABC):
    def update(self, ctx: dict[str, Any]) -> dict[str, Any]:
        return {}

    def compute(self) -> dict[str, float]:
        raise NotImplementedError


class _ShardAware(Metric):
    """Helpers for metrics of models whose feature axis may be sharded and whose batch may be split."""

    def __init__(self, sae):
        self.sae = sae

    def _sum_model(self, t: Tensor) -> Tensor:
        if mesh_dim_size(self.sae.device_mesh, "model") > 1:
            t = t.clone()
            dist.all_reduce(t, group=mesh_group(self.sae.device_mesh, "model"))
        return t

    def _mean_data(self, t: Tensor) -> Tensor:
        n = mesh_dim_size(self.sae.device_mesh, "data")
        if n > 1:
            t = t.clone().float()
            dist.all_reduce(t, group=mesh_group(self.sae.device_mesh, "data"))
            t = t / n
        return t


class GradientNormMetric(_ShardAware):
    def __init__(self, sae):
        super().__init__(sae)
        self.gradient_norm = Record("max")
        self.gradient_norm_before_clipping = Record("max")

    def update(self, ctx):
        before = ctx.get("grad_norm_before_clipping")
        assert before is not None, "Gradient norm before clipping must be provided"
        before = torch.as_tensor(before)
        self.gradient_norm_before_clipping.update(before)
        now = compute_grad_norm(self.sae.parameters(), self.sae.device_mesh)
        self.gradient_norm.update(now)
        return {"gradient_norm_per_param": now, "gradient_norm_before_clipping": before}

    def compute(self):
        return {
            "metrics/gradient_norm_per_param": _num(self.gradient_norm.compute()),
            "metrics/gradient_norm_before_clipping": _num(self.gradient_norm_before_clipping.compute()),
        }


class FrequencyMetric(_ShardAware):
    def __init__(self, sae):
        super().__init__(sae)
        self.act_freq_scores = Record()
        self.specs: tuple[str, ...] | None = None

    def update(self, ctx):
        acts, mask = ctx["feature_acts"], ctx.get("mask")
        counts, specs = apply_token_mask((acts > 0).float(), self.sae.specs.feature_acts(acts), mask, "sum")
        self.act_freq_scores.update(counts, ctx["n_tokens"])
        self.specs = specs
        return {"act_freq_scores": counts}

    def compute(self):
        assert self.specs is not None, "Metrics must be updated before computing"
        freq = self._mean_data(self.act_freq_scores.compute())
        bounds = [("above_1e-1", freq > 1e-1), ("above_1e-2", freq > 1e-2), ("below_1e-5", freq < 1e-5),
                  ("below_1e-6", freq < 1e-6), ("below_1e-7", freq < 1e-7)]  # fmt: skip
        out: dict[str, float] = {}
        layer_dim = self.specs.index("layers") if "layers" in self.specs else None
        for name, m in bounds:
            out[f"sparsity/{name}"] = _num(self._sum_model(m.sum()))
            if layer_dim is not None:
                for l in range(freq.size(layer_dim)):
                    out[f"sparsity/{name}_layer{l}"] = _num(self._sum_model(m.select(layer_dim, l).sum()))
        return out


class LossMetric(_ShardAware):
    _KEYS = (("loss", "overall_loss"), ("l_rec", "mse_loss"), ("l_s", "sparsity_loss"), ("l_p", "lp_loss"), ("l_aux", "aux_loss"))

    def __init__(self, sae):
        super().__init__(sae)
        self.records = {k: Record() for k, _ in self._KEYS}

    def update(self, ctx):
        for k, _ in self._KEYS:
            v = ctx.get(k)
            if v is not None:
                self.records[k].update(v.detach().float().mean())
        return {}

    def compute(self):
        out = {}
        for k, name in self._KEYS:
            if self.records[k].value is not None:
                out[f"losses/{name}"] = _num(self._mean_data(self.records[k].compute()))
        return out


class MeanFeatureActMetric(_ShardAware):
    def __init__(self, sae):
        super().__init__(sae)
        self.total = Record("sum")
        self.active = Record("sum")

    def update(self, ctx):
        acts = ctx["feature_acts"]
        self.total.update(acts.float().sum())
        self.active.update(acts.gt(0).float().sum())
        return {}

    def compute(self):
        s = self._sum_model(torch.stack([self.total.compute(), self.active.compute()]))
        n = mesh_dim_size(self.sae.device_mesh, "data")
        if n > 1:
            dist.all_reduce(s, group=mesh_group(self.sae.device_mesh, "data"))
        return {"metrics/mean_feature_act": _num(s[0] / s[1])}


class ExplainedVarianceMetric(_ShardAware):
    def __init__(self, sae):
        super().__init__(sae)
        self.explained_variance = Record()
        self.explained_variance_legacy = Record()

    def update(self, ctx):
        label, rec, mask = ctx["label"].float(), ctx["reconstructed"].float(), ctx.get("mask")
        specs = self.sae.specs.label(label)
        label_mean = apply_token_mask(label, specs, mask, "mean")[0]
        # the mean goes back under the token axes it was taken over, wherever the model keeps them ([layers, batch, d] for a
        # cross-layer transcoder, where a plain trailing-axes broadcast would pair layers with tokens)
        label_mean = label_mean.reshape([1 if s in ("batch", "context") else label.shape[i] for i, s in enumerate(specs)])
        err = (rec - label).pow(2).sum(dim=-1)
        var = (label - label_mean).pow(2).sum(dim=-1)
        legacy = apply_token_mask(1 - err / var, specs[:-1], mask, "mean")[0]
        ev = 1 - apply_token_mask(err, specs[:-1], mask, "mean")[0] / apply_token_mask(var, specs[:-1], mask, "mean")[0]
        self.explained_variance.update(ev)
        self.explained_variance_legacy.update(legacy)
        return {"explained_variance": ev, "explained_variance_legacy": legacy}

    def compute(self):
        return {
            "metrics/explained_variance": _num(self._mean_data(self.explained_variance.compute().mean())),
            "metrics/explained_variance_legacy": _num(self._mean_data(self.explained_variance_legacy.compute().mean())),
        }


class L0Metric(_ShardAware):
    def __init__(self, sae):
        super().__init__(sae)
        self.l0 = Record()
        self.specs: tuple[str, ...] | None = None

    def update(self, ctx):
        acts, mask = ctx["feature_acts"], ctx.get("mask")
        l0, specs = apply_token_mask((acts > 0).float(), self.sae.specs.feature_acts(acts), mask, "sum")
        l0, specs = reduce(l0, specs, {"sae": "sum"})
        self.l0.update(l0, ctx["n_tokens"])
        self.specs = specs
        return {"l0": l0}

    def compute(self):
        assert self.specs is not None, "Metrics must be updated before computing"
        l0 = reduce(self.l0.compute(), self.specs, {"layers": "sum"})[0]
        return {"metrics/l0": _num(self._mean_data(self._sum_model(l0.mean())))}


class L2NormErrorMetric(_ShardAware):
    def __init__(self, sae):
        super().__init__(sae)
        self.l2_norm_error = Record()
        self.l2_norm_error_ratio = Record()

    def update(self, ctx):
        label, rec, mask = ctx["label"].float(), ctx["reconstructed"].float(), ctx.get("mask")
        specs = self.sae.specs.label(label)[:-1]
        err = apply_token_mask((rec - label).pow(2).sum(dim=-1).sqrt(), specs, mask, "mean")[0]
        ratio = err / apply_token_mask(label.norm(p=2, dim=-1), specs, mask, "mean")[0]
        self.l2_norm_error.update(err)
        self.l2_norm_error_ratio.update(ratio)
        return {}

    def compute(self):
        return {
            "metrics/l2_norm_error": _num(self._mean_data(self.l2_norm_error.compute().mean())),
            "metrics/l2_norm_error_ratio": _num(self._mean_data(self.l2_norm_error_ratio.compute().mean())),
        }


class ModelSpecificMetric(Metric):
    def __init__(self, sae):
        self.sae = sae
        self.metrics: dict[str, Record] = {}

    def update(self, ctx):
        for k, v in self.sae.compute_training_metrics(**ctx).items():
            self.metrics.setdefault(k, Record()).update(v)
        return {}

    def compute(self):
        return {k: _num(v.compute()) for k, v in self.metrics.items()}


class DownstreamMetric(Metric):
    """Language-model loss with the hooked activation left alone / replaced by the reconstruction / zeroed.

    ``model`` is a hooked transformer exposing ``run_with_cache`` and ``run_with_hooks`` with
    ``return_type="loss", loss_per_token=True`` (the interface of ``backend.hooked_transformer``)."""

    def __init__(self, sae, model):
        self.sae = sae
        self.model = model
        self.original = Record()
        self.reconstructed = Record()
        self.ablated = Record()
        self.ratio = Record()

    @torch.no_grad()
    def update(self, ctx):
        tokens, mask = ctx["tokens"], ctx["mask"]
        assert tokens.ndim == 2, "Tokens must be a 2D tensor"
        hin, hout = self.sae.cfg.hook_point_in, self.sae.cfg.hook_point_out
        loss, cache = self.model.run_with_cache(tokens, return_type="loss", loss_per_token=True, names_filter=[hin, hout])
        batch = {"tokens": tokens, "mask": mask, **cache}
        batch, scale = self.sae.normalize_activations(batch, return_scale_factor=True)
        x, ekw, dkw = self.sae.prepare_input(batch)
        rec = self.sae.forward(x, encoder_kwargs=ekw, decoder_kwargs=dkw)
        rec = self.sae.denormalize_activations({hout: rec}, scale_factors=scale)[hout]
        m = mask.bool().unsqueeze(-1)

        def put_rec(act, hook):
            return torch.where(m, rec.to(act.dtype), act)

        def put_zero(act, hook):
            return torch.where(m, torch.zeros_like(act), act)

        rec_loss = self.model.run_with_hooks(tokens, return_type="loss", loss_per_token=True, fwd_hooks=[(hout, put_rec)])
        abl_loss = self.model.run_with_hooks(tokens, return_type="loss", loss_per_token=True, fwd_hooks=[(hout, put_zero)])
        lm = mask[:, 1:] if loss.shape[1] == mask.shape[1] - 1 else mask
        specs = ("batch", "context")
        loss = apply_token_mask(loss, specs, lm, "mean")[0]
        rec_loss = apply_token_mask(rec_loss, specs, lm, "mean")[0]
        abl_loss = apply_token_mask(abl_loss, specs, lm, "mean")[0]
        self.original.update(loss)
        self.reconstructed.update(rec_loss)
        self.ablated.update(abl_loss)
        self.ratio.update((abl_loss - loss) / (abl_loss - rec_loss))
        return {}

    def compute(self):
        return {
            "metrics/downstream_loss_original": _num(self.original.compute()),
            "metrics/downstream_loss_reconstructed": _num(self.reconstructed.compute()),
            "metrics/downstream_loss_ablated": _num(self.ablated.compute()),
            "metrics/downstream_loss_ratio": _num(self.ratio.compute()),
        }
