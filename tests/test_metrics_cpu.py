"""The logged metrics against their plain definitions, for 2-D and 3-D inputs, with and without a token mask, and for a
crosscoder's head axis. The definitions are those of metrics.py of the reference project (FrequencyMetric :100, L0Metric
:254, L2NormErrorMetric :286, ExplainedVarianceMetric :203, MeanFeatureActMetric :185)."""

import pytest
import torch

from language_model_saes_b200.metrics import (
    ExplainedVarianceMetric,
    FrequencyMetric,
    L0Metric,
    L2NormErrorMetric,
    LossMetric,
    MeanFeatureActMetric,
    Record,
)
from language_model_saes_b200.models.crosscoder import CrosscoderSpecs
from language_model_saes_b200.utils.tensor_specs import TensorSpecs, apply_token_mask, reduce


class _Dictionary:
    """What the metrics read of a model: the dimension names and the (absent) mesh."""

    device_mesh = None

    def __init__(self, specs=TensorSpecs):
        self.specs = specs


def _acts(*shape, density=0.2, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.rand(*shape, generator=g) * (torch.rand(*shape, generator=g) < density)


def test_record_reductions():
    r = Record()
    r.update(torch.tensor([2.0, 4.0]), 2)
    r.update(torch.tensor([4.0, 0.0]), 1)
    assert torch.allclose(r.compute(), torch.tensor([2.0, 4.0 / 3]))
    assert r.value is None and r.count == 0  # compute resets
    for how, want in (("sum", 5.0), ("max", 3.0), ("min", 2.0)):
        r = Record(how)
        r.update(torch.tensor(2.0))
        r.update(torch.tensor(3.0))
        assert float(r.compute()) == want
    r = Record()
    r.update(torch.tensor(1.0, dtype=torch.bfloat16))
    assert r.value.dtype == torch.float32  # half precision is accumulated in fp32
    with pytest.raises(AssertionError):
        Record().compute()


def test_token_mask_and_named_reductions():
    t = torch.arange(24.0).reshape(2, 3, 4)
    specs = ("batch", "context", "sae")
    s, left = apply_token_mask(t, specs, None, "sum")
    assert left == ("sae",) and torch.equal(s, t.sum((0, 1)))
    mask = torch.tensor([[1, 0, 1], [0, 0, 1]])
    s, _ = apply_token_mask(t, specs, mask, "sum")
    assert torch.equal(s, t[mask.bool()].sum(0))
    m, _ = apply_token_mask(t, specs, mask, "mean")
    assert torch.allclose(m, t[mask.bool()].mean(0))
    # the token axes need not be the leading ones
    u = t.permute(2, 0, 1)
    s2, left = apply_token_mask(u, ("layers", "batch", "context"), mask, "sum")
    assert left == ("layers",) and torch.equal(s2, s)
    r, left = reduce(t, specs, {"sae": "max", "heads": "sum"})  # absent names are ignored
    assert left == ("batch", "context") and torch.equal(r, t.amax(-1))
    with pytest.raises(AssertionError):
        apply_token_mask(t, specs, torch.ones(2, 4), "sum")


@pytest.mark.parametrize("with_context,masked", [(False, False), (True, False), (True, True)])
def test_frequency_l0_and_mean_act_of_a_single_layer_dictionary(with_context, masked):
    F = 64
    sae = _Dictionary()
    freq, l0, mean_act = FrequencyMetric(sae), L0Metric(sae), MeanFeatureActMetric(sae)
    fired = torch.zeros(F)
    n_total, l0_sum, act_sum, act_cnt = 0, 0.0, 0.0, 0.0
    per_step_l0 = []
    for step in range(3):
        acts = _acts(*((5, 7, F) if with_context else (35, F)), seed=step)
        mask = (torch.rand(5, 7, generator=torch.Generator().manual_seed(10 + step)) < 0.7) if masked else None
        rows = acts[mask] if masked else acts.reshape(-1, F)
        n = rows.shape[0]
        ctx = {"feature_acts": acts, "mask": mask, "n_tokens": n}
        for m in (freq, l0, mean_act):
            m.update(ctx)
        fired += (rows > 0).float().sum(0)
        n_total += n
        per_step_l0.append((rows > 0).float().sum())
        # the mean activation counts every entry it is given (a mask is applied by the caller to the activations themselves)
        act_sum += float(acts.sum())
        act_cnt += float((acts > 0).sum())
    rate = fired / n_total
    got = freq.compute()
    assert got["sparsity/above_1e-1"] == float((rate > 0.1).sum())
    assert got["sparsity/above_1e-2"] == float((rate > 0.01).sum())
    assert got["sparsity/below_1e-5"] == float((rate < 1e-5).sum())
    assert not any("layer" in k for k in got)
    assert l0.compute()["metrics/l0"] == pytest.approx(float(sum(per_step_l0)) / n_total, rel=1e-6)
    assert mean_act.compute()["metrics/mean_feature_act"] == pytest.approx(act_sum / act_cnt, rel=1e-5)


def test_frequency_and_l0_with_layers_report_per_layer_counts():
    class LayerSpecs(TensorSpecs):
        @staticmethod
        def feature_acts(t):
            return ("batch", "layers", "sae")

    sae = _Dictionary(LayerSpecs)
    acts = _acts(40, 3, 16, density=0.3)
    acts[:, 1, :4] = 0  # four features of layer 1 never fire
    freq, l0 = FrequencyMetric(sae), L0Metric(sae)
    ctx = {"feature_acts": acts, "mask": None, "n_tokens": 40}
    freq.update(ctx), l0.update(ctx)
    got = freq.compute()
    rate = (acts > 0).float().mean(0)  # [layers, F]
    for l in range(3):
        assert got[f"sparsity/below_1e-7_layer{l}"] == float((rate[l] < 1e-7).sum())
        assert got[f"sparsity/above_1e-1_layer{l}"] == float((rate[l] > 0.1).sum())
    assert got["sparsity/below_1e-7_layer1"] >= 4
    assert got["sparsity/below_1e-7"] == sum(got[f"sparsity/below_1e-7_layer{l}"] for l in range(3))
    # l0 of a layered dictionary is the number of active features per token over all layers
    assert l0.compute()["metrics/l0"] == pytest.approx(float((acts > 0).float().sum((1, 2)).mean()), rel=1e-6)


@pytest.mark.parametrize("masked", [False, True])
def test_explained_variance_and_l2_error(masked):
    g = torch.Generator().manual_seed(0)
    sae = _Dictionary()
    label = torch.randn(4, 6, 8, generator=g) + 2.0
    rec = label + 0.3 * torch.randn(4, 6, 8, generator=g)
    mask = (torch.rand(4, 6, generator=g) < 0.6) if masked else None
    ev, l2 = ExplainedVarianceMetric(sae), L2NormErrorMetric(sae)
    ctx = {"label": label, "reconstructed": rec, "mask": mask}
    out = ev.update(ctx)
    l2.update(ctx)
    rows_l = label[mask] if masked else label.reshape(-1, 8)
    rows_r = rec[mask] if masked else rec.reshape(-1, 8)
    err = (rows_r - rows_l).pow(2).sum(-1)
    var = (rows_l - rows_l.mean(0)).pow(2).sum(-1)
    want_ev = 1 - err.mean() / var.mean()
    want_legacy = (1 - err / var).mean()
    assert float(out["explained_variance"]) == pytest.approx(float(want_ev), rel=1e-5)
    got = ev.compute()
    assert got["metrics/explained_variance"] == pytest.approx(float(want_ev), rel=1e-5)
    assert got["metrics/explained_variance_legacy"] == pytest.approx(float(want_legacy), rel=1e-4)
    got = l2.compute()
    assert got["metrics/l2_norm_error"] == pytest.approx(float(err.sqrt().mean()), rel=1e-5)
    assert got["metrics/l2_norm_error_ratio"] == pytest.approx(float(err.sqrt().mean() / rows_l.norm(dim=-1).mean()), rel=1e-5)
    # a perfect reconstruction explains everything, the mean explains nothing
    ev.update({"label": label, "reconstructed": label, "mask": mask})
    assert ev.compute()["metrics/explained_variance"] == pytest.approx(1.0)
    mean = (rows_l.mean(0)).expand_as(label)
    ev.update({"label": label, "reconstructed": mean, "mask": mask})
    assert ev.compute()["metrics/explained_variance"] == pytest.approx(0.0, abs=1e-5)


def test_crosscoder_heads_keep_their_own_explained_variance_and_counts():
    g = torch.Generator().manual_seed(1)
    sae = _Dictionary(CrosscoderSpecs)
    label = torch.randn(32, 3, 8, generator=g) * torch.tensor([1.0, 2.0, 0.5]).view(1, 3, 1)
    noise = torch.randn(32, 3, 8, generator=g) * torch.tensor([0.1, 1.0, 0.0]).view(1, 3, 1)
    rec = label + noise
    ev = ExplainedVarianceMetric(sae)
    out = ev.update({"label": label, "reconstructed": rec, "mask": None})
    per_head = out["explained_variance"]
    assert per_head.shape == (3,)
    for h in range(3):
        e = (rec[:, h] - label[:, h]).pow(2).sum(-1).mean()
        v = (label[:, h] - label[:, h].mean(0)).pow(2).sum(-1).mean()
        assert float(per_head[h]) == pytest.approx(float(1 - e / v), rel=1e-5)
    assert float(per_head[2]) == pytest.approx(1.0)
    assert ev.compute()["metrics/explained_variance"] == pytest.approx(float(per_head.mean()), rel=1e-6)
    # frequency and l0 keep the head axis until the end: a feature counts once per head it fires in
    acts = _acts(32, 3, 16, density=0.25, seed=3)
    freq, l0 = FrequencyMetric(sae), L0Metric(sae)
    ctx = {"feature_acts": acts, "mask": None, "n_tokens": 32}
    freq.update(ctx), l0.update(ctx)
    rate = (acts > 0).float().mean(0)
    assert freq.compute()["sparsity/above_1e-1"] == float((rate > 0.1).sum())
    assert l0.compute()["metrics/l0"] == pytest.approx(float((acts > 0).float().sum(-1).mean()), rel=1e-6)


def test_loss_metric_reports_only_the_terms_it_saw():
    m = LossMetric(_Dictionary())
    m.update({"loss": torch.tensor([1.0, 3.0]), "l_rec": torch.tensor(2.0), "l_s": None})
    m.update({"loss": torch.tensor(4.0), "l_rec": torch.tensor(4.0)})
    got = m.compute()
    assert got == {"losses/overall_loss": pytest.approx(3.0), "losses/mse_loss": pytest.approx(3.0)}
    assert m.compute() == {}  # nothing new since
