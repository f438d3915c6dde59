"""Per-feature records built from the analyser's tensors, and what each dictionary family adds to them: decoder norms and
head-by-head similarity for crosscoders, decoder norms per target layer for cross-layer transcoders, z patterns (which
source position feeds a head's activation at a target position) for attention dictionaries
(analysis/post_analysis/*.py of the reference project)."""

import numpy as np
import pytest
import torch

from language_model_saes_b200.analysis.post_analysis import get_post_analysis_processor
from language_model_saes_b200.models.clt import CLTConfig, CrossLayerTranscoder
from language_model_saes_b200.models.crosscoder import Crosscoder, CrosscoderConfig
from language_model_saes_b200.models.lorsa import LorsaConfig, LowRankSparseAttention
from language_model_saes_b200.utils.discrete import KeyedDiscreteMapper


def _samples(n, F, ctx, mapper, seed=0, values=None):
    """``n`` kept samples per feature: activations ``[n, F, ctx]``, the context each came from, dataset / model names."""
    g = torch.Generator().manual_seed(seed)
    acts = torch.relu(torch.randn(n, F, ctx, generator=g) - 0.5) if values is None else values
    return {"feature_acts": acts, "elt": acts.amax(-1), "context_idx": torch.arange(n)[:, None].expand(n, F).clone(),
            "dataset_name": torch.tensor(mapper.encode("dataset_name", ["toy"] * (n * F))).view(n, F),
            "model_name": torch.tensor(mapper.encode("model_name", ["tiny"] * (n * F))).view(n, F)}  # fmt: skip


def test_registry_knows_every_family_and_refuses_others():
    for kind in ("sae", "generic", "crosscoder", "clt", "lorsa"):
        assert get_post_analysis_processor(kind) is not None
    with pytest.raises(KeyError, match="No post-analysis processor"):
        get_post_analysis_processor("molt")
    # the analyser falls back to the common record for a family without a processor of its own
    from language_model_saes_b200.analysis.feature_analyzer import FeatureAnalyzer, FeatureAnalyzerConfig

    fallback = FeatureAnalyzer(FeatureAnalyzerConfig(total_analyzing_tokens=1)).get_post_analysis_func("molt")
    assert type(fallback).__name__ == "GenericPostAnalysisProcessor"


def test_generic_records_hold_statistics_and_sparse_samples():
    from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder

    F, n, ctx = 6, 3, 5
    sae = SparseAutoEncoder(SAEConfig(hook_point_in="h", hook_point_out="h", d_model=8, expansion_factor=F / 8, act_fn="relu"))
    mapper = KeyedDiscreteMapper()
    sub = _samples(n, F, ctx, mapper)
    act_times = torch.tensor([4, 0, 2, 9, 1, 3])
    peaks = sub["feature_acts"].amax((0, 2))
    out = get_post_analysis_processor("sae").process(sae, act_times, 1000, peaks, {"top_activations": sub, "skipped": None}, mapper)
    assert len(out) == F and [r["act_times"] for r in out] == act_times.tolist() and out[0]["n_analyzed_tokens"] == 1000
    for f, rec in enumerate(out):
        assert rec["max_feature_acts"] == pytest.approx(float(peaks[f]))
        (s,) = rec["samplings"]  # the empty sampling is dropped
        assert s["name"] == "top_activations" and s["dataset_name"] == ["toy"] * n and s["model_name"] == ["tiny"] * n
        dense = np.zeros((n, ctx), dtype=np.float32)
        r, c = s["feature_acts_indices"].astype(int)
        dense[r, c] = s["feature_acts_values"]
        assert np.allclose(dense, sub["feature_acts"][:, f].numpy())
        assert s["context_idx"].tolist() == [0, 1, 2] and s["n_shards"].tolist() == [1, 1, 1]


def test_crosscoder_records_add_norms_and_head_similarities():
    torch.manual_seed(0)
    H, d, F = 3, 8, 4
    cc = Crosscoder(CrosscoderConfig(hook_points=[f"s{i}" for i in range(H)], d_model=d, expansion_factor=F / d, act_fn="relu"))
    cc.init_parameters(encoder_uniform_bound=0.3, decoder_uniform_bound=0.3)
    with torch.no_grad():
        cc.W_D.copy_(torch.randn(H, F, d))
    mapper = KeyedDiscreteMapper()
    out = get_post_analysis_processor("crosscoder").process(cc, torch.ones(F, dtype=torch.long), 10, torch.ones(F), {"top": _samples(2, F, 3, mapper)}, mapper)
    W = cc.W_D.detach()
    for f, rec in enumerate(out):
        assert np.allclose(rec["decoder_norms"], W[:, f].norm(dim=-1).numpy(), atol=1e-6)
        inner = W[:, f] @ W[:, f].T
        assert np.allclose(rec["decoder_inner_product_matrices"], inner.numpy(), atol=1e-5)
        cos = inner / (W[:, f].norm(dim=-1)[:, None] * W[:, f].norm(dim=-1)[None, :])
        assert np.allclose(rec["decoder_similarity_matrices"], cos.numpy(), atol=1e-5) and np.allclose(np.diag(rec["decoder_similarity_matrices"]), 1.0, atol=1e-5)


def test_cross_layer_records_add_the_norm_towards_every_target_layer():
    torch.manual_seed(0)
    L, d, F = 3, 8, 4
    clt = CrossLayerTranscoder(CLTConfig(hook_points_in=[f"i{l}" for l in range(L)], hook_points_out=[f"o{l}" for l in range(L)], d_model=d,
                                         expansion_factor=F / d, act_fn="relu"))  # fmt: skip
    clt.init_parameters()
    mapper = KeyedDiscreteMapper()
    out = get_post_analysis_processor("clt").process(clt, torch.ones(F, dtype=torch.long), 10, torch.ones(F), {"top": _samples(2, F, 3, mapper)}, mapper,
                                                     clt_layer=1)  # fmt: skip
    for f, rec in enumerate(out):
        norms = rec["decoder_norms"]
        assert norms.shape == (L,) and norms[0] == 0  # layer 1 does not write to layer 0
        for t in (1, 2):
            assert norms[t] == pytest.approx(float(clt.W_D[t][1, f].norm()), rel=1e-5)


class _Replay:
    """Stands in for the activation factory: the contexts again, in batches, with the metadata that names them."""

    def __init__(self, xs, hook):
        self.xs, self.hook, self.calls = xs, hook, 0

    def process(self, **kwargs):
        self.calls += 1
        for lo in range(0, len(self.xs), 2):
            yield {self.hook: torch.stack(self.xs[lo : lo + 2]), "meta": [{"context_idx": lo + j} for j in range(len(self.xs[lo : lo + 2]))]}


def test_attention_dictionary_records_add_z_patterns_that_sum_to_the_activations():
    torch.manual_seed(0)
    d, ctx, n_ctx_total = 16, 6, 4
    lo = LowRankSparseAttention(LorsaConfig(hook_point_in="blocks.0.ln1.hook_normalized", hook_point_out="blocks.0.hook_attn_out", d_model=d,
                                            expansion_factor=0.5, n_qk_heads=2, d_qk_head=8, rotary_dim=8, n_ctx=ctx, act_fn="relu",
                                            norm_activation="inference"))  # fmt: skip
    lo.init_parameters()
    F = lo.cfg.d_sae
    g = torch.Generator().manual_seed(1)
    xs = [torch.randn(ctx, d, generator=g) for _ in range(n_ctx_total)]
    with torch.no_grad():
        acts_all = torch.stack([lo.encode(x[None])[0] for x in xs])  # [contexts, ctx, F]
    # every head keeps two samples: contexts (head % 4) and ((head + 1) % 4)
    n = 2
    which = torch.stack([torch.arange(F) % n_ctx_total, (torch.arange(F) + 1) % n_ctx_total])  # [n, F]
    vals = torch.stack([torch.stack([acts_all[which[s, f], :, f] for f in range(F)]) for s in range(n)])  # [n, F, ctx]
    mapper = KeyedDiscreteMapper()
    sub = _samples(n, F, ctx, mapper, values=vals)
    sub["context_idx"] = which.clone()
    act_times = (vals != 0).sum((0, 2))
    proc = get_post_analysis_processor("lorsa")
    proc.rel_threshold = 0.0  # keep every contribution, so that they add up exactly
    replay = _Replay(xs, lo.cfg.hook_point_in)
    out = proc.process(lo, act_times, 100, vals.amax((0, 2)), {"top_activations": sub}, mapper, activation_factory=replay)
    assert replay.calls == 1 and len(out) == F
    checked = 0
    for f, rec in enumerate(out):
        (s,) = rec["samplings"]
        zi, zv = np.asarray(s["z_pattern_indices"]).astype(int), np.asarray(s["z_pattern_values"])
        assert zi.shape[0] == 3 and zi.shape[1] == zv.shape[0]
        if act_times[f] == 0:
            assert zv.size == 0
            continue
        assert (zi[2] <= zi[1]).all()  # causal: a source position is never after its target
        total = np.zeros((n, ctx))
        np.add.at(total, (zi[0], zi[1]), zv)
        want = vals[:, f].numpy()
        live = want != 0
        assert np.allclose(total[live], want[live], atol=1e-4)  # the contributions of all source positions make up the activation
        assert not total[~live].any()  # nothing is kept where the head is silent
        checked += int(live.sum())
    assert checked > 10
