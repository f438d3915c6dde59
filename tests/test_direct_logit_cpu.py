"""Direct logit attribution of every dictionary family against the written definition: a feature's decoder direction (for a
cross-layer transcoder the directions from its layer towards every later one, summed after the final norm) goes through
the model's final norm and unembedding; the k largest and smallest logits are reported with their tokens
(analysis/direct_logit_attributor.py:15-164 of the reference project)."""

import pytest
import torch
from conftest import tiny_lm_config

from language_model_saes_b200.analysis import DirectLogitAttributor, DirectLogitAttributorConfig
from language_model_saes_b200.models.clt import CLTConfig, CrossLayerTranscoder
from language_model_saes_b200.models.crosscoder import Crosscoder, CrosscoderConfig
from language_model_saes_b200.models.lorsa import LorsaConfig, LowRankSparseAttention
from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
from language_model_saes_b200.resource_loaders import load_model


@pytest.fixture(scope="module")
def lm(tiny_lm_workspace):
    return load_model(tiny_lm_config(tiny_lm_workspace))


def _expected(directions, lm):
    h = lm.ln_final(directions[:, None, :]) if lm.cfg.normalization_type is not None else directions[:, None, :]
    return (h @ lm.W_U + lm.b_U)[:, 0]


def _check(records, logits, lm, k):
    assert len(records) == logits.shape[0]
    for f in (0, logits.shape[0] // 2, logits.shape[0] - 1):
        tv, ti = logits[f].topk(k)
        bv, bi = logits[f].topk(k, largest=False)
        assert [r["logit"] for r in records[f]["top_positive"]] == pytest.approx(tv.tolist(), rel=1e-5, abs=1e-6)
        assert [r["logit"] for r in records[f]["top_negative"]] == pytest.approx(bv.tolist(), rel=1e-5, abs=1e-6)
        assert [r["token"] for r in records[f]["top_positive"]] == [lm.tokenizer.decode([i]) for i in ti.tolist()]
        assert [r["token"] for r in records[f]["top_negative"]] == [lm.tokenizer.decode([i]) for i in bi.tolist()]


@torch.no_grad()
def test_single_layer_families(lm):
    torch.manual_seed(0)
    k = 4
    dla = DirectLogitAttributor(DirectLogitAttributorConfig(top_k=k))
    sae = SparseAutoEncoder(SAEConfig(hook_point_in="blocks.1.hook_resid_post", hook_point_out="blocks.1.hook_resid_post", d_model=16, expansion_factor=2, act_fn="topk", top_k=4))
    sae.init_parameters(encoder_uniform_bound=0.5, decoder_uniform_bound=0.5)
    _check(dla.direct_logit_attribute(sae, lm), _expected(sae.W_D, lm), lm, k)

    cc = Crosscoder(CrosscoderConfig(hook_points=["blocks.0.hook_resid_post", "blocks.1.hook_resid_post"], d_model=16, expansion_factor=2, act_fn="relu"))
    cc.init_parameters(encoder_uniform_bound=0.5, decoder_uniform_bound=0.5)
    _check(dla.direct_logit_attribute(cc, lm), _expected(cc.W_D[-1], lm), lm, k)  # the last head is the one nearest the logits

    lo = LowRankSparseAttention(LorsaConfig(hook_point_in="blocks.1.ln1.hook_normalized", hook_point_out="blocks.1.hook_attn_out", d_model=16,
                                            expansion_factor=2, n_qk_heads=4, d_qk_head=8, rotary_dim=8, n_ctx=32, act_fn="topk", top_k=4))  # fmt: skip
    lo.init_parameters(encoder_uniform_bound=0.5, decoder_uniform_bound=0.5)
    recs = dla.direct_logit_attribute(lo, lm)
    assert len(recs) == lo.cfg.n_ov_heads
    _check(recs, _expected(lo.W_O, lm), lm, k)


@torch.no_grad()
def test_cross_layer_transcoder_sums_over_the_layers_a_feature_writes_to(lm):
    torch.manual_seed(1)
    clt = CrossLayerTranscoder(CLTConfig(hook_points_in=[f"blocks.{l}.ln2.hook_normalized" for l in range(2)],
                                         hook_points_out=[f"blocks.{l}.hook_mlp_out" for l in range(2)], d_model=16, expansion_factor=2, act_fn="relu"))  # fmt: skip
    clt.init_parameters(encoder_uniform_bound=0.5, decoder_uniform_bound=0.5)
    k = 3
    dla = DirectLogitAttributor(DirectLogitAttributorConfig(top_k=k, clt_layer=0))
    both = _expected(clt.W_D[0][0], lm) + _expected(clt.W_D[1][0], lm)
    _check(dla.direct_logit_attribute(clt, lm), both, lm, k)  # the layer of the settings
    _check(dla.direct_logit_attribute(clt, lm, layer_idx=1), _expected(clt.W_D[1][1], lm), lm, k)  # an explicit layer wins
    with pytest.raises(AssertionError, match="layer_idx"):
        DirectLogitAttributor(DirectLogitAttributorConfig(top_k=k)).direct_logit_attribute(clt, lm)


def test_other_objects_are_refused(lm):
    dla = DirectLogitAttributor(DirectLogitAttributorConfig(top_k=2))
    with pytest.raises(NotImplementedError):
        dla.direct_logit_attribute(torch.nn.Linear(2, 2), lm)
    with pytest.raises(AssertionError, match="hooked"):
        dla.direct_logit_attribute(torch.nn.Linear(2, 2), object())
