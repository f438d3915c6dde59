"""The initialiser's model-aware paths on the tiny language model: a Lorsa whose QK heads are copies of the model's
attention heads attends like the model; value / output projections are placed in the principal subspace of each original
head; a transcoder's decoder rows are the MLP's responses to its encoder directions; an SAE's decoder lies in the active
subspace of its labels (initializer.py:164-271, models/lorsa.py:280-503, models/sae.py:440-507 of the reference project)."""

import math

import pytest
import torch
from conftest import tiny_lm_config

from language_model_saes_b200.backend.language_model import HookedLanguageModel
from language_model_saes_b200.initializer import Initializer, InitializerConfig
from language_model_saes_b200.models.lorsa import LorsaConfig, LowRankSparseAttention
from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder

LAYER = 1
RAW = {"text": ["the cat sat on a mat the dog ran far away", "big red sun is blue sky a cat ran on the mat"]}


@pytest.fixture(scope="module")
def lm(tiny_lm_workspace):
    model = HookedLanguageModel(tiny_lm_config(tiny_lm_workspace))
    with torch.no_grad():  # the copies take the projections only: compare against a model without attention biases
        attn = model.attention_module(LAYER)
        attn.b_Q.zero_()
        attn.b_K.zero_()
    return model


def _acts(lm, hooks):
    out = lm.to_activations(RAW, hooks + ["blocks.1.attn.hook_pattern"])
    return out


def _lorsa(norm, rep=2, **kw):
    cfg = LorsaConfig(hook_point_in=f"blocks.{LAYER}.ln1.hook_normalized", hook_point_out=f"blocks.{LAYER}.hook_attn_out", d_model=16,
                      expansion_factor=2, n_qk_heads=2 * rep, d_qk_head=8, rotary_dim=8, positional_embedding_type="none", n_ctx=32,
                      act_fn="relu", norm_activation="dataset-wise", **kw)  # fmt: skip
    lo = LowRankSparseAttention(cfg)
    lo.init_parameters()
    lo.set_dataset_average_activation_norm(norm)
    return lo


def test_lorsa_with_the_models_qk_heads_attends_like_the_model(lm):
    hin, hout = f"blocks.{LAYER}.ln1.hook_normalized", f"blocks.{LAYER}.hook_attn_out"
    a = _acts(lm, [hin, hout])
    norm = {hin: float(a[hin].norm(dim=-1).mean()), hout: float(a[hout].norm(dim=-1).mean())}
    lo = _lorsa(norm)
    with torch.no_grad():
        lo.init_lorsa_with_mhsa(lm.attention_module(LAYER))
        x = lo.normalize_activations({hin: a[hin], hout: a[hout]})[hin]
        q, k, _ = lo._compute_qkv(x)
        patterns = lo._compute_attention_pattern(q, k)  # [qk heads, batch, q, k]
    want = a["blocks.1.attn.hook_pattern"]  # [batch, heads, q, k]
    for h in range(4):  # each of the model's two heads was copied twice, in order
        assert torch.allclose(patterns[h], want[:, h // 2], atol=1e-4), h
    assert not torch.allclose(patterns[0], patterns[2], atol=1e-3)  # and the two originals differ from each other


@pytest.mark.parametrize("side", ["value", "output"])
def test_lorsa_ov_heads_start_inside_the_active_subspace_of_their_original_head(lm, side):
    hin, hout = f"blocks.{LAYER}.ln1.hook_normalized", f"blocks.{LAYER}.hook_attn_out"
    a = _acts(lm, [hin, hout])
    norm = {hin: float(a[hin].norm(dim=-1).mean()), hout: float(a[hout].norm(dim=-1).mean())}
    lo = _lorsa(norm)
    mhsa = lm.attention_module(LAYER)
    batch = lo.normalize_activations({hin: a[hin], hout: a[hout]})
    with torch.no_grad():
        if side == "value":
            lo.init_W_V_with_active_subspace_per_head(batch=batch, mhsa=mhsa)
        else:
            lo.init_W_D_with_active_subspace_per_head(batch=batch, mhsa=mhsa)
    assert torch.allclose(lo.W_V.norm(dim=1), torch.ones(lo.cfg.d_sae), atol=1e-5) and torch.allclose(lo.W_O.norm(dim=1), torch.ones(lo.cfg.d_sae), atol=1e-5)
    per = lo.cfg.d_sae // 2
    for h in range(2):  # the OV heads derived from original head h
        sl = slice(h * per, (h + 1) * per)
        ov = mhsa.W_V[h] @ mhsa.W_O[h]  # [d, d]: what the original head writes for a value read from x
        if side == "value":
            # W_O follows W_V through the original head's OV map
            want = lo.W_V[sl] @ ov
            assert torch.allclose(lo.W_O[sl], want / want.norm(dim=1, keepdim=True), atol=1e-4)
            assert torch.linalg.matrix_rank(lo.W_V[sl]) <= lo.cfg.d_qk_head
        else:
            assert torch.linalg.matrix_rank(lo.W_O[sl]) <= lo.cfg.d_qk_head
            want = lo.W_O[sl] @ ov.T
            cos = torch.nn.functional.cosine_similarity(lo.W_V[sl], want, dim=1)
            assert float(cos.min()) > 0.999


def test_transcoder_decoder_rows_are_the_mlps_responses_to_the_encoder_directions(lm):
    hin, hout = f"blocks.{LAYER}.ln2.hook_normalized", f"blocks.{LAYER}.hook_mlp_out"
    a = lm.to_activations(RAW, [hin, hout])
    norm = {hin: float(a[hin].norm(dim=-1).mean()), hout: float(a[hout].norm(dim=-1).mean())}
    tc = SparseAutoEncoder(SAEConfig(hook_point_in=hin, hook_point_out=hout, d_model=16, expansion_factor=2, act_fn="relu",
                                     norm_activation="dataset-wise"))  # fmt: skip
    tc.init_parameters(encoder_uniform_bound=0.3, decoder_uniform_bound=0.3)
    tc.set_dataset_average_activation_norm(norm)
    mlp = lm.mlp_module(LAYER)
    batch = tc.normalize_activations({hin: a[hin], hout: a[hout]})
    before = tc.W_E.detach().clone()
    with torch.no_grad():
        tc.init_tc_with_mlp(batch=batch, mlp=mlp)
        dirs = before / before.norm(dim=0, keepdim=True)
        assert torch.allclose(tc.W_E, dirs, atol=1e-6)  # encoder columns: the same directions, unit length
        x = a[hin].reshape(-1, 16)  # the raw activations (the model's scale)
        mean, radius = x.mean(0), (x - x.mean(0)).norm(dim=1).mean()
        resp = mlp.forward(mean + (dirs * radius).T)
        resp = resp - resp.mean(0)
        assert torch.allclose(tc.W_D, resp / resp.norm(dim=1, keepdim=True), atol=1e-4)
    assert torch.allclose(tc.W_D.norm(dim=1), torch.ones(32), atol=1e-5)


def test_initializer_runs_the_model_aware_paths_from_its_config(lm):
    hin, hout = f"blocks.{LAYER}.ln1.hook_normalized", f"blocks.{LAYER}.hook_attn_out"
    a = _acts(lm, [hin, hout])
    stream = [{hin: a[hin], hout: a[hout], "tokens": a["tokens"]} for _ in range(10)]
    cfg = LorsaConfig(hook_point_in=hin, hook_point_out=hout, d_model=16, expansion_factor=2, n_qk_heads=4, d_qk_head=8, rotary_dim=8,
                      positional_embedding_type="none", n_ctx=32, act_fn="topk", top_k=4, norm_activation="dataset-wise")  # fmt: skip
    init = Initializer(InitializerConfig(initialize_lorsa_with_mhsa=True, initialize_W_D_with_active_subspace=True, model_layer=LAYER,
                                         grid_search_init_norm=False, init_encoder_with_decoder_transpose=False))  # fmt: skip
    lo = init.initialize_sae_from_config(cfg, activation_stream=iter(stream), model=lm)
    mhsa = lm.attention_module(LAYER)
    f_in = math.sqrt(16) / lo.dataset_average_activation_norm[hin]
    assert torch.allclose(lo.W_Q[0] * f_in, mhsa.W_Q[0], atol=1e-5) and torch.allclose(lo.W_Q[1] * f_in, mhsa.W_Q[0], atol=1e-5)
    assert torch.allclose(lo.W_V.norm(dim=1), torch.ones(lo.cfg.d_sae), atol=1e-4)
    with pytest.raises(AssertionError, match="hooked language model and model_layer"):
        init.initialize_sae_from_config(cfg, activation_stream=iter(stream), model=None)


def test_sae_decoder_can_start_inside_the_active_subspace_of_its_labels():
    torch.manual_seed(0)
    sae = SparseAutoEncoder(SAEConfig(hook_point_in="h", hook_point_out="h", d_model=16, expansion_factor=4, act_fn="relu", norm_activation="inference"))
    sae.init_parameters(encoder_uniform_bound=0.3, decoder_uniform_bound=0.3)
    basis = torch.linalg.qr(torch.randn(16, 5)).Q  # the data lives in 5 directions (plus a little noise)
    x = torch.randn(400, 5) @ basis.T * 3 + 0.01 * torch.randn(400, 16)
    with torch.no_grad():
        sae.init_W_D_with_active_subspace(batch={"h": x}, d_active_subspace=5)
    outside = sae.W_D - (sae.W_D @ basis) @ basis.T
    assert float(outside.norm()) < 0.02 * float(sae.W_D.norm()) and int(torch.linalg.matrix_rank(sae.W_D, atol=1e-3)) == 5
