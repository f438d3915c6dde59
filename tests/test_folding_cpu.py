"""Folding the dataset-wise scale into the weights (``standardize_parameters_of_dataset_norm``): afterwards the model takes
raw activations and returns raw-scale reconstructions, and computes the same function as before on normalised ones."""

import pytest
import torch

from language_model_saes_b200.models.clt import CLTConfig, CrossLayerTranscoder
from language_model_saes_b200.models.lorsa import LorsaConfig, LowRankSparseAttention
from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder

D = 16


def _check(model, raw, hooks_in, hooks_out, norms, out_of):
    """``out_of(model, batch)`` -> reconstruction(s); compared on the raw scale of every output hook point."""
    model.set_dataset_average_activation_norm(norms)
    with torch.no_grad():
        before = out_of(model, model.normalize_activations(raw))
        model.standardize_parameters_of_dataset_norm()
        assert model.cfg.norm_activation == "inference"
        after = out_of(model, raw)
    return before, after


@pytest.mark.parametrize("act,gate", [("relu", False), ("topk", True), ("topk", False), ("jumprelu", False), ("jumprelu", True)])
@pytest.mark.parametrize("transcoder", [False, True])
def test_sae_and_transcoder(act, gate, transcoder):
    torch.manual_seed(0)
    hout = "post" if transcoder else "pre"
    m = SparseAutoEncoder(SAEConfig(hook_point_in="pre", hook_point_out=hout, d_model=D, expansion_factor=4, act_fn=act, top_k=6,
                                    norm_activation="dataset-wise", sparsity_include_decoder_norm=gate))  # fmt: skip
    m.init_parameters(encoder_uniform_bound=0.5, decoder_uniform_bound=0.5, init_log_jumprelu_threshold_value=-1.0)
    with torch.no_grad():
        m.b_E.normal_(std=0.2)
        m.b_D.normal_(std=0.2)
    g = torch.Generator().manual_seed(1)
    raw = {"pre": torch.randn(32, D, generator=g) * 3.0, "post": torch.randn(32, D, generator=g) * 0.5}
    norms = {"pre": 12.0, "post": 2.0} if transcoder else {"pre": 12.0}
    f_out = D**0.5 / norms[hout]
    before, after = _check(m, raw, ["pre"], [hout], norms, lambda mod, b: mod(b["pre"]))
    assert torch.allclose(after, before / f_out, atol=1e-4, rtol=1e-4)
    assert float(after.abs().mean()) > 0.01


@pytest.mark.parametrize("kw", [dict(), dict(positional_embedding_type="none"), dict(use_post_qk_ln=True, normalization_type="RMS")])
def test_lorsa(kw):
    torch.manual_seed(0)
    m = LowRankSparseAttention(LorsaConfig(hook_point_in="a", hook_point_out="b", d_model=D, expansion_factor=1, n_qk_heads=4, d_qk_head=8,
                                           rotary_dim=8, n_ctx=12, act_fn="topk", top_k=5, norm_activation="dataset-wise", **kw))  # fmt: skip
    m.init_parameters()
    with torch.no_grad():
        for b in (m.b_Q, m.b_K, m.b_V, m.b_D):
            b.normal_(std=0.1)
        m.W_Q.mul_(3)
        m.W_K.mul_(3)
    g = torch.Generator().manual_seed(1)
    raw = {"a": torch.randn(2, 12, D, generator=g) * 4.0, "b": torch.randn(2, 12, D, generator=g)}
    norms = {"a": 16.0, "b": 3.0}
    before, after = _check(m, raw, ["a"], ["b"], norms, lambda mod, b: mod(b["a"]))
    assert torch.allclose(after, before / (D**0.5 / 3.0), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("act", ["relu", "jumprelu"])
def test_cross_layer_transcoder_with_a_scale_per_hook_point(act):
    torch.manual_seed(0)
    L = 3
    m = CrossLayerTranscoder(CLTConfig(hook_points_in=[f"i{l}" for l in range(L)], hook_points_out=[f"o{l}" for l in range(L)], d_model=D,
                                       expansion_factor=2, act_fn=act, norm_activation="dataset-wise", sparsity_include_decoder_norm=False))  # fmt: skip
    m.init_parameters(init_log_jumprelu_threshold_value=-1.5)
    with torch.no_grad():
        m.W_E.mul_(4)
        m.b_E.normal_(std=0.1)
        for b in m.b_D:
            b.normal_(std=0.1)
    g = torch.Generator().manual_seed(1)
    raw = {f"i{l}": torch.randn(20, D, generator=g) * (l + 2) for l in range(L)} | {f"o{l}": torch.randn(20, D, generator=g) for l in range(L)}
    norms = {f"i{l}": 4.0 * (l + 2) for l in range(L)} | {f"o{l}": 1.0 + l for l in range(L)}

    def run(mod, b):
        x, kw, _ = mod.prepare_input(b)
        return mod.decode(mod.encode(x, **kw))  # [L, tokens, d]

    before, after = _check(m, raw, None, None, norms, run)
    for t in range(L):
        assert torch.allclose(after[t], before[t] / (D**0.5 / norms[f"o{t}"]), atol=1e-4, rtol=1e-4), t
