"""Cross-layer transcoder: the decode definition ``y_t = sum_{s<=t} a_s W_D[t][s] + b_D[t]`` in its dense and sparse-matrix
forms, the single-layer analysis helpers, the per-feature decoder norms and the per-layer training metrics
(models/clt.py:526-876 of the reference project)."""

import pytest
import torch

from language_model_saes_b200.models.clt import CLTConfig, CrossLayerTranscoder


def _clt(act="relu", gate=False, L=3, d=8, F=16, k=4):
    torch.manual_seed(0)
    cfg = CLTConfig(hook_points_in=[f"i{l}" for l in range(L)], hook_points_out=[f"o{l}" for l in range(L)], d_model=d, expansion_factor=F / d,
                    act_fn=act, top_k=k, norm_activation="inference", sparsity_include_decoder_norm=gate)  # fmt: skip
    m = CrossLayerTranscoder(cfg)
    m.init_parameters(init_log_jumprelu_threshold_value=0.0)
    with torch.no_grad():
        m.W_E.mul_(4.0)
        for b in m.b_D:
            b.normal_(std=0.1)
    return m


def test_decode_is_the_sum_over_source_layers_up_to_the_target():
    m = _clt()
    g = torch.Generator().manual_seed(1)
    x = torch.randn(10, 3, 8, generator=g)
    acts = m.encode(x)
    y = m.decode(acts)
    assert y.shape == (3, 10, 8) and m.decode(acts, batch_first=True).shape == (10, 3, 8)
    for t in range(3):
        want = sum(acts[:, s] @ m.W_D[t][s] for s in range(t + 1)) + m.b_D[t]
        assert torch.allclose(y[t], want, atol=1e-5), t
    assert torch.equal(m.decode(acts, batch_first=True), y.movedim(0, -2))
    # a list of sparse matrices (one per source layer) decodes to the same thing
    sparse = [acts[:, s].to_sparse_csr() for s in range(3)]
    assert torch.allclose(m.decode(sparse), y, atol=1e-5)
    assert m.get_decoder_weights(2) is m.W_D[2] and m.W_D[2].shape == (3, 16, 8)
    assert m.cfg.n_decoders == 6


def test_single_layer_helpers_agree_with_the_full_encoder():
    m = _clt("relu")
    g = torch.Generator().manual_seed(2)
    batch = {f"i{l}": torch.randn(7, 8, generator=g) for l in range(3)}
    x, _, _ = m.prepare_input(batch)
    full, hp = m.encode(x, return_hidden_pre=True)
    for layer in range(3):
        xl, _, _ = m.prepare_input_single_layer(batch, layer)
        one, hp1 = m.encode_single_layer(xl, layer, return_hidden_pre=True)
        assert torch.allclose(one, full[:, layer], atol=1e-6) and torch.allclose(hp1, hp[:, layer], atol=1e-6)
    with pytest.raises(ValueError, match="Missing hook point i1"):
        m.prepare_input({"i0": batch["i0"], "i2": batch["i2"]})
    with pytest.raises(ValueError, match="Missing hook point i2"):
        m.prepare_input_single_layer({"i0": batch["i0"]}, 2)
    with pytest.raises(ValueError, match="Missing hook point o0"):
        m.prepare_label(batch)
    # a JumpReLU model: the layer's own thresholds
    j = _clt("jumprelu")
    with torch.no_grad():
        j.activation_function.log_jumprelu_threshold.fill_(0.0)  # threshold 1
    fullj = j.encode(x)
    for layer in range(3):
        assert torch.allclose(j.encode_single_layer(batch[f"i{layer}"], layer), fullj[:, layer], atol=1e-6)
    assert int((fullj != 0).sum()) < int((full != 0).sum())


def test_decoder_norms_per_feature_and_the_cached_single_layer_decoders():
    m = _clt()
    n = m.decoder_norm_per_feature()
    for s in range(3):
        want = torch.sqrt(sum(m.W_D[t][s].pow(2).sum(-1) for t in range(s, 3)))
        assert torch.allclose(n[s], want, atol=1e-6)
    one = m.decoder_norm_per_feature(layer=1)
    assert one.shape == (3, 16) and not one[0].any()
    assert torch.allclose(one[2], m.W_D[2][1].norm(dim=-1), atol=1e-6)
    assert torch.allclose(one[1:].pow(2).sum(0).sqrt(), n[1], atol=1e-6)  # the same norm, split by target layer
    m.keep_only_decoders_for_layer_from(1)
    assert torch.allclose(m.decoder_norm_per_feature(layer=1), one)
    with pytest.raises(AssertionError):
        m.decoder_norm_per_feature(layer=0)  # only the cached layer can be asked for
    assert torch.equal(m.decoder_norm(), torch.ones_like(m.decoder_norm()))  # the generic accessor is a placeholder here
    per_dec = m.decoder_norm_per_decoder()
    assert per_dec.numel() == 6 or per_dec.shape[0] == 6 or per_dec.shape == (3, 3)


def test_gated_selection_scales_back_to_pre_activations():
    m = _clt("topk", gate=True)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(9, 3, 8, generator=g)
    acts, gated_pre = m.encode(x, return_hidden_pre=True)
    raw = torch.einsum("bld,lds->bls", x, m.W_E) + m.b_E
    n = m.decoder_norm_per_feature()
    assert torch.allclose(gated_pre, raw * n, atol=1e-5)  # the encoder hands back what the selection ran on
    assert int((acts != 0).sum(-1).max()) <= 4
    on = acts != 0
    assert torch.allclose(acts[on], raw[on], atol=1e-5)  # activations themselves are un-gated
    # the kept entries are the largest GATED ones of their layer
    for b in range(9):
        for l in range(3):
            kept = set(torch.nonzero(acts[b, l]).flatten().tolist())
            score = (raw[b, l] * n[l]).clamp_min(0)
            best = set(score.topk(4).indices[score.topk(4).values > 0].tolist())
            assert kept == best


def test_training_metrics_name_every_layer():
    m = _clt()
    out = m.compute_training_metrics(l0=torch.tensor([[3.0, 5.0, 7.0], [5.0, 5.0, 9.0]]), explained_variance_legacy=torch.tensor([0.5, 0.6, 0.7]))
    assert out["metrics/explained_variance_L2"] == pytest.approx(0.7) and out["metrics/l0_layer0"] == pytest.approx(4.0)
    assert set(out) == {f"metrics/explained_variance_L{l}" for l in range(3)} | {f"metrics/l0_layer{l}" for l in range(3)}
