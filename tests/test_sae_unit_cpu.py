"""Closed-form behaviour of the dictionaries on tiny literal weights (d_model 2, d_sae 4): norms, activation functions,
normalisation modes, dataset-norm folding, forward pass, state round trips. The cases restate what the reference
project checks in tests/unit/test_sae.py and tests/unit/test_crosscoder.py; the expected numbers are worked out by hand."""

import math

import pytest
import torch

from language_model_saes_b200.models.crosscoder import Crosscoder, CrosscoderConfig
from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
from language_model_saes_b200.models.sparse_dictionary import SparseDictionary
from language_model_saes_b200.utils.math import topk


def _sae(**kw):
    cfg = SAEConfig(hook_point_in="in", hook_point_out="out", d_model=2, expansion_factor=2, device="cpu", dtype=torch.float32,
                    **{"act_fn": "relu", "norm_activation": "token-wise", "sparsity_include_decoder_norm": True, **kw})  # fmt: skip
    sae = SparseAutoEncoder(cfg)
    with torch.no_grad():
        sae.W_E.copy_(torch.tensor([[1.0, 2.0, 3.0, 4.0], [5.0, 6.0, 7.0, 8.0]]))
        sae.b_E.copy_(torch.tensor([3.0, 2.0, 3.0, 4.0]))
        sae.W_D.copy_(torch.tensor([[1.0, 2.0], [3.0, 4.0], [5.0, 6.0], [7.0, 8.0]]))
        if cfg.use_decoder_bias:
            sae.b_D.copy_(torch.tensor([1.0, 2.0]))
    return sae


def test_norms_and_fixed_norm_ops():
    sae = _sae()
    assert torch.allclose(sae.encoder_norm(), torch.tensor([math.sqrt(26), math.sqrt(40), math.sqrt(58), math.sqrt(80)]))
    assert torch.allclose(sae.decoder_norm(), torch.tensor([math.sqrt(5), 5.0, math.sqrt(61), math.sqrt(113)]))
    assert torch.allclose(sae.decoder_bias_norm(), torch.tensor([math.sqrt(5)]))
    sae.set_decoder_to_fixed_norm(3.0, force_exact=True)
    assert torch.allclose(sae.decoder_norm(), torch.full((4,), 3.0))
    sae.set_decoder_to_fixed_norm(5.0, force_exact=False)  # rows below the bound are left alone
    assert torch.allclose(sae.decoder_norm(), torch.full((4,), 3.0))
    sae.set_encoder_to_fixed_norm(2.0)
    assert torch.allclose(sae.encoder_norm(), torch.full((4,), 2.0))
    sae2 = _sae()
    sae2.transform_to_unit_decoder_norm()
    assert torch.allclose(sae2.decoder_norm(), torch.ones(4))
    sae2.init_encoder_with_decoder_transpose(factor=2.0)
    assert torch.allclose(sae2.W_E, 2.0 * sae2.W_D.t())


def test_forward_relu_with_decoder_norm_gate():
    sae = _sae()
    x = torch.tensor([[1.0, -1.0]])
    h = x @ sae.W_E + sae.b_E  # [-1, -2, -1, 0]
    assert torch.allclose(h, torch.tensor([[-1.0, -2.0, -1.0, 0.0]]))
    acts, pre = sae.encode(x, return_hidden_pre=True)
    assert torch.equal(pre, h) and torch.equal(acts, torch.zeros(1, 4))
    x = torch.tensor([[1.0, 1.0]])
    acts = sae.encode(x)
    assert torch.allclose(acts, torch.tensor([[9.0, 10.0, 13.0, 16.0]]))  # relu(h * n) / n == h for h > 0
    out = sae.decode(acts)
    assert torch.allclose(out, acts @ sae.W_D + sae.b_D)
    assert torch.allclose(sae(x), out)


def test_topk_and_batchtopk_select_on_gated_values():
    sae = _sae(act_fn="topk", top_k=1)
    x = torch.tensor([[1.0, 1.0], [1.0, 0.0]])
    acts = sae.encode(x)
    # gated values h * ||W_D row||: the last feature wins in both rows; the activation is the ungated h
    assert torch.allclose(acts, torch.tensor([[0.0, 0.0, 0.0, 16.0], [0.0, 0.0, 0.0, 8.0]]))
    sae.set_current_k(2)
    assert (sae.encode(x) != 0).sum(-1).tolist() == [2, 2]
    bt = _sae(act_fn="batchtopk", top_k=1)
    acts = bt.encode(x)  # k * batch = 2 entries over the whole batch: 16*sqrt(113) and 13*sqrt(61) beat row 2
    assert (acts != 0).sum().item() == 2 and acts[0, 3] == 16.0 and acts[0, 2] == 13.0 and acts[1].abs().sum() == 0


def test_topk_helper_matches_definition():
    x = torch.tensor([[3.0, -5.0, 1.0, 4.0], [0.5, 0.2, -0.1, 0.0]])
    out, thr = topk(x, k=2, dim=-1, return_threshold=True)
    assert torch.equal(out, torch.tensor([[3.0, 0.0, 0.0, 4.0], [0.5, 0.2, 0.0, 0.0]])) and thr.tolist() == [3.0, pytest.approx(0.2)]
    assert torch.equal(topk(x, k=1, dim=-1, abs=True), torch.tensor([[0.0, -5.0, 0.0, 0.0], [0.5, 0.0, 0.0, 0.0]]))
    assert torch.equal(topk(x, k=3, dim=(0, 1)), torch.tensor([[3.0, 0.0, 1.0, 4.0], [0.0, 0.0, 0.0, 0.0]]))


def test_normalisation_modes():
    batch = {"in": torch.tensor([[3.0, 4.0], [6.0, 8.0]]), "out": torch.tensor([[0.0, 2.0], [2.0, 0.0]])}
    tok = _sae(norm_activation="token-wise")
    n = tok.normalize_activations(batch)
    assert torch.allclose(n["in"].norm(dim=-1), torch.full((2,), math.sqrt(2.0)))  # every token to sqrt(d_model)
    bw = _sae(norm_activation="batch-wise")
    n, scale = bw.normalize_activations(batch, return_scale_factor=True)
    assert torch.allclose(n["in"].norm(dim=-1).mean(), torch.tensor(math.sqrt(2.0)))
    back = bw.denormalize_activations(n, scale)
    assert torch.allclose(back["in"], batch["in"]) and torch.allclose(back["out"], batch["out"])
    ds = _sae(norm_activation="dataset-wise")
    ds.set_dataset_average_activation_norm({"in": 5.0, "out": 2.0})
    n = ds.normalize_activations(batch)
    assert torch.allclose(n["in"], batch["in"] * math.sqrt(2.0) / 5.0) and torch.allclose(n["out"], batch["out"] * math.sqrt(2.0) / 2.0)
    inf = _sae(norm_activation="inference")
    assert torch.equal(inf.normalize_activations(batch)["in"], batch["in"])


def test_dataset_norm_folding_keeps_the_function():
    sae = _sae(norm_activation="dataset-wise", act_fn="relu", sparsity_include_decoder_norm=False)
    sae.set_dataset_average_activation_norm({"in": 5.0, "out": 2.0})
    batch = {"in": torch.tensor([[3.0, 4.0], [1.0, -0.5]]), "out": torch.zeros(2, 2)}
    n, scale = sae.normalize_activations(batch, return_scale_factor=True)
    want = sae.denormalize_activations({"out": sae(n["in"])}, scale)["out"]  # normalise -> model -> un-normalise
    sae.standardize_parameters_of_dataset_norm()
    assert sae.cfg.norm_activation == "inference"
    got = sae(batch["in"])  # raw activations straight in
    assert torch.allclose(got, want, atol=1e-5)


def test_checkpoint_round_trip_formats(tmp_path):
    sae = _sae(norm_activation="dataset-wise")
    sae.set_dataset_average_activation_norm({"in": 5.0, "out": 2.0})
    for ext in ("safetensors", "pt"):
        d = tmp_path / ext
        d.mkdir()
        sae.save_checkpoint(d / f"sae_weights.{ext}")
        sae.cfg.save_hyperparameters(d)
        again = SparseDictionary.from_pretrained(str(d), fold_activation_scale=False, device="cpu", dtype=torch.float32)
        assert type(again) is SparseAutoEncoder and again.cfg.norm_activation == "dataset-wise"
        for k, v in sae.state_dict().items():
            assert torch.equal(again.state_dict()[k], v), k
        assert again.dataset_average_activation_norm == {"in": 5.0, "out": 2.0}
    folded = SparseDictionary.from_pretrained(str(tmp_path / "pt"), fold_activation_scale=True, device="cpu", dtype=torch.float32)
    assert folded.cfg.norm_activation == "inference"
    with pytest.raises(Exception):
        SparseDictionary.from_pretrained(str(tmp_path / "missing"))


def test_compute_loss_values_and_mask():
    sae = _sae(norm_activation="inference", act_fn="relu", sparsity_include_decoder_norm=False)
    x = torch.tensor([[1.0, 1.0], [1.0, -1.0]])
    batch = {"in": x, "out": torch.zeros(2, 2), "tokens": torch.tensor([5, 6])}
    out = sae.compute_loss(batch, return_aux_data=True, sparsity_loss_type=None)
    rec = sae(x)
    assert torch.allclose(out["l_rec"], rec.pow(2).sum(-1).mean()) and torch.allclose(out["loss"], rec.pow(2).sum(-1).mean())
    assert out["n_tokens"] == 2 and torch.equal(out["reconstructed"], rec)
    masked = sae.compute_loss({**batch, "mask": torch.tensor([True, False])}, return_aux_data=True, sparsity_loss_type=None)
    assert torch.allclose(masked["loss"], rec[0].pow(2).sum()) and masked["n_tokens"] == 1
    l1 = sae.compute_loss(batch, return_aux_data=True, sparsity_loss_type="power", p=1, l1_coefficient=0.5)
    want_l1 = 0.5 * (sae.encode(x) * sae.decoder_norm()).sum(-1)
    assert torch.allclose(l1["l_s"], want_l1) and torch.allclose(l1["loss"], (rec.pow(2).sum(-1) + want_l1).mean())


def _crosscoder():
    cfg = CrosscoderConfig(hook_points=["h0", "h1"], d_model=2, expansion_factor=2, act_fn="relu", device="cpu", dtype=torch.float32,
                           norm_activation="inference")  # fmt: skip
    cc = Crosscoder(cfg)
    with torch.no_grad():
        cc.W_E.copy_(torch.arange(16.0).view(2, 2, 4) / 10)
        cc.b_E.copy_(torch.tensor([[0.1, -0.2, 0.0, 0.3], [0.0, 0.1, -0.5, 0.2]]))
        cc.W_D.copy_(torch.arange(16.0).view(2, 4, 2) / 10 - 0.5)
        cc.b_D.copy_(torch.tensor([[0.1, 0.2], [0.3, 0.4]]))
    return cc


def test_crosscoder_shared_latent_and_per_head_decode():
    cc = _crosscoder()
    x = torch.tensor([[[1.0, 0.0], [0.0, 1.0]], [[-1.0, 2.0], [0.5, 0.5]]])  # [batch, head, d]
    pre_per_head = torch.einsum("bhd,hdf->bhf", x, cc.W_E) + cc.b_E
    shared = torch.relu(pre_per_head.sum(dim=1))  # pre-activations are summed over heads, one latent for all heads
    acts = cc.encode(x)
    assert acts.shape == (2, 2, 4) and torch.allclose(acts[:, 0], shared) and torch.allclose(acts[:, 1], shared)
    rec = cc.decode(acts)
    want = torch.einsum("bhf,hfd->bhd", acts, cc.W_D) + cc.b_D
    assert torch.allclose(rec, want)
    assert cc.decoder_norm().shape == (2, 4) and torch.allclose(cc.decoder_norm(), cc.W_D.norm(dim=-1))
    sims = cc.decoder_similarity_matrices()
    assert sims.shape == (4, 2, 2) and torch.allclose(sims[:, 0, 0], torch.ones(4)) and torch.allclose(sims, sims.transpose(1, 2))
    batch = {"h0": x[:, 0], "h1": x[:, 1], "tokens": torch.tensor([1, 2])}
    out = cc.compute_loss(batch, return_aux_data=True, sparsity_loss_type=None)
    assert torch.isfinite(out["loss"]) and out["feature_acts"].shape == (2, 2, 4)
    state = cc.full_state_dict()
    other = Crosscoder(cc.cfg)
    other.load_full_state_dict(state)
    assert torch.allclose(other.encode(x), acts)
