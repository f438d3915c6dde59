"""``Crosscoder`` method by method on hand-sized tensors: the behaviours that tests/unit/test_crosscoder.py of the reference
project pins down (initialisation shapes and ranges, encode / decode / forward values, the norms, fixed-norm rescaling,
encoder from decoder transpose, input / label preparation incl. padding of narrow heads, loss values with and without
sparsity terms and token masks, folding of the dataset norms, decoder inner-product and similarity matrices)."""

import math

import pytest
import torch

from language_model_saes_b200.models.crosscoder import Crosscoder, CrosscoderConfig

H, D, F = 2, 2, 4
HOOKS = ["h0", "h1"]


def _cfg(**kw) -> CrosscoderConfig:
    base = dict(hook_points=HOOKS, d_model=D, expansion_factor=F / D, act_fn="relu", device="cpu", dtype=torch.float32, norm_activation="inference")
    base.update(kw)
    return CrosscoderConfig(**base)


@pytest.fixture
def cc() -> Crosscoder:
    m = Crosscoder(_cfg())
    with torch.no_grad():
        m.W_E.copy_(torch.tensor([[[1.0, 2.0, 3.0, 4.0], [5.0, 6.0, 7.0, 8.0]], [[9.0, 10.0, 11.0, 12.0], [13.0, 14.0, 15.0, 16.0]]]))
        m.b_E.copy_(torch.tensor([[1.0, 2.0, 3.0, 4.0], [5.0, 6.0, 7.0, 8.0]]))
        m.W_D.copy_(torch.tensor([[[1.0, 2.0], [3.0, 4.0], [5.0, 6.0], [7.0, 8.0]], [[9.0, 10.0], [11.0, 12.0], [13.0, 14.0], [15.0, 16.0]]]))
        m.b_D.copy_(torch.tensor([[1.0, 2.0], [3.0, 4.0]]))
    return m


X = torch.tensor([[[1.0, 2.0], [3.0, 4.0]], [[5.0, 6.0], [7.0, 8.0]]])  # [batch, head, d]


def test_init_parameters_shapes_and_ranges():
    m = Crosscoder(_cfg(act_fn="jumprelu"))
    m.init_parameters(encoder_uniform_bound=0.25, decoder_uniform_bound=0.5, init_log_jumprelu_threshold_value=-0.7)
    assert m.W_E.shape == (H, D, F) and m.W_D.shape == (H, F, D) and m.b_E.shape == (H, F) and m.b_D.shape == (H, D)
    assert m.W_E.abs().max() <= 0.25 and m.W_D.abs().max() <= 0.5 and m.W_D.abs().max() > 0.05
    assert torch.all(m.b_E == 0) and torch.all(m.b_D == 0)
    assert torch.allclose(m.activation_function.log_jumprelu_threshold, torch.full((F,), -0.7))
    assert m.n_heads_local == H and m.cfg.n_heads == H and m.local_hook_points() == HOOKS
    assert m.cfg.associated_hook_points == HOOKS and m.cfg.hooks_in == HOOKS and m.cfg.hooks_out == HOOKS


def test_encode_sums_pre_activations_over_heads(cc):
    per_head = torch.einsum("bhd,hdf->bhf", X, cc.W_E) + cc.b_E
    # head 0, token 0: [1, 2] @ [[1, 2, 3, 4], [5, 6, 7, 8]] + [1, 2, 3, 4] = [12, 16, 20, 24]
    assert per_head[0, 0].tolist() == [12.0, 16.0, 20.0, 24.0]
    shared = per_head.sum(1)
    acts, pre = cc.encode(X, return_hidden_pre=True)
    assert acts.shape == (2, H, F) and pre.shape == (2, H, F)
    for h in range(H):  # every head sees the same summed pre-activation; with ReLU and positive values act == pre
        assert torch.allclose(pre[:, h], shared) and torch.allclose(acts[:, h], shared)
    neg = cc.encode(-X * 10)
    assert torch.all(neg == 0)  # all pre-activations negative: ReLU kills everything
    single = cc.encode(X[0])  # an unbatched token works too
    assert single.shape == (H, F) and torch.allclose(single, acts[0])


def test_decode_is_per_head(cc):
    acts = torch.tensor([[[1.0, 0.0, 2.0, 0.0], [0.0, 1.0, 0.0, 1.0]]])
    rec = cc.decode(acts)
    # head 0: 1 * [1, 2] + 2 * [5, 6] + b_D[0] = [12, 16]; head 1: [11, 12] + [15, 16] + [3, 4] = [29, 32]
    assert rec.tolist() == [[[12.0, 16.0], [29.0, 32.0]]]


def test_forward_is_decode_of_encode(cc):
    out = cc.forward(X)
    assert out.shape == X.shape and torch.allclose(out, cc.decode(cc.encode(X)))


def test_norms(cc):
    assert torch.allclose(cc.decoder_norm(), cc.W_D.norm(dim=-1)) and cc.decoder_norm().shape == (H, F)
    assert cc.decoder_norm(keepdim=True).shape == (H, F, 1)
    assert torch.allclose(cc.encoder_norm(), cc.W_E.norm(dim=-2)) and cc.encoder_norm().shape == (H, F)
    assert math.isclose(float(cc.decoder_norm()[0, 0].detach()), math.sqrt(5.0), rel_tol=1e-6)
    assert torch.allclose(cc.decoder_bias_norm(), cc.b_D.norm(dim=-1, keepdim=True)) and cc.decoder_bias_norm().shape == (H, 1)


def test_set_decoder_to_fixed_norm(cc):
    before = cc.W_D.clone()
    cc.set_decoder_to_fixed_norm(2.0, force_exact=True)
    assert torch.allclose(cc.decoder_norm(), torch.full((H, F), 2.0), atol=1e-6)
    assert torch.allclose(torch.nn.functional.normalize(cc.W_D, dim=-1), torch.nn.functional.normalize(before, dim=-1), atol=1e-6)
    cc.set_decoder_to_fixed_norm(5.0, force_exact=False)  # rows already shorter than the bound stay as they are
    assert torch.allclose(cc.decoder_norm(), torch.full((H, F), 2.0), atol=1e-6)
    cc.set_decoder_to_fixed_norm(1.0, force_exact=False)  # longer rows are brought down to it
    assert torch.allclose(cc.decoder_norm(), torch.ones(H, F), atol=1e-6)


def test_set_encoder_to_fixed_norm(cc):
    cc.set_encoder_to_fixed_norm(3.0)
    assert torch.allclose(cc.encoder_norm(), torch.full((H, F), 3.0), atol=1e-5)


def test_init_encoder_with_decoder_transpose(cc):
    cc.init_encoder_with_decoder_transpose()
    assert torch.equal(cc.W_E, cc.W_D.transpose(1, 2))
    cc.init_encoder_with_decoder_transpose(0.5)
    assert torch.allclose(cc.W_E, 0.5 * cc.W_D.transpose(1, 2))


def test_prepare_input_and_label_stack_heads_and_pad_narrow_ones(cc):
    batch = {"h0": X[:, 0], "h1": X[:, 1], "tokens": torch.tensor([3, 4])}
    x, enc_kw, dec_kw = cc.prepare_input(batch)
    assert x.shape == (2, H, D) and torch.equal(x, X) and enc_kw == {} and dec_kw == {}
    assert torch.equal(cc.prepare_label(batch), X)
    narrow = {"h0": X[:, 0], "h1": X[:, 1, :1], "tokens": torch.tensor([3, 4])}  # a head with a narrower residual stream
    xn, _, _ = cc.prepare_input(narrow)
    assert xn.shape == (2, H, D) and torch.equal(xn[:, 1], torch.tensor([[3.0, 0.0], [7.0, 0.0]]))
    with pytest.raises(Exception):
        cc.prepare_input({"h0": torch.zeros(2, D + 1), "h1": X[:, 1]})  # wider than d_model: no way to fit


def test_compute_loss_values(cc):
    batch = {"h0": X[:, 0], "h1": X[:, 1], "tokens": torch.tensor([3, 4])}
    out = cc.compute_loss(batch, return_aux_data=True, sparsity_loss_type=None)
    rec = cc.forward(X)
    want = (rec - X).pow(2).sum(-1).mean()  # mean over tokens AND heads of the squared error
    assert torch.allclose(out["loss"], want) and out["feature_acts"].shape == (2, H, F) and torch.allclose(out["reconstructed"], rec)
    assert out["l_s"] is None and out["n_tokens"] == 2 and torch.allclose(out["l_rec"].mean(), want)
    plain = cc.compute_loss(batch, return_aux_data=False, sparsity_loss_type=None)
    assert isinstance(plain, torch.Tensor) and torch.allclose(plain, want)
    # tanh penalty on the decoder-norm-gated activations, summed over features, mean over tokens and heads
    acts = cc.encode(X)
    l_s = torch.tanh(4.0 * acts * cc.decoder_norm()).sum(-1).mean()
    with_s = cc.compute_loss(batch, return_aux_data=True, sparsity_loss_type="tanh", l1_coefficient=0.1, tanh_stretch_coefficient=4.0)
    assert torch.allclose(with_s["loss"], want + 0.1 * l_s, rtol=1e-6)
    # power (L1) penalty
    l1 = (acts * cc.decoder_norm()).abs().sum(-1).mean()
    with_l1 = cc.compute_loss(batch, return_aux_data=True, sparsity_loss_type="power", l1_coefficient=0.01, p=1)
    assert torch.allclose(with_l1["loss"], want + 0.01 * l1, rtol=1e-6)
    # a token mask drops tokens from every head's mean
    masked = cc.compute_loss({**batch, "mask": torch.tensor([True, False])}, return_aux_data=True, sparsity_loss_type=None)
    assert torch.allclose(masked["loss"], (rec[:1] - X[:1]).pow(2).sum(-1).mean())


def test_loss_gradients_reach_every_parameter(cc):
    batch = {"h0": X[:, 0], "h1": X[:, 1], "tokens": torch.tensor([3, 4])}
    cc.compute_loss(batch, return_aux_data=True, sparsity_loss_type="tanh", l1_coefficient=0.1)["loss"].backward()
    for name, p in cc.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all() and p.grad.abs().sum() > 0, name


def test_standardize_parameters_of_dataset_norm_rescales_the_biases_per_head():
    """As in the reference (models/crosscoder.py:522-538): both biases of head h are divided by sqrt(d) / norm_h, the
    weights stay, and the model switches to ``inference`` normalisation. With equal norms on all heads the folded model
    reproduces, on raw activations, what the unfolded one computed on normalised ones."""
    m = Crosscoder(_cfg(norm_activation="dataset-wise"))
    torch.manual_seed(0)
    m.init_parameters(encoder_uniform_bound=0.5, decoder_uniform_bound=0.5)
    with torch.no_grad():
        m.b_E.normal_()
        m.b_D.normal_()
    m.set_dataset_average_activation_norm({"h0": 3.0, "h1": 0.5})
    b_E, b_D, W_E, W_D = (t.clone() for t in (m.b_E, m.b_D, m.W_E, m.W_D))
    m.standardize_parameters_of_dataset_norm()
    assert m.cfg.norm_activation == "inference"
    f = torch.tensor([math.sqrt(D) / 3.0, math.sqrt(D) / 0.5]).view(H, 1)
    assert torch.allclose(m.b_E, b_E / f) and torch.allclose(m.b_D, b_D / f) and torch.equal(m.W_E, W_E) and torch.equal(m.W_D, W_D)

    same = Crosscoder(_cfg(norm_activation="dataset-wise"))
    same.init_parameters(encoder_uniform_bound=0.5, decoder_uniform_bound=0.5)
    with torch.no_grad():
        same.b_E.normal_()
        same.b_D.normal_()
    same.set_dataset_average_activation_norm({"h0": 2.0, "h1": 2.0})
    x = torch.randn(5, H, D) * 2.0
    s = math.sqrt(D) / 2.0
    before = same.forward(x * s) / s  # normalise, run, bring back to the raw scale
    same.standardize_parameters_of_dataset_norm()
    assert torch.allclose(same.forward(x), before, atol=1e-5)


def test_decoder_inner_product_and_similarity_matrices(cc):
    inner = cc.decoder_inner_product_matrices()
    assert inner.shape == (F, H, H)
    want = torch.einsum("hfd,gfd->fhg", cc.W_D, cc.W_D)
    assert torch.allclose(inner, want) and torch.allclose(inner, inner.transpose(1, 2))
    assert inner[0, 0, 1] == 1 * 9 + 2 * 10  # feature 0: <[1, 2], [9, 10]>
    sims = cc.decoder_similarity_matrices()
    unit = torch.nn.functional.normalize(cc.W_D, dim=-1)
    assert torch.allclose(sims, torch.einsum("hfd,gfd->fhg", unit, unit), atol=1e-6)
    assert torch.allclose(torch.diagonal(sims, dim1=1, dim2=2), torch.ones(F, H), atol=1e-6) and sims.abs().max() <= 1 + 1e-6


def test_state_dict_round_trip_and_jumprelu_thresholds(tmp_path):
    m = Crosscoder(_cfg(act_fn="jumprelu"))
    m.init_parameters(encoder_uniform_bound=0.5, decoder_uniform_bound=0.5, init_log_jumprelu_threshold_value=0.2)
    acts, pre = m.encode(X, return_hidden_pre=True)
    gated = pre * m.decoder_norm()
    theta = m.activation_function.log_jumprelu_threshold.exp()
    assert torch.equal(acts != 0, gated > theta)  # a head is active where ITS gated pre-activation passes the shared threshold
    assert torch.allclose(acts[acts != 0], pre[acts != 0])
    m.save_pretrained(str(tmp_path / "cc"))
    m.cfg.save_hyperparameters(str(tmp_path / "cc"))
    again = Crosscoder.from_pretrained(str(tmp_path / "cc"), device="cpu", dtype=torch.float32)
    assert type(again) is Crosscoder and torch.allclose(again.encode(X), acts)
