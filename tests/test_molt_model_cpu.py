"""Mixture of linear transforms: ``out = sum_c a_c U_c V_c x`` with transforms of several ranks gated by a sparse encoder;
norms of the low-rank products, normalisation, folding of the dataset scale, metrics per rank group, and feature shards
whose gathered encoder keeps the logical (rank group, index) order (models/molt.py:72-99, 283-291, 543-654 of the
reference project)."""

import pytest
import torch

from language_model_saes_b200.models.molt import MixtureOfLinearTransform, MOLTConfig
from language_model_saes_b200.testing import distributed_test


def _molt(mesh=None, **kw):
    torch.manual_seed(0)
    base = dict(hook_point_in="a", hook_point_out="b", d_model=16, expansion_factor=0.75, rank_counts={2: 8, 4: 4}, act_fn="relu",
                norm_activation="inference", dtype=torch.float32, device="cpu")  # fmt: skip
    base.update(kw)
    m = MixtureOfLinearTransform(MOLTConfig(**base), mesh)
    m.init_parameters()
    with torch.no_grad():
        m.W_E.mul_(3.0)
        m.b_D.normal_(std=0.1)
    return m


def test_config_counts_transforms_and_splits_them_evenly_over_shards():
    cfg = _molt().cfg
    assert cfg.d_sae == 12 and cfg.available_ranks == [2, 4] and cfg.num_rank_types == 2
    assert cfg.generate_rank_assignments() == [2] * 8 + [4] * 4
    assert cfg.get_local_rank_assignments(2) == [2] * 4 + [4] * 2
    with pytest.raises(AssertionError, match="not divisible"):
        cfg.get_local_rank_assignments(3)
    with pytest.raises(Exception, match="Expansion factor"):
        MOLTConfig(hook_point_in="a", hook_point_out="b", d_model=16, expansion_factor=4, rank_counts={2: 8})


def test_decode_is_the_gated_sum_of_low_rank_maps_of_the_input():
    m = _molt()
    g = torch.Generator().manual_seed(1)
    x = torch.randn(9, 16, generator=g)
    acts = m.encode(x)
    assert acts.shape == (9, 12) and (acts >= 0).all() and 0 < int((acts > 0).sum()) < acts.numel()
    out = m.decode(acts, original_x=x)
    want = torch.zeros(9, 16)
    c = 0
    for r in (2, 4):
        U, V = m.U_matrices[str(r)], m.V_matrices[str(r)]  # [n, d, r], [n, r, d]
        for i in range(U.shape[0]):
            want += acts[:, c : c + 1] * (x @ V[i].T @ U[i].T)
            c += 1
    assert torch.allclose(out, want + m.b_D, atol=1e-5)
    assert torch.allclose(m(x), out, atol=1e-6)
    with pytest.raises(AssertionError, match="original_x"):
        m.decode(acts)


def test_decoder_norm_is_the_frobenius_norm_of_each_product_and_can_be_fixed():
    m = _molt()
    n = m.decoder_norm()
    c = 0
    for r in (2, 4):
        U, V = m.U_matrices[str(r)], m.V_matrices[str(r)]
        for i in range(U.shape[0]):
            assert float(n[c]) == pytest.approx(float((U[i] @ V[i]).norm()), rel=1e-4)
            c += 1
    g = torch.Generator().manual_seed(2)
    x = torch.randn(5, 16, generator=g)
    before = [(m.U_matrices[str(r)][0] @ m.V_matrices[str(r)][0]).clone() for r in (2, 4)]
    m.transform_to_unit_decoder_norm()
    assert torch.allclose(m.decoder_norm(), torch.ones(12), atol=1e-5)
    for r, b in zip((2, 4), before):  # the direction of every map is kept
        now = m.U_matrices[str(r)][0] @ m.V_matrices[str(r)][0]
        assert torch.allclose(now / now.norm(), b / b.norm(), atol=1e-5)
    m.set_decoder_to_fixed_norm(0.5, force_exact=False)  # only larger norms are brought down
    assert torch.allclose(m.decoder_norm(), torch.full((12,), 0.5), atol=1e-5)
    m.set_decoder_to_fixed_norm(2.0, force_exact=False)
    assert torch.allclose(m.decoder_norm(), torch.full((12,), 0.5), atol=1e-5)
    m.set_encoder_to_fixed_norm(1.5)
    assert torch.allclose(m.encoder_norm(), torch.full((12,), 1.5), atol=1e-5)
    assert m(x).shape == (5, 16)


def test_folding_the_dataset_scale_keeps_the_function_on_raw_activations():
    m = _molt(norm_activation="dataset-wise")
    m.set_dataset_average_activation_norm({"a": 8.0, "b": 2.0})
    g = torch.Generator().manual_seed(3)
    raw = {"a": torch.randn(6, 16, generator=g) * 2, "b": torch.randn(6, 16, generator=g)}
    with torch.no_grad():
        nb = m.normalize_activations(raw)
        want = m(nb["a"]) / (16**0.5 / 2.0)  # the model's output, back on the scale of hook point b
        m.standardize_parameters_of_dataset_norm()
        assert m.cfg.norm_activation == "inference"
        got = m(raw["a"])
    assert torch.allclose(got, want, atol=1e-4)


def test_training_metrics_report_l0_per_rank_group():
    m = _molt()
    acts = torch.zeros(4, 12)
    acts[:, 0] = 1.0  # one rank-2 transform fires everywhere
    acts[:2, 9] = 1.0  # one rank-4 transform on half of the tokens
    out = m.compute_training_metrics(l0=torch.tensor(0.0), feature_acts=acts)
    assert out["molt_metrics/l0_rank2"] == pytest.approx(1.0) and out["molt_metrics/l0_rank4"] == pytest.approx(0.5)
    assert out["molt_metrics/l0_rank2_ratio"] == pytest.approx(1 / 8) and out["molt_metrics/total_rank_sum"] == pytest.approx(1.0 * 2 + 0.5 * 4)


@distributed_test(nproc_per_node=2, backend="gloo")
def test_feature_shards_compute_the_same_function_and_gather_in_logical_order():
    import torch.distributed as dist

    from language_model_saes_b200.parallel.mesh import build_mesh

    full = _molt()
    mesh = build_mesh("cpu", (1, 2), ("data", "model"))
    shard = MixtureOfLinearTransform(full.cfg.model_copy(), mesh)
    shard.load_full_state_dict(full.full_state_dict())
    assert shard.rank_assignments == [2] * 4 + [4] * 2
    g = torch.Generator().manual_seed(4)
    x = torch.randn(7, 16, generator=g, requires_grad=True)
    y = torch.randn(7, 16, generator=g)
    want, got = full(x), shard(x)
    assert torch.allclose(want, got, atol=1e-5)
    back = shard.full_state_dict()
    for k, v in full.full_state_dict().items():
        assert torch.allclose(back[k], v, atol=1e-6, equal_nan=True), k  # the encoder's columns come back in (rank group, index) order
    # gradients of a shard are the matching slices of the single-process ones
    (want - y).pow(2).sum().backward()
    gx = x.grad.clone()
    x.grad = None
    (got - y).pow(2).sum().backward()
    part = x.grad.clone()  # every shard holds the part of the input gradient that flows through its own transforms
    dist.all_reduce(part)
    assert torch.allclose(part, gx, atol=1e-4)
    r = dist.get_rank()
    assert torch.allclose(shard.U_matrices["2"].grad, full.U_matrices["2"].grad[r * 4 : (r + 1) * 4], atol=1e-5)
    assert torch.allclose(shard.V_matrices["4"].grad, full.V_matrices["4"].grad[r * 2 : (r + 1) * 2], atol=1e-5)
    dist.barrier()
