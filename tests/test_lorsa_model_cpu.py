"""Low-rank sparse attention model: rotary tables (plain and NTK-by-parts), scores that depend on relative position only,
the fast attention path against the pattern path, z patterns, and loading a checkpoint with fewer QK heads
(models/lorsa.py:525-575, 642-762, 831-904, 960-980 of the reference project)."""

import math

import pytest
import torch

from language_model_saes_b200.models.lorsa import LorsaConfig, LowRankSparseAttention


def _lorsa(**kw):
    torch.manual_seed(0)
    base = dict(hook_point_in="blocks.0.ln1.hook_normalized", hook_point_out="blocks.0.hook_attn_out", d_model=16, expansion_factor=1,
                n_qk_heads=4, d_qk_head=8, rotary_dim=8, n_ctx=24, act_fn="relu", norm_activation="inference")  # fmt: skip
    base.update(kw)
    m = LowRankSparseAttention(LorsaConfig(**base))
    m.init_parameters()
    with torch.no_grad():
        m.W_Q.mul_(4)
        m.W_K.mul_(4)
    return m


@pytest.mark.parametrize("adjacent", [True, False])
def test_rotary_tables_and_relative_position_property(adjacent):
    m = _lorsa(rotary_adjacent_pairs=adjacent)
    sin, cos = m.rotary_sin, m.rotary_cos
    assert sin.shape == (24, 8) and torch.allclose(sin.pow(2) + cos.pow(2), torch.ones(24, 8), atol=1e-6)
    freq = 10000 ** (torch.arange(4) / 4)
    want = torch.arange(24.0)[:, None] / (freq.repeat_interleave(2) if adjacent else freq.repeat(2))[None, :]
    assert torch.allclose(sin, want.sin(), atol=1e-5)
    # rotating q at position i and k at position j gives a score that depends on i - j only
    g = torch.Generator().manual_seed(1)
    qv, kv = torch.randn(8, generator=g), torch.randn(8, generator=g)
    q = m._apply_rotary(qv.expand(1, 24, 1, 8))
    k = m._apply_rotary(kv.expand(1, 24, 1, 8))
    scores = torch.einsum("bqhd,bkhd->qk", q, k)
    for shift in (1, 5):
        diag = torch.diagonal(scores, offset=-shift)  # q at i + shift, k at i
        assert torch.allclose(diag, diag[0].expand_as(diag), atol=1e-4)
    assert not torch.allclose(torch.diagonal(scores, -1)[0], torch.diagonal(scores, -5)[0], atol=1e-3)


def test_ntk_by_parts_tables_stretch_only_the_long_wavelengths():
    kw = dict(use_NTK_by_parts_rope=True, NTK_by_parts_factor=8.0, NTK_by_parts_low_freq_factor=1.0, NTK_by_parts_high_freq_factor=4.0,
              old_context_len=64, rotary_base=10000)  # fmt: skip
    plain, ntk = _lorsa(), _lorsa(**kw)
    inv = 1.0 / (10000 ** (torch.arange(0, 8, 2).float() / 8))
    wavelen = 2 * math.pi / inv
    # restated from the published definition: short wavelengths untouched, long ones divided by the factor, a blend between
    scaled = torch.where(wavelen > 64 / 1.0, inv / 8.0, inv)
    smooth = (64 / wavelen - 1.0) / (4.0 - 1.0)
    blended = (1 - smooth) * scaled / 8.0 + smooth * scaled
    medium = ~(wavelen < 64 / 4.0) & ~(wavelen > 64 / 1.0)
    want_inv = torch.where(medium, blended, scaled)
    angles = torch.arange(24.0)[:, None] * want_inv.repeat_interleave(2)[None, :]
    assert torch.allclose(ntk.rotary_sin, angles.sin(), atol=1e-5) and torch.allclose(ntk.rotary_cos, angles.cos(), atol=1e-5)
    short = wavelen < 64 / 4.0
    cols = short.repeat_interleave(2)
    assert cols.any() and not cols.all()
    assert torch.allclose(ntk.rotary_sin[:, cols], plain.rotary_sin[:, cols], atol=1e-6)  # the fastest channels are the plain ones
    assert not torch.allclose(ntk.rotary_sin[:, ~cols], plain.rotary_sin[:, ~cols], atol=1e-3)


@pytest.mark.parametrize("kw", [dict(), dict(positional_embedding_type="none"), dict(use_post_qk_ln=True, normalization_type="RMS"),
                                dict(rotary_dim=4)])  # fmt: skip
def test_fast_attention_path_equals_the_pattern_path_and_z_patterns_sum_to_it(kw):
    m = _lorsa(**kw)
    g = torch.Generator().manual_seed(2)
    x = torch.randn(2, 10, 16, generator=g)
    with torch.no_grad():
        fast = m.compute_hidden_pre(x)  # fused attention, QK heads as attention heads with the OV group as value width
        q, k, v = m._compute_qkv(x)
        pattern = m._compute_attention_pattern(q, k)  # [heads, batch, q, k]
        assert torch.allclose(pattern.sum(-1), torch.ones_like(pattern.sum(-1)), atol=1e-5)
        assert not torch.triu(pattern[0, 0], diagonal=1).any()  # causal
        slow = m._compute_head_outputs(pattern.permute(1, 0, 2, 3), v)
        assert torch.allclose(fast, slow, atol=1e-4)
        z = m.encode_z_patterns(x[:1])  # [F, q, k]: contribution of source k to head f at target q
        assert z.shape == (16, 10, 10) and torch.allclose(z.sum(-1).T, fast[0], atol=1e-4)
        some = torch.tensor([3, 9])
        assert torch.allclose(m.encode_z_pattern_for_head(x[:1], some), z[some], atol=1e-6)
    assert m.cfg.ov_group_size == 4 and m.cfg.n_ov_heads == 16


def test_checkpoint_with_fewer_qk_heads_is_expanded_by_repeating_them():
    small = _lorsa(n_qk_heads=2)
    big = _lorsa(n_qk_heads=4)
    sd = small.full_state_dict()
    big.load_full_state_dict(sd)
    assert big.W_Q.shape[0] == 4
    for h in range(4):
        assert torch.equal(big.W_Q[h], small.W_Q[h // 2]) and torch.equal(big.b_K[h], small.b_K[h // 2])
    assert torch.equal(big.W_V, small.W_V) and torch.equal(big.W_O, small.W_O)
    g = torch.Generator().manual_seed(3)
    x = torch.randn(1, 6, 16, generator=g)
    with torch.no_grad():  # each pair of new heads attends like the head it came from: the same function
        assert torch.allclose(big.compute_hidden_pre(x), small.compute_hidden_pre(x), atol=1e-5)
