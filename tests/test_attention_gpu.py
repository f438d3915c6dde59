"""tcgen05 causal attention with d_v != d_qk against the fp32 torch oracle."""

import pytest
import torch

from language_model_saes_b200.ops import attention as A
from language_model_saes_b200.ops import sae_kernels as K

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("b,s,h,dqk,dv", [(2, 256, 3, 64, 128), (1, 384, 2, 128, 64), (2, 200, 2, 64, 256), (1, 1024, 4, 64, 128),
                                          (3, 128, 1, 128, 128), (1, 72, 2, 64, 64)])  # fmt: skip
def test_forward_matches_oracle(b, s, h, dqk, dv):
    torch.manual_seed(0)
    dev = torch.device("cuda")
    q = torch.randn(b, s, h, dqk, device=dev).to(torch.bfloat16)
    k = torch.randn(b, s, h, dqk, device=dev).to(torch.bfloat16)
    v = torch.randn(b, s, h, dv, device=dev).to(torch.bfloat16)
    scale = 1.7 / dqk**0.5
    out, lse = A.causal_attention_fwd(q, k, v, scale, want_lse=True)
    K.check_status(dev)
    want, want_lse = A.ref_causal_attention(q, k, v, scale)
    assert out.shape == want.shape and out.dtype == torch.bfloat16
    assert torch.allclose(lse, want_lse, atol=2e-3, rtol=1e-3), float((lse - want_lse).abs().max())
    assert torch.allclose(out.float(), want, atol=2e-2, rtol=2e-2), float((out.float() - want).abs().max())


@pytest.mark.parametrize("b,s,h,dqk,dv", [(2, 256, 2, 64, 128), (1, 384, 2, 128, 64), (1, 200, 2, 64, 256), (1, 512, 3, 64, 64),
                                          (2, 128, 1, 128, 128), (1, 72, 1, 64, 192)])  # fmt: skip
def test_backward_matches_autograd_of_the_oracle(b, s, h, dqk, dv):
    torch.manual_seed(1)
    dev = torch.device("cuda")
    q, k = (torch.randn(b, s, h, dqk, device=dev).to(torch.bfloat16).float().requires_grad_() for _ in range(2))
    v = torch.randn(b, s, h, dv, device=dev).to(torch.bfloat16).float().requires_grad_()
    scale = 1.3 / dqk**0.5
    dout = torch.randn(b, s, h, dv, device=dev).to(torch.bfloat16).float()
    out = A.causal_attention(q, k, v, scale)
    out.backward(dout)
    K.check_status(dev)
    got = [t.grad.clone() for t in (q, k, v)]
    for t in (q, k, v):
        t.grad = None
    want_out, _ = A.ref_causal_attention(q, k, v, scale)
    want_out.backward(dout)
    assert torch.allclose(out, want_out, atol=2e-2, rtol=2e-2)
    for name, g, t in zip("qkv", got, (q, k, v)):
        rel = float((g - t.grad).norm() / t.grad.norm())
        assert rel < 2e-2, (name, rel)
        assert torch.allclose(g, t.grad, atol=0.05 * float(t.grad.abs().max()), rtol=0.05), name


def test_lorsa_encode_uses_the_tensor_core_attention_and_matches_the_score_path():
    from language_model_saes_b200.models.lorsa import LorsaConfig, LowRankSparseAttention

    torch.manual_seed(0)
    cfg = LorsaConfig(hook_point_in="in", hook_point_out="out", d_model=128, expansion_factor=4, n_qk_heads=4, d_qk_head=64,
                      n_ctx=64, act_fn="relu", device="cuda", dtype=torch.bfloat16, norm_activation="inference",
                      positional_embedding_type="rotary", rotary_dim=64, attention_kernel="tensor_core")  # fmt: skip
    m = LowRankSparseAttention(cfg)
    m.init_parameters(encoder_uniform_bound=0.2, decoder_uniform_bound=0.2, init_log_jumprelu_threshold_value=0.0)
    x = torch.randn(2, 64, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    before = K.kernel_launch_count()
    fast, hidden_fast = m.encode(x, return_hidden_pre=True)
    assert K.kernel_launch_count() > before  # the tcgen05 forward ran (OV group 128, d_qk 64)
    slow, hidden_slow, _ = m.encode(x, return_hidden_pre=True, return_attention_pattern=True)
    K.check_status(torch.device("cuda"))
    assert torch.allclose(hidden_fast.float(), hidden_slow.float(), atol=3e-2, rtol=3e-2)
    hidden_fast.float().pow(2).sum().backward()
    g_fast = x.grad.clone()
    x.grad = None
    hidden_slow.float().pow(2).sum().backward()
    rel = float((g_fast.float() - x.grad.float()).norm() / x.grad.float().norm())
    assert rel < 5e-2, rel
