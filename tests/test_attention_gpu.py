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
