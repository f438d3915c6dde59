"""Cross-layer transcoder decoder fan-out: the sparse path (torch oracle on CPU, sm_100a kernels on a GPU) against the
dense per-target-layer products, values and gradients."""

import pytest
import torch

from language_model_saes_b200.models.clt import CLTConfig, CrossLayerTranscoder
from language_model_saes_b200.ops import clt_kernels as CK


def _codes(B, L, F, k, device, seed=0):
    g = torch.Generator().manual_seed(seed)
    acts = torch.zeros(B, L * F)
    for b in range(B):
        cols = torch.randperm(L * F, generator=g)[:k]
        acts[b, cols] = torch.rand(k, generator=g) + 0.1
    return acts.view(B, L, F).to(device)


def _dense(acts, weights, bias):
    outs = []
    for t, w in enumerate(weights):
        y = torch.einsum("blf,lfd->bd", acts[:, : t + 1].float(), w.float())
        outs.append(y + (bias[t].float() if bias is not None else 0))
    return torch.stack(outs)


def _weights(L, F, d, device, dtype, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [(torch.randn(t + 1, F, d, generator=g) / d**0.5).to(device=device, dtype=dtype) for t in range(L)]


def test_oracles_match_dense_products_cpu():
    B, L, F, d, k = 5, 3, 16, 8, 6
    acts = _codes(B, L, F, k, "cpu")
    weights = [w.requires_grad_() for w in _weights(L, F, d, "cpu", torch.float32)]
    bias = torch.randn(L, d, requires_grad=True)
    a1 = acts.clone().requires_grad_()
    got = CK.clt_sparse_decode(a1, weights, bias)
    dy = torch.randn_like(got)
    got.backward(dy)
    g_sparse = [w.grad.clone() for w in weights], a1.grad.clone(), bias.grad.clone()
    for w in weights:
        w.grad = None
    bias.grad = None
    a2 = acts.clone().requires_grad_()
    want = _dense(a2, weights, bias)
    want.backward(dy)
    assert torch.allclose(got, want, atol=2e-2, rtol=2e-2)  # the sparse path rounds its operands to bf16
    nz = acts != 0
    assert torch.allclose(g_sparse[1][nz], a2.grad[nz], atol=3e-2, rtol=3e-2)
    assert torch.equal(g_sparse[1][~nz], torch.zeros_like(g_sparse[1][~nz]))  # only the active codes get a gradient
    for gs, w in zip(g_sparse[0], weights):
        assert torch.allclose(gs, w.grad, atol=3e-2, rtol=3e-2)
    assert torch.allclose(g_sparse[2], bias.grad, atol=1e-5)


def test_clt_model_decode_uses_fan_out_when_sparse_cpu():
    cfg = CLTConfig(hook_points_in=[f"in{i}" for i in range(3)], hook_points_out=[f"out{i}" for i in range(3)], d_model=8,
                    expansion_factor=4, act_fn="topk", top_k=2, device="cpu", dtype=torch.float32, norm_activation="inference",
                    decode_with_csr=True, sparsity_threshold_for_csr=0.5)  # fmt: skip
    clt = CrossLayerTranscoder(cfg)
    clt.init_parameters()
    x = torch.randn(4, 3, 8)
    acts = clt.encode(x)
    sparse = clt.decode(acts)
    clt.cfg.decode_with_csr = False
    dense = clt.decode(acts)
    assert sparse.shape == dense.shape == (3, 4, 8)
    assert torch.allclose(sparse, dense, atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("B,L,F,d,k", [(64, 4, 512, 768, 24), (33, 6, 1000, 1024, 40), (16, 2, 256, 4096, 8), (8, 3, 128, 8192, 5)])
def test_fan_out_kernels_match_oracles(B, L, F, d, k):
    dev = "cuda"
    acts = _codes(B, L, F, k, dev)
    w16 = _weights(L, F, d, dev, torch.bfloat16)
    bias = torch.randn(L, d, device=dev)
    idx, val = CK.dense_to_padded_sparse(acts.reshape(B, L * F))
    y = CK.clt_decode(idx, val, w16, bias)
    want = CK.ref_clt_decode(idx, val, w16, bias)
    assert torch.allclose(y, want, atol=1e-3, rtol=1e-3)
    assert torch.allclose(y, _dense(acts, w16, bias), atol=1e-3, rtol=1e-3)
    y16 = CK.clt_decode(idx, val, w16, bias, torch.bfloat16)
    assert torch.allclose(y16.float(), want, atol=3e-2, rtol=3e-2)
    dy = torch.randn(L, B, d, device=dev).to(torch.bfloat16)
    assert torch.allclose(CK.clt_dact(idx, w16, dy), CK.ref_clt_dact(idx, w16, dy), atol=2e-3, rtol=2e-3)
    got = CK.clt_wgrad(idx, val, dy, L, F)
    for g, r in zip(got, CK.ref_clt_wgrad(idx, val, dy, L, F)):
        assert torch.allclose(g, r, atol=2e-3, rtol=2e-3)


@pytest.mark.gpu
def test_fan_out_autograd_matches_dense_on_gpu():
    B, L, F, d, k = 48, 3, 256, 512, 12
    dev = "cuda"
    acts = _codes(B, L, F, k, dev)
    weights = [w.requires_grad_() for w in _weights(L, F, d, dev, torch.float32)]
    bias = torch.randn(L, d, device=dev, requires_grad=True)
    a1 = acts.clone().requires_grad_()
    got = CK.clt_sparse_decode(a1, weights, bias)
    dy = torch.randn_like(got)
    got.backward(dy)
    gw = [w.grad.clone() for w in weights]
    for w in weights:
        w.grad = None
    a2 = acts.clone().requires_grad_()
    want = _dense(a2, weights, None) + bias.detach()[:, None]
    want.backward(dy)
    assert torch.allclose(got, want, atol=3e-2, rtol=3e-2)
    nz = acts != 0
    assert torch.allclose(a1.grad[nz], a2.grad[nz], atol=5e-2, rtol=5e-2)
    for g, w in zip(gw, weights):
        assert torch.allclose(g, w.grad, atol=5e-2, rtol=5e-2)
