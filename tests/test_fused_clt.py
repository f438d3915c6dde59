"""The fused cross-layer transcoder step (``ops.fused_clt.FusedCLTStep``) against the generic autograd path of the same
model: losses and parameters after a few Adam steps (CPU: plain-torch statements of the kernels; GPU: the kernels)."""

import copy

import pytest
import torch

from language_model_saes_b200.models.clt import CLTConfig, CrossLayerTranscoder
from language_model_saes_b200.ops.fused_clt import FusedCLTStep

DEVICES = [pytest.param("cuda", marks=pytest.mark.gpu), "cpu"]


def _model(dev, L=3, d=64, F=256, k=8, gate=True):
    torch.manual_seed(0)
    ins, outs = [f"blocks.{i}.ln2.hook_normalized" for i in range(L)], [f"blocks.{i}.hook_mlp_out" for i in range(L)]
    cfg = CLTConfig(hook_points_in=ins, hook_points_out=outs, d_model=d, expansion_factor=F / d, act_fn="topk", top_k=k, device=dev,
                    dtype=torch.float32, norm_activation="inference", sparsity_include_decoder_norm=gate)  # fmt: skip
    m = CrossLayerTranscoder(cfg)
    m.init_parameters(encoder_uniform_bound=0.1, decoder_uniform_bound=0.1)
    with torch.no_grad():
        m.W_E.mul_(4.0)
        m.b_E.add_(0.02 * torch.randn_like(m.b_E))
    return m


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("gate", [True, False])
def test_fused_clt_step_matches_autograd(dev, gate):
    L, d, F, k, B, lr, steps = 3, 64, 256, 8, 128, 1e-3, 4
    ref = _model(dev, L, d, F, k, gate)
    start = {n: p.detach().clone() for n, p in ref.named_parameters()}
    fused_model = copy.deepcopy(ref)
    assert FusedCLTStep.supports(fused_model)[0]
    engine = FusedCLTStep(fused_model)
    g = torch.Generator(device=dev).manual_seed(1)
    basis = torch.randn(6, d, device=dev, generator=g)
    opt = torch.optim.Adam(ref.parameters(), lr=lr)
    tokens = torch.zeros(B, dtype=torch.long, device=dev)
    ref_losses, fused_losses = [], []
    for _ in range(steps):
        z = torch.randn(B, 6, device=dev, generator=g)
        x = torch.stack([z @ basis * (1 + 0.1 * l) + 0.2 * torch.randn(B, d, device=dev, generator=g) for l in range(L)], dim=1)
        y = torch.stack([(z @ basis).roll(l + 1, dims=-1) + 0.2 * torch.randn(B, d, device=dev, generator=g) for l in range(L)], dim=0)
        x, y = x.to(torch.bfloat16), y.to(torch.bfloat16)
        batch = {h: x[:, l].float() for l, h in enumerate(ref.cfg.hook_points_in)} | {h: y[l].float() for l, h in enumerate(ref.cfg.hook_points_out)}
        batch["tokens"] = tokens
        opt.zero_grad()
        with torch.autocast(dev, dtype=torch.bfloat16, enabled=dev == "cuda"):
            out = ref.compute_loss(batch, return_aux_data=True)
        out["loss"].backward()
        opt.step()
        ref_losses.append(float(out["loss"].detach()))
        fused_losses.append(float(engine.step(x, y, k, lr)))
    r, f = torch.tensor(ref_losses), torch.tensor(fused_losses)
    assert torch.allclose(r, f, rtol=3e-2 if dev == "cuda" else 2e-3), (ref_losses, fused_losses)
    for name, p in ref.named_parameters():
        a, b = p.detach().float(), dict(fused_model.named_parameters())[name].detach().float()
        moved = (a - start[name].float()).abs().mean()
        assert float((a - b).abs().mean()) < (0.25 if dev == "cuda" else 0.05) * float(moved) + 1e-7, name
    # the engine's running per-feature norms agree with the model's definition
    want = fused_model.decoder_norm_per_feature().reshape(-1)
    assert torch.allclose(engine.norm_sq.sqrt(), want, rtol=1e-3, atol=1e-5)
