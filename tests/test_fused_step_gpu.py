"""The fused kernel training step against the same step written with autograd + torch.optim.Adam."""

import copy

import pytest
import torch

from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
from language_model_saes_b200.ops import sae_kernels as K
from language_model_saes_b200.ops.fused_step import FusedTopKSAEStep

pytestmark = pytest.mark.gpu


def _model(d=256, expansion=8, k=16, gate=True, bias=True):
    torch.manual_seed(0)
    cfg = SAEConfig(hook_point_in="h", hook_point_out="h", d_model=d, expansion_factor=expansion, act_fn="topk", top_k=k,
                    sparsity_include_decoder_norm=gate, use_decoder_bias=bias, device="cuda", dtype=torch.float32)  # fmt: skip
    sae = SparseAutoEncoder(cfg)
    sae.init_parameters(encoder_uniform_bound=0.06, decoder_uniform_bound=0.06)
    sae.set_decoder_to_fixed_norm(0.7, True)
    sae.init_encoder_with_decoder_transpose()
    sae.set_dataset_average_activation_norm({"h": d**0.5})
    return sae


def _data(n, B, d, rank=32):
    g = torch.Generator(device="cuda").manual_seed(1)
    A = torch.randn(rank, d, device="cuda", generator=g)
    out = []
    for _ in range(n):
        x = torch.randn(B, rank, device="cuda", generator=g) @ A + 0.1 * torch.randn(B, d, device="cuda", generator=g)
        x = x * (d**0.5 / x.norm(dim=-1).mean())
        out.append(x.to(torch.bfloat16))
    return out


@pytest.mark.parametrize("chunks", [1, 3])
@pytest.mark.parametrize("gate,bias,k", [(True, True, 16), (False, False, 8), (True, True, 50), (True, True, 100)])
def test_fused_matches_autograd(gate, bias, k, chunks):
    # chunks > 1: the update runs per feature chunk on its own stream and the next step's encoder GEMM follows it
    # chunk by chunk; results must not depend on it
    d, B, steps, lr = 256, 512, 12, 1e-3
    ref = _model(d=d, k=k, gate=gate, bias=bias)
    fused_model = copy.deepcopy(ref)
    engine = FusedTopKSAEStep(fused_model, overlap_chunks=chunks)
    assert len(engine.chunks) == chunks
    data = _data(steps, B, d)
    opt = torch.optim.Adam(ref.parameters(), lr=lr)
    ref_losses, fused_losses = [], []
    tokens = torch.zeros(B, dtype=torch.long, device="cuda")
    for x in data:
        opt.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = ref.compute_loss({"h": x.float(), "tokens": tokens})["loss"]
        loss.backward()
        opt.step()
        ref_losses.append(float(loss.detach()))
        fused_losses.append(float(engine.step(x, x, k, lr)))
    engine.join()
    K.check_status(torch.device("cuda"))
    r, f = torch.tensor(ref_losses), torch.tensor(fused_losses)
    assert torch.allclose(r, f, rtol=3e-2), (ref_losses, fused_losses)
    assert f[-1] < f[0]
    # parameters moved the same way
    for name in ("W_D", "W_E", "b_E") + (("b_D",) if bias else ()):
        a, b = getattr(ref, name).detach().float(), getattr(fused_model, name).detach().float()
        cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0)
        # biases take Adam steps of size ~lr whose sign flips on near-zero gradients and they start at zero, so their direction is noisy: looser bound
        assert cos > (0.9 if name.startswith("b_") else 0.999), (name, float(cos))


def test_fused_clipping_matches_generic_clip():
    from language_model_saes_b200.optim import clip_grad_norm

    d, B, k, lr = 256, 512, 16, 1e-3
    ref = _model(d=d, k=k)
    fused_model = copy.deepcopy(ref)
    unclipped = FusedTopKSAEStep(copy.deepcopy(ref))
    engine = FusedTopKSAEStep(fused_model)
    (x,) = _data(1, B, d)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss = ref.compute_loss({"h": x.float(), "tokens": torch.zeros(B, dtype=torch.long, device="cuda")})["loss"]
    loss.backward()
    params = [p for p in ref.parameters() if p.grad is not None]
    want = clip_grad_norm(params, float("inf"))  # the trainer's norm on the generic path: |g|_2 / sqrt(non-zero entries)
    unclipped.step(x, x, k, lr, clip_grad_norm=1e9)  # a bound far above the norm: measured, nothing scaled
    norm = unclipped.last_grad_norm
    assert torch.allclose(norm, want, rtol=3e-2), (norm, want)
    max_norm = 0.25 * float(norm)
    engine.step(x, x, k, lr, clip_grad_norm=max_norm)
    K.check_status(torch.device("cuda"))
    assert torch.allclose(engine.last_grad_norm, norm, rtol=1e-4)
    # first Adam moments = 0.1 x gradient: the clipped ones are the unclipped ones times max_norm / (norm + 1e-6)
    mom = lambda e: torch.sqrt(sum(st[0].square().sum() for st in e.state.values() if st is not None))  # noqa: E731
    assert torch.allclose(mom(engine), mom(unclipped) * max_norm / (norm + 1e-6), rtol=1e-3)
    cos = torch.nn.functional.cosine_similarity(engine.state["W_D"][0].flatten(), ref.W_D.grad.flatten(), dim=0)
    assert cos > 0.99, float(cos)


def test_fused_row_mask_and_transcoder_label():
    d, B, k = 128, 256, 8
    sae = _model(d=d, k=k)
    engine = FusedTopKSAEStep(sae)
    x, y = _data(2, B, d)
    w = (torch.rand(B, device="cuda") > 0.3).float()
    idx, act = engine.encode(x, k)
    xhat = K.ref_sparse_decode(idx, act, engine.WD_bf16, engine.bD)
    want = (((xhat - y.float()) ** 2).sum(-1) * w).sum() / w.sum()
    got = engine.step(x, y, k, 1e-3, row_weight=w, n_tokens_global=int(w.sum()))
    assert torch.allclose(got, want, rtol=1e-3)


@pytest.mark.parametrize("k_aux", [16, 96])
def test_fused_auxk_matches_autograd(k_aux):
    """Aux-K on the fused path against the autograd path: same dead set, same losses, same parameter motion."""
    from language_model_saes_b200.ops.fused_step import AuxK

    d, B, k, steps, lr, alpha, thr = 256, 512, 16, 6, 1e-3, 1 / 32, 1000
    ref = _model(d=d, k=k)
    F = ref.cfg.d_sae
    with torch.no_grad():
        ref.b_E[: F // 4] -= 0.5  # a quarter of the dictionary rarely fires: it goes dead after two batches
    fused_model = copy.deepcopy(ref)
    engine = FusedTopKSAEStep(fused_model)
    aux = AuxK(F, k_aux, alpha, thr, "cuda")
    counter = torch.zeros(F, dtype=torch.long, device="cuda")

    def update_dead(feature_acts, mask, specs):
        nonlocal counter
        fired = (feature_acts > 0).any(dim=0)
        counter = torch.where(fired, torch.zeros_like(counter), counter + feature_acts.shape[0])
        return counter >= thr

    opt = torch.optim.Adam(ref.parameters(), lr=lr)
    tokens = torch.zeros(B, dtype=torch.long, device="cuda")
    ref_l, ref_a, fus_l, fus_a, n_dead = [], [], [], [], []
    for x in _data(steps, B, d):
        opt.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = ref.compute_loss({"h": x.float(), "tokens": tokens}, auxk_coefficient=alpha, k_aux=k_aux,
                                   update_dead_statistics=update_dead, return_aux_data=True)  # fmt: skip
        out["loss"].backward()
        opt.step()
        ref_l.append(float(out["loss"].detach()))
        ref_a.append(float(out["l_aux"].detach().mean()))
        fus_l.append(float(engine.step(x, x, k, lr, aux=aux)))
        fus_a.append(float(engine.last_aux_loss))
        n_dead.append(int(aux.is_dead.sum()))
        # the two paths round differently (bf16 kernels vs autocast), so a feature on the edge of firing may differ
        assert (aux.is_dead != (counter >= thr)).float().mean() < 0.02
    K.check_status(torch.device("cuda"))
    assert n_dead[-1] > 0 and max(fus_a) > 0, (n_dead, fus_a)
    assert torch.allclose(torch.tensor(ref_l), torch.tensor(fus_l), rtol=3e-2), (ref_l, fus_l)
    assert torch.allclose(torch.tensor(ref_a), torch.tensor(fus_a), rtol=6e-2, atol=1e-3), (ref_a, fus_a)
    for name in ("W_D", "W_E"):
        a, b = getattr(ref, name).detach().float(), getattr(fused_model, name).detach().float()
        assert torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0) > 0.999
    # the dead features moved (only the auxiliary loss reaches them) and moved the same way
    dead = aux.is_dead & (counter >= thr)
    moved_ref = (ref.W_D.detach()[dead] - _model(d=d, k=k).W_D.detach()[dead]).flatten()
    moved_fus = (fused_model.W_D.detach()[dead] - _model(d=d, k=k).W_D.detach()[dead]).flatten()
    assert moved_fus.abs().sum() > 0
    assert torch.nn.functional.cosine_similarity(moved_ref, moved_fus, dim=0) > 0.9


@pytest.mark.parametrize("gate,k", [(True, 16), (False, 8)])
def test_fused_batchtopk_matches_autograd(gate, k):
    """Batch-level top-k on the fused path (radix-select threshold + threshold compaction) against the generic model."""
    d, B, steps, lr = 256, 512, 10, 1e-3
    ref = _model(d=d, k=k, gate=gate)
    ref.cfg.act_fn = "batchtopk"
    ref.activation_function = ref.activation_function_factory(None)
    fused_model = copy.deepcopy(ref)
    fused_model.activation_function = fused_model.activation_function_factory(None)
    assert FusedTopKSAEStep.supports(fused_model)[0]
    engine = FusedTopKSAEStep(fused_model)
    assert engine.batch_level
    engine.batch_list_factor = 32  # tiny shapes: a token can hold many times the average number of codes
    data = _data(steps, B, d)
    idx, act = engine.encode(data[0], k)
    n_codes = int((idx >= 0).sum())
    assert n_codes == k * B, n_codes  # exactly k codes per token on average (ties at the bf16 threshold are rationed)
    assert int((idx >= 0).sum(-1).max()) > k  # ... but not k per token
    opt = torch.optim.Adam(ref.parameters(), lr=lr)
    ref_losses, fused_losses = [], []
    tokens = torch.zeros(B, dtype=torch.long, device="cuda")
    for x in data:
        opt.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = ref.compute_loss({"h": x.float(), "tokens": tokens})["loss"]
        loss.backward()
        opt.step()
        ref_losses.append(float(loss.detach()))
        fused_losses.append(float(engine.step(x, x, k, lr)))
    K.check_status(torch.device("cuda"))
    r, f = torch.tensor(ref_losses), torch.tensor(fused_losses)
    assert torch.allclose(r, f, rtol=3e-2), (ref_losses, fused_losses)
    for name in ("W_D", "W_E"):
        a, b = getattr(ref, name).detach().float(), getattr(fused_model, name).detach().float()
        assert torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0) > 0.999, name
