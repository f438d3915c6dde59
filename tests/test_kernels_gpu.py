"""Numerics of every sm_100a kernel against its plain PyTorch fp32 definition (ops/sae_kernels.py ref_*)."""

import pytest
import torch

from language_model_saes_b200.ops import sae_kernels as K

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _mk(M, N, Kd, seed=0, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = (torch.randn(M, Kd, generator=g) * scale).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, Kd, generator=g) / Kd**0.5).to(torch.bfloat16).to(DEV)
    b = (torch.randn(N, generator=g) * 0.1).to(DEV)
    gate = (torch.rand(N, generator=g) + 0.5).to(DEV)
    return x, w, b, gate


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("M,N,Kd", [(128, 256, 64), (256, 512, 128), (300, 1032, 200), (4096, 4096, 512), (77, 264, 72), (512, 1288, 328)])
def test_encoder_hidden(M, N, Kd, pair):
    # pair=True runs the CTA-pair (cta_group::2) kernel when M fills whole pairs of 128-row panels (256, 4096, 512
    # here; M = 300 has three panels and exercises the fall-back to the single-CTA kernel)
    x, w, b, _ = _mk(M, N, Kd)
    H = K.encoder_hidden(x, w, b, pair=pair)
    K.check_status(x.device)
    ref = K.ref_hidden(x, w, b)
    err = (H.float() - ref).abs().max().item()
    tol = 2e-2 * max(1.0, ref.abs().max().item())
    assert err < tol, (err, tol)


def _codes_to_dense(idx, val, N):
    out = torch.zeros(idx.shape[0], N, device=idx.device)
    m = idx >= 0
    rows = torch.arange(idx.shape[0], device=idx.device).unsqueeze(1).expand_as(idx)
    out[rows[m], idx[m].long()] = val[m]
    return out


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("M,N,Kd,k", [(128, 512, 64, 8), (256, 2048, 128, 32), (300, 4104, 256, 50), (1024, 8192, 256, 64), (64, 264, 64, 1),
                                      (512, 4104, 264, 50)])
@pytest.mark.parametrize("use_gate", [False, True])
def test_encoder_topk_fused(M, N, Kd, k, use_gate, pair):
    x, w, b, gate = _mk(M, N, Kd, seed=1)
    gate = gate if use_gate else None
    idx, act = K.encoder_topk(x, w, b, gate, k, pair=pair)
    K.check_status(x.device)
    h = K.ref_hidden(x, w, b)
    g = h * gate if use_gate else h
    g = torch.where(g > 0, g, torch.zeros_like(g))
    kth = torch.topk(g, k, dim=-1).values[:, -1:]
    # every selected entry must be >= the exact k-th largest (up to fp32 accumulation-order noise) and the
    # selected activation must equal the reference pre-activation
    dense = _codes_to_dense(idx, act, N)
    sel = dense != 0
    assert ((sel.sum(-1) == (g > 0).sum(-1).clamp(max=k))).all()
    gsel = torch.where(sel, g, torch.full_like(g, float("inf")))
    assert (gsel.min(-1).values >= kth.squeeze(-1) - 1e-3).all()
    assert torch.allclose(dense[sel], h[sel], atol=2e-3, rtol=2e-3)
    # no duplicates
    srt = torch.sort(torch.where(idx >= 0, idx, torch.arange(-k, 0, device=DEV).expand_as(idx)), dim=-1).values
    assert (srt[:, 1:] != srt[:, :-1]).all()


@pytest.mark.parametrize("M,N,pair", [(1024, 8192, True), (768, 8192, True), (640, 8192, False)])
def test_encoder_gemm_with_a_ragged_deal_of_column_ranges(M, N, pair, monkeypatch):
    """``LMSAE_GEMM_RAGGED=1``: panel units get unequal numbers of column ranges so that every SM (pair) has work; the
    unused candidate lists of the panels with fewer ranges are marked empty. Same codes and pre-activations as the
    plain product."""
    monkeypatch.setenv("LMSAE_GEMM_RAGGED", "1")
    units, splits = K.choose_units(M, N, pair)
    assert units > 0 and units % ((M // 128) // (2 if pair else 1)) != 0  # the deal really is ragged for these shapes
    x, w, b, gate = _mk(M, N, 128, seed=4)
    k = 24
    idx, act = K.encoder_topk(x, w, b, gate, k, pair=pair)
    H = K.encoder_hidden(x, w, b, pair=pair)
    K.check_status(x.device)
    h = K.ref_hidden(x, w, b)
    assert (H.float() - h).abs().max().item() < 2e-2 * max(1.0, h.abs().max().item())
    g = torch.where(h * gate > 0, h * gate, torch.zeros_like(h))
    kth = torch.topk(g, k, dim=-1).values[:, -1:]
    dense = _codes_to_dense(idx, act, N)
    sel = dense != 0
    assert (sel.sum(-1) == (g > 0).sum(-1).clamp(max=k)).all()
    gsel = torch.where(sel, g, torch.full_like(g, float("inf")))
    assert (gsel.min(-1).values >= kth.squeeze(-1) - 1e-3).all()
    assert torch.allclose(dense[sel], h[sel], atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("k", [16, 100, 512])
def test_row_topk(k):
    M, N = 64, 4096
    g = torch.Generator().manual_seed(3)
    H = torch.randn(M, N, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.rand(N, generator=g) + 0.5).to(DEV)
    alive = (torch.rand(N, generator=g) > 0.3).to(DEV)
    idx, val = K.row_topk(H, k, gate, alive)
    ridx, rval = K.ref_topk_codes(H.float(), k, gate, alive)
    d1 = _codes_to_dense(idx, val, N)
    d2 = _codes_to_dense(ridx, rval, N)
    # ties in bf16 inputs can swap equal values; compare the multiset of selected values
    assert torch.allclose(torch.sort(d1, dim=-1).values, torch.sort(d2, dim=-1).values, atol=1e-5)


def _codes(B, k, F, seed=5):
    g = torch.Generator().manual_seed(seed)
    idx = torch.stack([torch.randperm(F, generator=g)[:k] for _ in range(B)]).to(torch.int32)
    idx[0, -1] = -1
    val = torch.rand(B, k, generator=g) + 0.1
    val[0, -1] = 0
    return idx.to(DEV), val.to(DEV)


@pytest.mark.parametrize("B,k,F,d", [(33, 7, 300, 64), (128, 50, 2048, 4096), (16, 64, 512, 776)])
def test_sparse_decode_and_loss(B, k, F, d):
    idx, val = _codes(B, k, F)
    g = torch.Generator().manual_seed(7)
    W = (torch.randn(F, d, generator=g) / d**0.5).to(torch.bfloat16).to(DEV)
    bias = torch.randn(d, generator=g).to(DEV) * 0.1
    label = torch.randn(B, d, generator=g).to(torch.bfloat16).to(DEV)
    rw = (torch.rand(B, generator=g) > 0.2).float().to(DEV)
    out = K.sparse_decode(idx, val, W, bias)
    ref = K.ref_sparse_decode(idx, val, W, bias)
    assert torch.allclose(out, ref, atol=1e-4, rtol=1e-4)
    out16 = K.sparse_decode(idx, val, W, bias, torch.bfloat16)
    assert torch.allclose(out16.float(), ref, atol=2e-2, rtol=2e-2)

    loss = torch.zeros(1, device=DEV)
    row_loss = torch.empty(B, device=DEV)
    gs = 2.0 / B
    dx, dval, xh = K.sparse_decode_loss(idx, val, W, bias, label, rw, gs, loss, True, True, row_loss)
    rxh, rdx, rls, rrl, rdv = K.ref_decode_loss(idx, val, W, bias, label, rw, gs)
    assert torch.allclose(xh, rxh, atol=1e-4, rtol=1e-4)
    assert torch.allclose(dx.float(), rdx.float(), atol=1e-3, rtol=2e-2)
    assert torch.allclose(loss[0], rls, rtol=1e-4)
    assert torch.allclose(row_loss, rrl, rtol=1e-4, atol=1e-4)
    assert torch.allclose(dval, rdv, atol=2e-3, rtol=2e-2)
    dv2 = K.sparse_dact(idx, W, dx)
    assert torch.allclose(dv2, dval, atol=1e-4, rtol=1e-3)

    # dense-row loss kernel (feature-sharded path)
    loss2 = torch.zeros(1, device=DEV)
    dx2 = K.mse_loss_grad(K.sparse_decode(idx, val, W, None), label, bias, rw, gs, loss2)
    assert torch.allclose(dx2.float(), rdx.float(), atol=1e-3, rtol=2e-2)
    assert torch.allclose(loss2[0], rls, rtol=1e-4)


@pytest.mark.parametrize("d", [256, 768, 1536])  # warp-per-row kernel (short rows) and CTA-per-row kernel
@pytest.mark.parametrize("side", ["decoder", "encoder"])
def test_one_sided_sparse_grad_adam_matches_the_plain_statement(d, side):
    """One-sided launches (decoder side with a norm penalty's self-scale and accumulated squared norms, encoder side with
    the bias) against the wrapper's plain-torch path on CPU copies of the same tensors, twice in a row."""
    B, k, F = 300, 6, 700
    idx, act = _codes(B, k, F, seed=5)
    g = torch.Generator().manual_seed(7)
    dact = torch.randn(B, k, generator=g)
    dact[idx.cpu() < 0] = 0
    rows = (torch.randn(B, d, generator=g) * 0.1).to(torch.bfloat16)
    W, m, v = torch.randn(F, d, generator=g), torch.rand(F, d, generator=g) * 0.01, torch.rand(F, d, generator=g) * 0.01
    b, mb, vb = torch.randn(F, generator=g), torch.rand(F, generator=g) * 0.01, torch.rand(F, generator=g) * 0.01
    scale = torch.rand(F, generator=g) * 0.1
    cpu = dict(idx=idx.cpu(), act=act.cpu(), dact=dact, rows=rows, W=W, m=m, v=v, W16=W.to(torch.bfloat16), b=b, mb=mb, vb=vb,
               scale=scale, acc=torch.zeros(F))  # fmt: skip
    gpu = {n_: t.clone().to(DEV) for n_, t in cpu.items()}

    def run(t, step):
        groups = K.FeatureGroups(F, B * k, t["idx"].device).build(t["idx"])
        if side == "decoder":
            K.sparse_grad_adam(groups, t["act"], t["dact"], t["rows"], t["rows"], t["W"], t["m"], t["v"], t["W16"], None, None, None, None,
                               None, None, None, None, None, None, 1e-3, 0.9, 0.999, 1e-8, step, True, wd_self_scale=t["scale"],
                               norm_sq_accum=t["acc"])  # fmt: skip
        else:
            K.sparse_grad_adam(groups, t["act"], t["dact"], t["rows"], t["rows"], None, None, None, None, t["W"], t["m"], t["v"], t["W16"],
                               t["b"], t["mb"], t["vb"], None, None, None, 1e-3, 0.9, 0.999, 1e-8, step, True)  # fmt: skip

    for step in (1, 2):
        run(cpu, step)
        run(gpu, step)
        K.check_status(torch.device(DEV))
    for n_ in ("W", "m", "v", "b", "mb", "vb", "acc"):
        assert torch.allclose(gpu[n_].cpu(), cpu[n_], atol=2e-5, rtol=2e-4), (n_, float((gpu[n_].cpu() - cpu[n_]).abs().max()))
    assert torch.allclose(gpu["W16"].float().cpu(), cpu["W"], atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("B,k,F,d", [(64, 8, 256, 128), (300, 20, 1500, 768), (512, 50, 4096, 1024), (100, 3, 1000, 4096)])
def test_sparse_grad_adam(B, k, F, d):
    idx, act = _codes(B, k, F, seed=11)
    g = torch.Generator().manual_seed(13)
    dact = torch.randn(B, k, generator=g).to(DEV)
    dact[idx < 0] = 0
    x = torch.randn(B, d, generator=g).to(torch.bfloat16).to(DEV)
    dxhat = (torch.randn(B, d, generator=g) * 0.01).to(torch.bfloat16).to(DEV)
    WD = torch.randn(F, d, generator=g).to(DEV)
    WE = torch.randn(F, d, generator=g).to(DEV)
    bE = torch.randn(F, generator=g).to(DEV)
    st = [torch.rand(F, d, generator=g).to(DEV) * 0.01 for _ in range(4)]
    sb = [torch.rand(F, generator=g).to(DEV) * 0.01 for _ in range(2)]
    ref = [t.clone() for t in (WD, st[0], st[1], WE, st[2], st[3], bE, sb[0], sb[1])]
    groups = K.FeatureGroups(F, B * k, torch.device(DEV)).build(idx)
    off = groups.offsets.cpu()
    cnt = torch.bincount(idx[idx >= 0].long().cpu(), minlength=F)
    assert torch.equal(off[1:] - off[:-1], cnt.to(torch.int32))
    ent = groups.entries[: int(off[-1])].long()
    assert torch.equal(torch.sort(ent).values, torch.sort(torch.nonzero(idx.reshape(-1) >= 0).squeeze(1)).values)
    assert (idx.reshape(-1)[ent].cpu() == torch.repeat_interleave(torch.arange(F), cnt)).all()

    WDb = torch.empty(F, d, dtype=torch.bfloat16, device=DEV)
    WEb = torch.empty(F, d, dtype=torch.bfloat16, device=DEV)
    dn = torch.empty(F, device=DEV)
    gsq = torch.zeros(1, device=DEV)
    hp = dict(lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, step=3)
    K.sparse_grad_adam(groups, act, dact, x, dxhat, WD, st[0], st[1], WDb, WE, st[2], st[3], WEb, bE, sb[0], sb[1], dn, None, gsq, **hp)
    gD, gE, gb = K.ref_sparse_grads(idx, act, dact, x, dxhat, F)
    K.ref_adam(ref[0], gD, ref[1], ref[2], **hp)
    K.ref_adam(ref[3], gE, ref[4], ref[5], **hp)
    K.ref_adam(ref[6], gb, ref[7], ref[8], **hp)
    for got, want in zip((WD, st[0], st[1], WE, st[2], st[3], bE, sb[0], sb[1]), ref):
        assert torch.allclose(got, want, atol=1e-5, rtol=1e-4)
    assert torch.allclose(WDb.float(), WD, atol=1e-2, rtol=1e-2)
    assert torch.allclose(dn, WD.norm(dim=1), rtol=1e-4)
    want_sq = gD.pow(2).sum() + gE.pow(2).sum() + gb.pow(2).sum()
    assert torch.allclose(gsq[0], want_sq, rtol=1e-3)


def test_dense_helpers():
    g = torch.Generator().manual_seed(17)
    a = torch.randn(300, 520, generator=g).to(torch.bfloat16).to(DEV)
    assert torch.allclose(K.colsum_bf16(a), a.float().sum(0), atol=1e-3, rtol=1e-4)
    p = torch.randn(1000, generator=g).to(DEV)
    gr = torch.randn(1000, generator=g).to(DEV)
    m = torch.zeros(1000, device=DEV)
    v = torch.zeros(1000, device=DEV)
    rp, rm, rv = p.clone(), m.clone(), v.clone()
    K.adam_flat(p, gr, m, v, 1e-2, 0.9, 0.999, 1e-8, 1)
    K.ref_adam(rp, gr, rm, rv, 1e-2, 0.9, 0.999, 1e-8, 1)
    assert torch.allclose(p, rp, atol=1e-5) and torch.allclose(m, rm, rtol=1e-4) and torch.allclose(v, rv, rtol=1e-4)
    W = torch.randn(77, 130, generator=g).to(DEV)
    n = torch.empty(77, device=DEV)
    sh = torch.empty(77, 130, dtype=torch.bfloat16, device=DEV)
    K.row_norm_shadow(W, n, sh)
    assert torch.allclose(n, W.norm(dim=1), rtol=1e-5) and torch.equal(sh, W.to(torch.bfloat16))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,tshape", [((64, 1024), (1024,)), ((8, 16, 512), (512,)), ((32, 3, 256), (3, 256))])
def test_jumprelu_fused_matches_autograd(dtype, shape, tshape):
    from language_model_saes_b200.activation_functions import FusedSTEFunction, STEFunction

    g = torch.Generator(device="cpu").manual_seed(0)
    x = (torch.randn(shape, generator=g) * 0.5 + 0.3).to(dtype).to(DEV)
    log_t = (torch.randn(tshape, generator=g) * 0.3 - 1.0).to(dtype).to(DEV)
    dy = torch.randn(shape, generator=g).to(dtype).to(DEV)
    window = 0.5  # wide window: many hits, a strict test of the threshold gradient
    keep = tuple(range(-len(tshape), 0))

    xr, lr = x.clone().requires_grad_(), log_t.clone().requires_grad_()
    yr = STEFunction.apply(xr, lr.exp(), window, keep)
    yr.backward(dy)
    xf, lf = x.clone().requires_grad_(), log_t.clone().requires_grad_()
    yf = FusedSTEFunction.apply(xf, lf, window)
    yf.backward(dy)
    assert torch.equal(yf, yr)
    assert torch.equal(xf.grad, xr.grad)
    tol = dict(rtol=1e-4, atol=1e-4) if dtype == torch.float32 else dict(rtol=5e-2, atol=5e-2)
    assert torch.allclose(lf.grad.float(), lr.grad.float(), **tol), (lf.grad.float() - lr.grad.float()).abs().max()
    assert lf.grad.abs().sum() > 0


def test_sparse_decode_autograd_matches_dense():
    from language_model_saes_b200.ops.sparse_autograd import dense_to_padded_sparse, sparse_decode

    g = torch.Generator(device="cpu").manual_seed(0)
    B, F, d, k = 96, 2048, 256, 12
    acts = torch.zeros(B, F)
    cols = torch.stack([torch.randperm(F, generator=g)[:k] for _ in range(B)])
    acts.scatter_(1, cols, torch.rand(B, k, generator=g) + 0.1)
    acts[3] = 0  # a row without any non-zero
    acts = acts.to(DEV).requires_grad_()
    W = (torch.randn(F, d, generator=g) / d**0.5).to(DEV).requires_grad_()
    dy = torch.randn(B, d, generator=g).to(DEV)
    idx, val = dense_to_padded_sparse(acts.detach())
    assert idx.shape[1] % 8 == 0 and int((idx >= 0).sum()) == int((acts != 0).sum())
    out = sparse_decode(acts, W)
    out.backward(dy)
    Wb = W.detach().to(torch.bfloat16).float()
    ref_out = acts.detach() @ Wb
    assert torch.allclose(out, ref_out, atol=2e-3, rtol=2e-3)
    dyb = dy.to(torch.bfloat16).float()
    ref_dW = acts.detach().t() @ dyb
    assert torch.allclose(W.grad, ref_dW, atol=2e-3, rtol=2e-3)
    ref_da = (dyb @ Wb.t()) * (acts.detach() != 0)
    assert torch.allclose(acts.grad, ref_da, atol=5e-3, rtol=5e-3)


@pytest.mark.parametrize("M,heads,d,N,pair", [(256, 3, 128, 1024, True), (128, 2, 64, 256, False), (384, 1, 256, 4096, True), (200, 4, 64, 512, True)])
def test_head_sum_gemm_single_rank(M, heads, d, N, pair):
    """K-concatenated head sum on one rank: the bf16 result in the communicator's buffer against an fp32 product."""
    from language_model_saes_b200.parallel.symm import HeadSumComm

    dev = torch.device("cuda")
    torch.manual_seed(0)
    rows_per_head = N + 64  # the weight blocks may be longer than the columns in use
    x = torch.randn(M, heads * d, device=dev).to(torch.bfloat16)
    w = (torch.randn(heads * rows_per_head, d, device=dev) / d**0.5).to(torch.bfloat16)
    bias = torch.randn(N, device=dev)
    comm = HeadSumComm(None, dev, max_rows=M, n_cols=N)
    want = bias + sum(x[:, h * d : (h + 1) * d].float() @ w[h * rows_per_head : h * rows_per_head + N].float().T for h in range(heads))
    for call in range(3):
        got = comm.head_sum(x, w, bias, heads, rows_per_head, torch.float32, pair=pair)
        K.check_status(dev)
        assert torch.allclose(got, want, atol=2e-2, rtol=8e-3), (call, float((got - want).abs().max()))  # bf16 store
    got16 = comm.head_sum(x, w, bias, heads, rows_per_head, torch.bfloat16, pair=pair)
    assert torch.allclose(got16.float(), want, atol=5e-2, rtol=2e-2)


def test_crosscoder_fused_head_sum_matches_generic():
    from language_model_saes_b200.models.crosscoder import Crosscoder, CrosscoderConfig

    def make(fused):
        torch.manual_seed(0)
        cfg = CrosscoderConfig(hook_points=["a", "b", "c"], d_model=128, expansion_factor=8, act_fn="relu", device="cuda",
                               dtype=torch.bfloat16, norm_activation="inference", fused_head_sum=fused)  # fmt: skip
        m = Crosscoder(cfg)
        m.init_parameters(encoder_uniform_bound=0.1, decoder_uniform_bound=0.1, init_log_jumprelu_threshold_value=0.0)
        with torch.no_grad():
            m.b_E.normal_(std=0.05)
            m.W_E.mul_(1 + 0.1 * torch.arange(3, device="cuda").view(3, 1, 1))  # the heads differ
        return m

    a, b = make(True), make(False)
    x = torch.randn(256, 3, 128, device="cuda", dtype=torch.bfloat16)
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    fa, ha = a.encode(xa, return_hidden_pre=True)
    fb, hb = b.encode(xb, return_hidden_pre=True)
    K.check_status(torch.device("cuda"))
    assert torch.allclose(ha.float(), hb.float(), atol=5e-2, rtol=5e-2)
    g = torch.randn_like(fa)
    (fa * g).sum().backward()
    (fb * g).sum().backward()

    def close(u, v):  # a few ReLU gates flip between the two roundings of the pre-activations: compare in norm
        return float((u.float() - v.float()).norm() / v.float().norm()) < 0.05

    assert close(xa.grad, xb.grad) and close(a.W_E.grad, b.W_E.grad) and close(a.b_E.grad, b.b_E.grad)


@pytest.mark.parametrize("M,C,k,own", [(257, 256, 50, None), (64, 400, 50, (100, 150)), (33, 96, 64, (32, 64)), (16, 24, 32, None), (8, 37, 5, (0, 37))])
@pytest.mark.parametrize("use_gate,emit_gated", [(False, False), (True, False), (True, True)])
def test_topk_merge_matches_its_plain_statement(M, C, k, own, use_gate, emit_gated):
    """Candidate lists with empty slots, repeated values (ties go to the earlier slot), rows with fewer than k positive
    candidates, a restricted own range, and k larger than the list."""
    torch.manual_seed(C + k)
    if own is None:
        val = torch.randint(1, 40, (M, C), device="cuda").float() / 8  # few distinct values: many ties
    else:  # which of several equal candidates wins decides whether a winner lies in the own range: distinct values here
        val = torch.rand(M, C, device="cuda") + 0.01
    idx = torch.stack([torch.randperm(4096, device="cuda")[:C] for _ in range(M)]).to(torch.int32)
    empty = torch.rand(M, C, device="cuda") < 0.3
    idx[empty] = -1
    val[torch.rand(M, C, device="cuda") < 0.1] = 0.0  # non-positive candidates never win
    idx[0] = -1  # a row with nothing
    idx[1, 3:] = -1  # a row with fewer than k candidates
    gate = torch.rand(4096, device="cuda") + 0.5 if use_gate else None
    got_i, got_v = K.topk_merge(val, idx, k, gate, own=own, emit_gated=emit_gated)
    want_i, want_v = K.ref_topk_merge(val, idx, k, gate, own=own, emit_gated=emit_gated)
    K.check_status(torch.device("cuda"))
    # the plain statement uses torch.topk, whose order among EQUAL values is unspecified: compare as sets per row and
    # per value, and check the kernel's own rule (value descending, earlier slot first among equals) separately
    assert torch.equal((got_i >= 0).sum(1), (want_i >= 0).sum(1))
    if own is not None:  # distinct values: the winners and their places are determined
        assert torch.equal(got_i, want_i) and torch.allclose(got_v, want_v, rtol=1e-6)
    if own is not None or gate is None or emit_gated:  # (with ties AND a division by the winner's gate the values depend on who won)
        assert torch.allclose(torch.sort(got_v, dim=1, descending=True).values, torch.sort(want_v, dim=1, descending=True).values, rtol=1e-6)
    if own is None and not use_gate:
        kept = got_i >= 0
        n = kept.sum(1)
        assert all(bool(kept[r, : n[r]].all()) for r in range(M))  # winners fill the first places
        assert bool((got_v[:, 1:] <= got_v[:, :-1]).all())  # value descending (empty places hold 0 at the end)
        # every winner's value is at least every loser's value of that row
        low = torch.where(kept, got_v, torch.full_like(got_v, float("inf"))).min(1).values
        pool = torch.where(idx >= 0, val, torch.zeros_like(val))
        for r in range(M):
            won = set(got_i[r][kept[r]].tolist())
            lost = [float(pool[r, c]) for c in range(C) if int(idx[r, c]) >= 0 and int(idx[r, c]) not in won]
            assert not lost or max(lost) <= float(low[r])
