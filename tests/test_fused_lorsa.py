"""The fused low-rank sparse attention step (``ops.fused_lorsa.FusedLorsaStep``) against the generic autograd path of
the same model: losses and every parameter after a few Adam steps. On the CPU the step runs the plain-torch statements of
its kernels (the math and the step's own bookkeeping are what is checked); on a GPU the kernels themselves."""

import copy

import pytest
import torch

from language_model_saes_b200.models.lorsa import LorsaConfig, LowRankSparseAttention
from language_model_saes_b200.ops.fused_lorsa import FusedLorsaStep, _rotate, rotate_pair

DEVICES = [pytest.param("cuda", marks=pytest.mark.gpu), "cpu"]


def _model(dev, d=64, nqk=2, dqk=16, n_ov=64, n_ctx=32, k=6, **kw):
    torch.manual_seed(0)
    cfg = LorsaConfig(hook_point_in="blocks.1.ln1.hook_normalized", hook_point_out="blocks.1.hook_attn_out", d_model=d,
                      expansion_factor=n_ov / d, n_qk_heads=nqk, d_qk_head=dqk, rotary_dim=kw.pop("rotary_dim", dqk), n_ctx=n_ctx,
                      act_fn="topk", top_k=k, device=dev, dtype=torch.float32, norm_activation="inference", **kw)  # fmt: skip
    m = LowRankSparseAttention(cfg)
    m.init_parameters()
    with torch.no_grad():
        m.W_Q.mul_(3.0)  # attention patterns that are not flat
        m.W_K.mul_(3.0)
        for b in (m.b_Q, m.b_K, m.b_V, m.b_D):
            b.normal_(std=0.05)
    return m


def _batches(dev, n, b, s, d, seed=1):
    g = torch.Generator(device=dev).manual_seed(seed)
    mix = torch.randn(d, d, device=dev, generator=g) / d**0.5
    out = []
    for _ in range(n):
        x = torch.randn(b, s, d, device=dev, generator=g)
        y = torch.tanh(x @ mix).cumsum(1) / 4 + 0.1 * torch.randn(b, s, d, device=dev, generator=g)
        out.append((x.to(torch.bfloat16), y.to(torch.bfloat16)))
    return out


def _fill_freed_memory_with_nans(dev):
    """Leave NaN bit patterns (as bf16 pairs and as fp32) in blocks of many sizes that the caching allocator will hand out
    again: a kernel that reads memory nobody wrote then shows up as NaN instead of passing on a fresh process's zeros."""
    if dev != "cuda":
        return
    keep = []
    for n, c in ((128, 1000), (1024, 1000), (16384, 1000), (131072, 200), (1 << 20, 32), (32 << 20, 2)):
        keep += [torch.full((n,), 0x7FC07FC0, dtype=torch.int32, device=dev) for _ in range(c)]
    del keep
    torch.cuda.synchronize()


@pytest.mark.parametrize("adjacent,rotary_dim", [(True, 16), (False, 16), (True, 8)])
def test_inverse_rotation_is_the_backward_of_the_rotation(adjacent, rotary_dim):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 5, 3, 16, generator=g, requires_grad=True)
    ang = torch.rand(5, rotary_dim // 2, generator=g) * 6
    ang = ang.repeat_interleave(2, dim=1) if adjacent else ang.repeat(1, 2)
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    y = _rotate(x, cos, sin, adjacent, rotary_dim)
    assert torch.allclose(_rotate(y, cos, -sin, adjacent, rotary_dim), x, atol=1e-6)  # a rotation: undone by the opposite angle
    dy = torch.randn(y.shape, generator=g)
    (dx,) = torch.autograd.grad(y, x, dy)
    assert torch.allclose(dx, _rotate(dy, cos, -sin, adjacent, rotary_dim), atol=1e-6)


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("adjacent,width,rotary_dim", [(True, 16, 16), (True, 64, 64), (True, 32, 16), (False, 64, 64), (False, 64, 32), (False, 16, 8)])
@pytest.mark.parametrize("inverse", [False, True])
def test_rotation_of_two_tensors_matches_the_plain_statement(dev, adjacent, width, rotary_dim, inverse):
    """On a GPU the aligned cases run the one-launch kernel (bf16 in and out, fp32 arithmetic); the others and the CPU
    run the torch statement. Either way the result is the fp32 rotation of the same bf16 inputs up to one rounding."""
    g = torch.Generator(device=dev).manual_seed(0)
    b, s, h = 3, 24, 5
    qa = torch.randn(b, s, h, width, device=dev, generator=g).to(torch.bfloat16)
    ka = torch.randn(b, s, h, width, device=dev, generator=g).to(torch.bfloat16)
    ang = torch.rand(s + 3, rotary_dim // 2, device=dev, generator=g) * 6  # a table longer than the sequence
    ang = ang.repeat_interleave(2, dim=1) if adjacent else ang.repeat(1, 2)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    oq, ok = rotate_pair(qa, ka, cos, sin, adjacent, inverse=inverse)
    sn = -sin if inverse else sin
    for got, x in ((oq, qa), (ok, ka)):
        want = _rotate(x.float(), cos[None, :s, None, :], sn[None, :s, None, :], adjacent, rotary_dim)
        assert got.shape == x.shape and got.dtype == x.dtype
        assert torch.allclose(got.float(), want, atol=3e-2, rtol=2e-2)
        if dev == "cuda" and rotary_dim % (8 if adjacent else 16) == 0:
            # the kernel rounds once, from the fp32 result (a fused multiply-add may move a tie)
            assert float((got != want.to(torch.bfloat16)).float().mean()) < 1e-3


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("variant", ["rotary", "half_split_partial_rotary", "no_positions_no_gate", "rotary_wide_heads",
                                     "rotary_wide_heads_library", "qk_norm"])  # fmt: skip
def test_fused_lorsa_step_matches_autograd(dev, variant, monkeypatch):
    if variant == "qk_norm":
        if dev == "cuda":
            pytest.skip("this variant is verified on the CPU only so far")
        monkeypatch.setenv("LMSAE_FUSED_LORSA_QK_NORM", "1")
    kw = {"rotary": {}, "half_split_partial_rotary": dict(rotary_adjacent_pairs=False, rotary_dim=8),
          "qk_norm": dict(use_post_qk_ln=True, normalization_type="RMS"),
          "no_positions_no_gate": dict(positional_embedding_type="none", sparsity_include_decoder_norm=False),
          # head widths that the tensor-core attention kernels take (on a GPU the step then runs them)
          "rotary_wide_heads": dict(dqk=64, n_ov=128), "rotary_wide_heads_library": dict(dqk=64, n_ov=128)}[variant]  # fmt: skip
    d, b, s, lr, steps = 64, 3, 32, 1e-3, 4
    ref = _model(dev, d=d, n_ctx=s, **kw)
    if variant == "qk_norm":
        with torch.no_grad():  # scales that are not all one
            ref.ln_q.w.mul_(1 + 0.2 * torch.randn_like(ref.ln_q.w))
            ref.ln_k.w.mul_(1 + 0.2 * torch.randn_like(ref.ln_k.w))
    fused_model = copy.deepcopy(ref)
    ok, why = FusedLorsaStep.supports(fused_model)
    assert ok, why
    engine = FusedLorsaStep(fused_model, attention="library" if variant.endswith("library") else "tensor_core")
    if dev == "cuda":
        from language_model_saes_b200.ops import attention as A

        q = torch.empty(b, s, engine.h, engine.dqk, device=dev)
        assert A.supported(q, torch.empty(b, s, engine.h, engine.group_size, device=dev)) == variant.startswith("rotary_wide")
    opt = torch.optim.Adam(ref.parameters(), lr=lr)
    start = {n: p.detach().clone() for n, p in ref.named_parameters()}
    ref_losses, fused_losses = [], []
    hin, hout = ref.cfg.hook_point_in, ref.cfg.hook_point_out
    for x, y in _batches(dev, steps, b, s, d):
        _fill_freed_memory_with_nans(dev)
        opt.zero_grad()
        batch = {hin: x.float(), hout: y.float(), "tokens": torch.zeros(b, s, dtype=torch.long, device=dev)}
        with torch.autocast(dev, dtype=torch.bfloat16, enabled=dev == "cuda"):
            out = ref.compute_loss(batch, sparsity_loss_type=None, return_aux_data=True)
        out["loss"].backward()
        opt.step()
        ref_losses.append(float(out["loss"].detach()))
        fused_losses.append(float(engine.step(x, y, ref.cfg.top_k, lr)))
    r, f = torch.tensor(ref_losses), torch.tensor(fused_losses)
    assert torch.allclose(r, f, rtol=3e-2 if dev == "cuda" else 5e-3), (ref_losses, fused_losses)
    # Adam's first steps move every weight that got any gradient by about lr whatever the gradient's size: compare the
    # movement, not a rounding tolerance
    for name, a in ref.named_parameters():
        if name == "b_K" and variant != "rotary":
            # one bias on every key shifts each score row by a constant, which the softmax ignores: without positions
            # (and on the columns that a partial rotation leaves alone) the true gradient is zero and Adam steps along
            # rounding noise in both implementations
            continue
        bb = dict(fused_model.named_parameters())[name].detach().float()
        moved = (a.detach().float() - start[name].float()).abs().mean()
        tol = (0.3 if dev == "cuda" else 0.08) * (3.0 if name == "b_K" else 1.0)  # b_K: small gradient, see above
        assert float((a.detach().float() - bb).abs().mean()) < tol * float(moved) + 1e-7, name
    # codes outside a step (evaluation): the same heads as the model's own encoder picks
    x, _ = _batches(dev, 1, b, s, d, seed=5)[0]
    idx, act = engine.encode(x, ref.cfg.top_k)
    with torch.no_grad(), torch.autocast(dev, dtype=torch.bfloat16, enabled=dev == "cuda"):
        acts = fused_model.encode(x.float())
    want = (acts.reshape(b * s, -1) != 0).sum(-1)
    assert torch.equal((idx >= 0).sum(-1), want) or float(((idx >= 0).sum(-1) - want).abs().float().mean()) < 0.5
    state = engine.optimizer_state()
    for name, p in fused_model.named_parameters():
        assert state[name]["exp_avg"].shape == p.shape, name


def _tp_body():
    import torch.distributed as dist

    from language_model_saes_b200.parallel.mesh import DimMap, build_mesh

    d, b, s, lr = 64, 2, 16, 1e-3
    full = _model("cpu", d=d, nqk=4, dqk=16, n_ov=64, n_ctx=s, k=6)
    single = copy.deepcopy(full)
    e1 = FusedLorsaStep(single)
    mesh = build_mesh("cpu", (1, 2), ("data", "model"))
    shard = LowRankSparseAttention(full.cfg.model_copy(), mesh)
    shard.load_full_state_dict(full.full_state_dict())
    e2 = FusedLorsaStep(shard)
    assert e2.tp == 2 and e2.h == 2 and e2.F == 32
    for x, y in _batches("cpu", 3, b, s, d):
        want = e1.step(x, y, 6, lr)
        got = e2.step(x, y, 6, lr)
        assert torch.allclose(want, got, rtol=1e-4), (want, got)
    for name in ("W_Q", "W_K", "W_V", "W_O", "b_Q", "b_V"):
        whole = DimMap({"model": 0}).gather(getattr(shard, name).data, mesh)
        assert torch.allclose(whole, getattr(single, name).data, atol=2e-5), name
    assert torch.allclose(shard.b_D.data, single.b_D.data, atol=2e-5)
    dist.barrier()


def _dp_body():
    import torch.distributed as dist

    from language_model_saes_b200.parallel.mesh import build_mesh

    d, b, s, lr = 64, 4, 16, 1e-3
    full = _model("cpu", d=d, nqk=4, dqk=16, n_ov=64, n_ctx=s, k=6)
    single = copy.deepcopy(full)
    e1 = FusedLorsaStep(single)
    r = dist.get_rank()
    mesh = build_mesh("cpu", (2, 1), ("data", "model"))
    rep = LowRankSparseAttention(full.cfg.model_copy(), mesh)
    rep.load_full_state_dict(full.full_state_dict())
    e2 = FusedLorsaStep(rep)
    assert e2.dp == 2 and e2.tp == 1
    g = torch.Generator().manual_seed(11)
    for x, y in _batches("cpu", 3, b, s, d):
        mask = torch.rand(b, s, generator=g) > 0.25
        w = mask.reshape(-1).float()
        want = e1.step(x, y, 6, lr, row_weight=w * (w.numel() / w.sum()))
        half = slice(r * b // 2, (r + 1) * b // 2)  # whole sequences per replica
        got = e2.step(x[half], y[half], 6, lr, row_weight=w.view(b, s)[half].reshape(-1) * (w.numel() / w.sum()))
        assert torch.allclose(want, got, rtol=1e-4), (want, got)
    for name, p in single.named_parameters():
        assert torch.allclose(dict(rep.named_parameters())[name].data, p.data, atol=2e-5), name
    dist.barrier()


def test_fused_lorsa_step_replicas_match_single():
    from language_model_saes_b200.testing import distributed_test

    distributed_test(nproc_per_node=2, backend="gloo")(_dp_body)()


def test_fused_lorsa_step_head_shards_match_single():
    from language_model_saes_b200.testing import distributed_test

    distributed_test(nproc_per_node=2, backend="gloo")(_tp_body)()


@pytest.mark.gpu
def test_trainer_picks_the_fused_lorsa_path_and_the_loss_goes_down():
    import tempfile

    from language_model_saes_b200.trainer import Trainer, TrainerConfig

    d, b, s, steps = 64, 8, 64, 30
    m = _model("cuda", d=d, nqk=4, dqk=16, n_ov=256, n_ctx=s, k=16)
    hin, hout = m.cfg.hook_point_in, m.cfg.hook_point_out
    data = _batches("cuda", 4, b, s, d)

    def stream():
        for i in range(steps + 1):
            x, y = data[i % len(data)]
            mask = torch.ones(b, s, dtype=torch.bool, device="cuda")
            mask[:, 0] = False  # the path with row weights
            yield {hin: x, hout: y, "tokens": torch.zeros(b, s, dtype=torch.long, device="cuda"), "mask": mask}

    losses = []
    with tempfile.TemporaryDirectory() as tmp:
        tr = Trainer(TrainerConfig(total_training_tokens=steps * b * s, lr=2e-3, lr_warm_up_steps=2, log_frequency=10**6, n_checkpoints=0,
                                   exp_result_path=tmp, skip_metrics_calculation=False))  # fmt: skip
        tr.cfg.log_frequency = 10
        emitted = []
        tr._emit = lambda sae, out: emitted.append(out)
        orig = tr._fused_iteration

        def spy(*a, **kw):
            out = orig(*a, **kw)
            losses.append(float(out))
            return out

        tr._fused_iteration = spy
        tr.fit(m, stream())
        assert type(tr.fused).__name__ == "FusedLorsaStep"
        assert len(emitted) == steps // 10 and all("metrics/explained_variance" in e and "details/current_learning_rate" in e for e in emitted)
    assert len(losses) == steps and all(l == l for l in losses) and sum(losses[-5:]) < sum(losses[:5]), losses


@pytest.mark.parametrize("dev", DEVICES)
def test_fused_lorsa_step_with_a_token_mask_matches_autograd(dev):
    """Masked tokens carry no loss (mean over the valid ones) but stay in the sequence as keys and values."""
    d, b, s, lr = 64, 3, 32, 1e-3
    ref = _model(dev, d=d, n_ctx=s)
    fused_model = copy.deepcopy(ref)
    engine = FusedLorsaStep(fused_model)
    opt = torch.optim.Adam(ref.parameters(), lr=lr)
    start = {n: p.detach().clone() for n, p in ref.named_parameters()}
    hin, hout = ref.cfg.hook_point_in, ref.cfg.hook_point_out
    g = torch.Generator(device=dev).manual_seed(3)
    for x, y in _batches(dev, 3, b, s, d):
        _fill_freed_memory_with_nans(dev)
        mask = torch.rand(b, s, device=dev, generator=g) > 0.3
        mask[:, 0] = False  # e.g. a beginning-of-sequence token
        opt.zero_grad()
        batch = {hin: x.float(), hout: y.float(), "tokens": torch.zeros(b, s, dtype=torch.long, device=dev), "mask": mask}
        with torch.autocast(dev, dtype=torch.bfloat16, enabled=dev == "cuda"):
            out = ref.compute_loss(batch, sparsity_loss_type=None, return_aux_data=True)
        out["loss"].backward()
        opt.step()
        w = mask.reshape(-1).float()
        got = engine.step(x, y, ref.cfg.top_k, lr, row_weight=w * (w.numel() / w.sum()))
        assert torch.allclose(out["loss"].detach().float(), got, rtol=3e-2 if dev == "cuda" else 5e-3), (out["loss"], got)
    for name, a in ref.named_parameters():
        bb = dict(fused_model.named_parameters())[name].detach().float()
        moved = (a.detach().float() - start[name].float()).abs().mean()
        tol = (0.3 if dev == "cuda" else 0.08) * (3.0 if name == "b_K" else 1.0)
        assert float((a.detach().float() - bb).abs().mean()) < tol * float(moved) + 1e-7, name


def test_family_metrics_of_a_logging_step_come_from_the_models_own_forward(tmp_path):
    """What the fused Lorsa / CLT / crosscoder iterations log on a logging step: the generic path's metric names, computed
    without a graph from one batch (here after a two-step CPU fit, which sets the trainer's schedules up)."""
    from language_model_saes_b200.trainer import Trainer, TrainerConfig

    d, b, s = 64, 2, 16
    m = _model("cpu", d=d, n_ctx=s)
    hin, hout = m.cfg.hook_point_in, m.cfg.hook_point_out
    data = _batches("cpu", 3, b, s, d)
    batches = [{hin: x.float(), hout: y.float(), "tokens": torch.zeros(b, s, dtype=torch.long)} for x, y in data]
    tr = Trainer(TrainerConfig(total_training_tokens=2 * b * s, lr=1e-3, lr_warm_up_steps=1, log_frequency=10**6, n_checkpoints=0,
                               exp_result_path=str(tmp_path), skip_metrics_calculation=True))  # fmt: skip
    tr.fit(m, iter(batches))
    before = {n: p.detach().clone() for n, p in m.named_parameters()}
    out = tr._family_metrics(m, batches[0])
    for key in ("metrics/explained_variance", "metrics/l0", "metrics/l2_norm_error", "losses/mse_loss"):
        assert key in out, (key, sorted(out))
    assert 0 < float(out["metrics/l0"]) <= m.cfg.top_k
    assert all(p.grad is None or not p.grad.any() for p in m.parameters())
    assert all(torch.equal(before[n], p) for n, p in m.named_parameters())  # a measurement: nothing moves


def test_fused_lorsa_optimizer_state_round_trip_continues_the_run():
    """Moments and step counter saved by parameter name and loaded into a fresh engine: the next step is the same."""
    d, b, s, lr = 64, 2, 16, 1e-3
    m1 = _model("cpu", d=d, n_ctx=s)
    e1 = FusedLorsaStep(m1)
    data = _batches("cpu", 3, b, s, d)
    for x, y in data[:2]:
        e1.step(x, y, 6, lr)
    m2 = copy.deepcopy(m1)
    saved = {k: ({kk: vv.clone() for kk, vv in v.items()} if isinstance(v, dict) else v) for k, v in e1.optimizer_state().items()}
    e2 = FusedLorsaStep(m2)
    e2.load_optimizer_state(saved)
    assert e2.t == e1.t == 2
    x, y = data[2]
    assert torch.equal(e1.step(x, y, 6, lr), e2.step(x, y, 6, lr))
    for (name, p), (_, q) in zip(m1.named_parameters(), m2.named_parameters()):
        assert torch.equal(p, q), name


def _tp_dp_body():
    import torch.distributed as dist

    from language_model_saes_b200.parallel.mesh import DimMap, build_mesh

    d, b, s, lr = 64, 4, 16, 1e-3
    full = _model("cpu", d=d, nqk=4, dqk=16, n_ov=64, n_ctx=s, k=6)
    single = copy.deepcopy(full)
    e1 = FusedLorsaStep(single)
    mesh = build_mesh("cpu", (2, 2), ("data", "model"))
    shard = LowRankSparseAttention(full.cfg.model_copy(), mesh)
    shard.load_full_state_dict(full.full_state_dict())
    e2 = FusedLorsaStep(shard)
    assert e2.tp == 2 and e2.dp == 2
    dr = mesh.get_local_rank("data")
    for x, y in _batches("cpu", 3, b, s, d):
        want = e1.step(x, y, 6, lr)
        half = slice(dr * b // 2, (dr + 1) * b // 2)
        got = e2.step(x[half], y[half], 6, lr)
        assert torch.allclose(want, got, rtol=1e-4), (want, got)
    for name in ("W_Q", "W_K", "W_V", "W_O", "b_Q", "b_V"):
        whole = DimMap({"model": 0}).gather(getattr(shard, name).data, mesh)
        assert torch.allclose(whole, getattr(single, name).data, atol=2e-5), name
    assert torch.allclose(shard.b_D.data, single.b_D.data, atol=2e-5)
    dist.barrier()


def test_fused_lorsa_step_head_shards_and_replicas_on_four_ranks_match_single():
    from language_model_saes_b200.testing import distributed_test

    distributed_test(nproc_per_node=4, backend="gloo")(_tp_dp_body)()
