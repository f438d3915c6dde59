"""The fused crosscoder step (``ops.fused_crosscoder.FusedCrosscoderStep``) against the generic autograd path of the
same model: losses and every parameter after a few Adam steps. On the CPU the step runs the plain-torch statements of
its kernels (the math and the step's own bookkeeping are what is checked); on a GPU the kernels themselves."""

import copy

import pytest
import torch

from language_model_saes_b200.models.crosscoder import Crosscoder, CrosscoderConfig
from language_model_saes_b200.ops.fused_crosscoder import FusedCrosscoderStep

DEVICES = [pytest.param("cuda", marks=pytest.mark.gpu), "cpu"]


def _model(dev, H=3, d=64, F=512, thr=-0.5):
    torch.manual_seed(0)
    cfg = CrosscoderConfig(hook_points=[f"s{i}" for i in range(H)], d_model=d, expansion_factor=F / d, act_fn="jumprelu", device=dev,
                           dtype=torch.float32, norm_activation="inference")  # fmt: skip
    m = Crosscoder(cfg)
    m.init_parameters(encoder_uniform_bound=0.2, decoder_uniform_bound=0.2, init_log_jumprelu_threshold_value=thr)
    m.set_decoder_to_fixed_norm(1.0, True)
    m.init_encoder_with_decoder_transpose(1.0 / H)
    with torch.no_grad():  # heads that differ, non-trivial biases and thresholds
        m.W_D.mul_(1 + 0.1 * torch.arange(H, device=dev).view(H, 1, 1))
        m.b_E.add_(0.02 * torch.randn_like(m.b_E))
        m.b_D.add_(0.02 * torch.randn_like(m.b_D))
        m.activation_function.log_jumprelu_threshold.add_(0.1 * torch.randn_like(m.activation_function.log_jumprelu_threshold))
    return m


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("l1,lp", [(0.0, 0.0), (3e-2, 0.0), (0.0, 2e-3), (3e-2, 2e-3)])
def test_fused_crosscoder_step_matches_autograd(dev, l1, lp):
    H, d, F, B, lr, steps = 3, 64, 512, 256, 1e-3, 4
    ref = _model(dev, H, d, F)
    fused_model = copy.deepcopy(ref)
    engine = FusedCrosscoderStep(fused_model, list_width=F)  # lists wide enough for every candidate
    assert FusedCrosscoderStep.supports(fused_model)[0]
    g = torch.Generator(device=dev).manual_seed(1)
    basis = torch.randn(8, d, device=dev, generator=g)
    data = []
    for _ in range(steps):
        z = torch.randn(B, 8, device=dev, generator=g)
        x = torch.stack([z @ basis * (1 + 0.2 * h) + 0.3 * torch.randn(B, d, device=dev, generator=g) for h in range(H)], dim=1)
        data.append((x * (d**0.5 / x.norm(dim=-1).mean())).to(torch.bfloat16))
    opt = torch.optim.Adam(ref.parameters(), lr=lr)
    ref_losses, fused_losses = [], []
    tokens = torch.zeros(B, dtype=torch.long, device=dev)
    for x in data:
        opt.zero_grad()
        batch = {f"s{h}": x[:, h].float() for h in range(H)} | {"tokens": tokens}
        with torch.autocast(dev, dtype=torch.bfloat16, enabled=dev == "cuda"):
            out = ref.compute_loss(batch, sparsity_loss_type="tanh" if l1 else None, l1_coefficient=l1, lp_coefficient=lp,
                                   return_aux_data=True)  # fmt: skip
        out["loss"].backward()
        opt.step()
        ref_losses.append(float(out["loss"].detach()))
        fused_losses.append(float(engine.step(x, lr, l1_coefficient=l1, lp_coefficient=lp)))
        if lp:
            assert float(engine.last["l_p"]) > 0 and abs(float(engine.last["l_p"]) - float(out["l_p"].mean())) < 3e-2 * float(out["l_p"].mean())
    assert int(engine.list_overflow) == 0
    r, f = torch.tensor(ref_losses), torch.tensor(fused_losses)
    tol = 3e-2 if dev == "cuda" else 2e-3  # (the GPU reference runs under bf16 autocast)
    assert torch.allclose(r, f, rtol=tol), (ref_losses, fused_losses)
    assert r[-1] < r[0]
    # Adam's first steps move every weight that got any gradient by about lr whatever the gradient's size: compare the
    # movement, not a rounding tolerance
    for name in ("W_D", "W_E", "b_E", "b_D", "activation_function.log_jumprelu_threshold"):
        a = dict(ref.named_parameters())[name].detach().float()
        b = dict(fused_model.named_parameters())[name].detach().float()
        moved = (a - dict(_model(dev, H, d, F).named_parameters())[name].detach().float()).abs().mean()
        assert float((a - b).abs().mean()) < (0.25 if dev == "cuda" else 0.05) * float(moved) + 1e-7, name


@pytest.mark.parametrize("dev", DEVICES)
@pytest.mark.parametrize("l1,lp", [(0.0, 0.0), (3e-2, 0.0), (3e-2, 2e-3)])
def test_jumprelu_sae_is_the_one_head_case_of_the_fused_step(dev, l1, lp):
    """A JumpReLU ``SparseAutoEncoder`` on the same step (parameters viewed with a head axis of one) against autograd on the
    model: losses, every parameter after a few Adam steps, and the optimizer state in the model's parameter shapes."""
    from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder

    d, F, B, lr, steps = 64, 512, 256, 1e-3, 4

    def make():
        torch.manual_seed(0)
        cfg = SAEConfig(hook_point_in="h", hook_point_out="h", d_model=d, expansion_factor=F / d, act_fn="jumprelu", device=dev,
                        dtype=torch.float32, norm_activation="inference")  # fmt: skip
        m = SparseAutoEncoder(cfg)
        m.init_parameters(encoder_uniform_bound=0.2, decoder_uniform_bound=0.2, init_log_jumprelu_threshold_value=-0.5)
        m.set_decoder_to_fixed_norm(1.0, True)
        m.init_encoder_with_decoder_transpose()
        with torch.no_grad():
            m.b_E.add_(0.02 * torch.randn_like(m.b_E))
            m.b_D.add_(0.02 * torch.randn_like(m.b_D))
            m.activation_function.log_jumprelu_threshold.add_(0.1 * torch.randn_like(m.activation_function.log_jumprelu_threshold))
        return m

    ref, fused_model = make(), make()
    ok, why = FusedCrosscoderStep.supports(fused_model)
    assert ok, why
    engine = FusedCrosscoderStep(fused_model, list_width=F)
    g = torch.Generator(device=dev).manual_seed(1)
    basis = torch.randn(8, d, device=dev, generator=g)
    opt = torch.optim.Adam(ref.parameters(), lr=lr)
    tokens = torch.zeros(B, dtype=torch.long, device=dev)
    ref_losses, fused_losses = [], []
    for _ in range(steps):
        x = torch.randn(B, 8, device=dev, generator=g) @ basis + 0.3 * torch.randn(B, d, device=dev, generator=g)
        x = (x * (d**0.5 / x.norm(dim=-1).mean())).to(torch.bfloat16)
        opt.zero_grad()
        with torch.autocast(dev, dtype=torch.bfloat16, enabled=dev == "cuda"):
            out = ref.compute_loss({"h": x.float(), "tokens": tokens}, sparsity_loss_type="tanh" if l1 else None, l1_coefficient=l1,
                                   lp_coefficient=lp)  # fmt: skip
        out["loss"].backward()
        opt.step()
        ref_losses.append(float(out["loss"].detach()))
        fused_losses.append(float(engine.step(x.unsqueeze(1), lr, l1_coefficient=l1, lp_coefficient=lp)))
    r, f = torch.tensor(ref_losses), torch.tensor(fused_losses)
    assert torch.allclose(r, f, rtol=3e-2 if dev == "cuda" else 2e-3), (ref_losses, fused_losses)
    start = dict(make().named_parameters())
    for name, a in ref.named_parameters():
        b = dict(fused_model.named_parameters())[name].detach().float()
        moved = (a.detach().float() - start[name].detach().float()).abs().mean()
        assert float((a.detach().float() - b).abs().mean()) < (0.25 if dev == "cuda" else 0.05) * float(moved) + 1e-7, name
    state = engine.optimizer_state()
    for name, p in fused_model.named_parameters():
        assert state[name]["exp_avg"].shape == p.shape, name


def test_fused_crosscoder_selection_is_the_union_over_heads_cpu():
    """A head's codes are exactly its own JumpReLU outputs: the union list only adds zero entries."""
    m = _model("cpu", 2, 32, 128)
    engine = FusedCrosscoderStep(m, list_width=128)
    x = torch.randn(16, 2, 32).to(torch.bfloat16)
    want, _ = m.encode(x.float(), return_hidden_pre=True)  # [B, H, F]
    engine.step(x, 0.0)  # lr 0: nothing moves
    assert float(engine.last["l0"]) >= float((want != 0).any(dim=1).sum(-1).float().mean()) - 1e-6


@pytest.mark.gpu
def test_trainer_picks_the_fused_crosscoder_path_and_the_loss_goes_down():
    import tempfile

    from language_model_saes_b200.trainer import Trainer, TrainerConfig

    H, d, F, B, steps = 4, 64, 2048, 512, 30
    m = _model("cuda", H, d, F, thr=0.3)
    m.cfg.norm_activation = "dataset-wise"
    m.set_dataset_average_activation_norm({f"s{i}": d**0.5 for i in range(H)})
    g = torch.Generator(device="cuda").manual_seed(1)
    basis = torch.randn(12, d, device="cuda", generator=g)

    def stream():
        for _ in range(steps + 1):
            z = torch.randn(B, 12, device="cuda", generator=g)
            rec = {}
            for h in range(H):
                x = z @ basis + 0.05 * (h + 1) * torch.randn(B, d, device="cuda", generator=g)
                rec[f"s{h}"] = (x * (d**0.5 / x.norm(dim=-1).mean())).to(torch.bfloat16)
            rec["tokens"] = torch.zeros(B, dtype=torch.long, device="cuda")
            yield rec

    losses = []
    with tempfile.TemporaryDirectory() as tmp:
        tr = Trainer(TrainerConfig(total_training_tokens=steps * B, lr=2e-3, lr_warm_up_steps=2, log_frequency=10**6, n_checkpoints=0,
                                   exp_result_path=tmp, skip_metrics_calculation=True, l1_coefficient=1e-3, sparsity_loss_type="tanh"))  # fmt: skip
        orig = tr._fused_iteration

        def spy(*a, **kw):
            out = orig(*a, **kw)
            losses.append(float(out))
            return out

        tr._fused_iteration = spy
        tr.fit(m, stream())
        assert type(tr.fused).__name__ == "FusedCrosscoderStep"
    assert len(losses) == steps and all(l == l for l in losses) and sum(losses[-5:]) < sum(losses[:5]), losses


@pytest.mark.gpu
def test_trainer_trains_a_jumprelu_sae_on_the_fused_path():
    import tempfile

    from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
    from language_model_saes_b200.trainer import Trainer, TrainerConfig

    d, F, B, steps = 64, 2048, 512, 30
    torch.manual_seed(0)
    cfg = SAEConfig(hook_point_in="h", hook_point_out="h", d_model=d, expansion_factor=F / d, act_fn="jumprelu", device="cuda",
                    dtype=torch.float32)  # fmt: skip
    m = SparseAutoEncoder(cfg)
    m.init_parameters(encoder_uniform_bound=0.2, decoder_uniform_bound=0.2, init_log_jumprelu_threshold_value=0.3)
    m.set_decoder_to_fixed_norm(1.0, True)
    m.init_encoder_with_decoder_transpose()
    m.set_dataset_average_activation_norm({"h": d**0.5})
    g = torch.Generator(device="cuda").manual_seed(1)
    basis = torch.randn(12, d, device="cuda", generator=g)

    def stream():
        for _ in range(steps + 1):
            x = torch.randn(B, 12, device="cuda", generator=g) @ basis + 0.05 * torch.randn(B, d, device="cuda", generator=g)
            yield {"h": (x * (d**0.5 / x.norm(dim=-1).mean())).to(torch.bfloat16), "tokens": torch.zeros(B, dtype=torch.long, device="cuda")}

    losses = []
    with tempfile.TemporaryDirectory() as tmp:
        tr = Trainer(TrainerConfig(total_training_tokens=steps * B, lr=2e-3, lr_warm_up_steps=2, log_frequency=10**6, n_checkpoints=0,
                                   exp_result_path=tmp, skip_metrics_calculation=True, l1_coefficient=1e-3, sparsity_loss_type="tanh"))  # fmt: skip
        orig = tr._fused_iteration

        def spy(*a, **kw):
            out = orig(*a, **kw)
            losses.append(float(out))
            return out

        tr._fused_iteration = spy
        tr.fit(m, stream())
        assert type(tr.fused).__name__ == "FusedCrosscoderStep" and tr.fused.single
    assert len(losses) == steps and all(l == l for l in losses) and sum(losses[-5:]) < sum(losses[:5]), losses


def _replica_body():
    import torch.distributed as dist

    from language_model_saes_b200.parallel.mesh import build_mesh

    H, d, F, B, lr, steps, l1 = 3, 64, 512, 128, 1e-3, 3, 3e-2
    full = _model("cpu", H, d, F)
    single = copy.deepcopy(full)
    mesh = build_mesh("cpu", (2, 1), ("data", "model"))
    replica = Crosscoder(full.cfg.model_copy(), mesh)
    replica.load_full_state_dict(full.full_state_dict())
    e1, e2 = FusedCrosscoderStep(single, list_width=F), FusedCrosscoderStep(replica, list_width=F)
    assert e2.dp == 2 and FusedCrosscoderStep.supports(replica)[0]
    g = torch.Generator().manual_seed(1)
    basis = torch.randn(8, d, generator=g)
    r, half = dist.get_rank(), B // 2
    for _ in range(steps):
        z = torch.randn(B, 8, generator=g)
        x = torch.stack([z @ basis * (1 + 0.2 * h) + 0.3 * torch.randn(B, d, generator=g) for h in range(H)], dim=1)
        x = (x * (d**0.5 / x.norm(dim=-1).mean())).to(torch.bfloat16)
        a = e1.step(x, lr, l1_coefficient=l1)
        b = e2.step(x[r * half : (r + 1) * half], lr, l1_coefficient=l1)
        assert torch.allclose(a, b, rtol=1e-4), (a, b)
        assert torch.allclose(e1.last["l0"], e2.last["l0"])
    for (name, p), (_, q) in zip(single.named_parameters(), replica.named_parameters()):
        assert torch.allclose(p.data, q.data, atol=2e-6), name
    dist.barrier()


def test_fused_crosscoder_step_with_replicas_matches_one_process():
    """Tokens split over two gloo ranks (reconstruction and tanh sparsity losses, shared thresholds): same losses and
    parameters as one process on the whole batch."""
    from language_model_saes_b200.testing import distributed_test

    distributed_test(nproc_per_node=2, backend="gloo")(_replica_body)()


@pytest.mark.parametrize("H", [3, 1])
def test_tanh_quad_penalty_on_the_fused_step_matches_autograd(H):
    """The frequency-weighted penalty ``l1 * sum_f q_f (1 + q_f / scale)`` (the reference's usual choice for JumpReLU
    dictionaries): losses and every parameter after a few Adam steps against the model's own loss on the CPU. A large
    ``l1`` and a small scale make the penalty's gradients (decoder norms, thresholds, encoder) count."""
    dev, d, F, B, lr, steps, l1, scale = "cpu", 64, 512, 256, 1e-3, 4, 5e-2, 0.05
    ref = _model(dev, H, d, F)
    fused_model = copy.deepcopy(ref)
    engine = FusedCrosscoderStep(fused_model, list_width=F)
    g = torch.Generator().manual_seed(2)
    basis = torch.randn(8, d, generator=g)
    opt = torch.optim.Adam(ref.parameters(), lr=lr)
    start = {n: p.detach().clone() for n, p in ref.named_parameters()}
    tokens = torch.zeros(B, dtype=torch.long)
    for _ in range(steps):
        z = torch.randn(B, 8, generator=g)
        x = torch.stack([z @ basis * (1 + 0.2 * h) + 0.3 * torch.randn(B, d, generator=g) for h in range(H)], dim=1)
        x = (x * (d**0.5 / x.norm(dim=-1).mean())).to(torch.bfloat16)
        opt.zero_grad()
        batch = {f"s{h}": x[:, h].float() for h in range(H)} | {"tokens": tokens}
        out = ref.compute_loss(batch, sparsity_loss_type="tanh-quad", l1_coefficient=l1, frequency_scale=scale, return_aux_data=True)
        out["loss"].backward()
        opt.step()
        got = engine.step(x, lr, l1_coefficient=l1, sparsity_loss_type="tanh-quad", frequency_scale=scale)
        assert torch.allclose(out["loss"].detach(), got, rtol=2e-3), (out["loss"], got)
        assert torch.allclose(out["l_s"].detach().float().mean(), engine.last["l_s"], rtol=5e-3)
        assert float(engine.last["l_s"]) > 0.02 * float(got)  # the penalty is a visible part of the loss
    for name, a in ref.named_parameters():
        b = dict(fused_model.named_parameters())[name].detach().float()
        moved = (a.detach().float() - start[name].float()).abs().mean()
        assert float((a.detach().float() - b).abs().mean()) < 0.05 * float(moved) + 1e-7, name


def _quad_replica_body():
    import torch.distributed as dist

    from language_model_saes_b200.parallel.mesh import build_mesh

    H, d, F, B, lr, l1, scale = 2, 64, 256, 128, 1e-3, 5e-2, 0.05
    full = _model("cpu", H, d, F)
    single = copy.deepcopy(full)
    replica = Crosscoder(full.cfg.model_copy(), build_mesh("cpu", (2, 1), ("data", "model")))
    replica.load_full_state_dict(full.full_state_dict())
    e1, e2 = FusedCrosscoderStep(single, list_width=F), FusedCrosscoderStep(replica, list_width=F)
    g = torch.Generator().manual_seed(4)
    r, half = dist.get_rank(), B // 2
    for _ in range(3):
        x = (torch.randn(B, H, d, generator=g) * 1.5).to(torch.bfloat16)
        a = e1.step(x, lr, l1_coefficient=l1, sparsity_loss_type="tanh-quad", frequency_scale=scale)
        b = e2.step(x[r * half : (r + 1) * half], lr, l1_coefficient=l1, sparsity_loss_type="tanh-quad", frequency_scale=scale)
        assert torch.allclose(a, b, rtol=1e-4), (a, b)  # the frequencies are those of the whole batch on every replica
    for (name, p), (_, q) in zip(single.named_parameters(), replica.named_parameters()):
        assert torch.allclose(p.data, q.data, atol=2e-6), name
    dist.barrier()


def test_tanh_quad_penalty_with_replicas_matches_one_process():
    from language_model_saes_b200.testing import distributed_test

    distributed_test(nproc_per_node=2, backend="gloo")(_quad_replica_body)()


def test_trainer_takes_the_fused_step_for_tanh_quad_only_on_request(monkeypatch, tmp_path):
    from language_model_saes_b200.trainer import TrainerConfig

    m = _model("cpu", 2, 64, 256)
    cfg = TrainerConfig(total_training_tokens=10, exp_result_path=str(tmp_path), n_checkpoints=0, sparsity_loss_type="tanh-quad", l1_coefficient=0.3)
    monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True))  # only "is it on a GPU" is answered for the model
    monkeypatch.delenv("LMSAE_FUSED_TANH_QUAD", raising=False)
    ok, why = FusedCrosscoderStep.supports(m, cfg)
    assert not ok and "tanh-quad" in why
    monkeypatch.setenv("LMSAE_FUSED_TANH_QUAD", "1")
    assert FusedCrosscoderStep.supports(m, cfg) == (True, "")
    cfg.sparsity_loss_type = "power"
    assert not FusedCrosscoderStep.supports(m, cfg)[0]


def _head_parallel_body(penalty: str, lp: float, dims=(2, 1, 1)):
    """Heads over the ``head`` ranks (and tokens over ``data`` ranks when there are any) against ONE process holding all
    heads and the whole batch: the sum over heads of the pre-activations, the frequencies of the tanh-quad penalty and the
    shared thresholds' gradient cross ranks."""
    import torch.distributed as dist

    from language_model_saes_b200.parallel.mesh import DimMap, build_mesh

    H, d, F, B, lr, l1, scale = 4, 64, 256, 128, 1e-3, 5e-2, 0.05
    full = _model("cpu", H, d, F)
    single = copy.deepcopy(full)
    mesh = build_mesh("cpu", dims, ("head", "data", "model"))
    sharded = Crosscoder(full.cfg.model_copy(), mesh)
    sharded.load_full_state_dict(full.full_state_dict())
    e1, e2 = FusedCrosscoderStep(single, list_width=F), FusedCrosscoderStep(sharded, list_width=F)
    hp, dp = dims[0], dims[1]
    assert e2.head_size == hp and e2.dp == dp and e2.H_l == H // hp
    hr, dr = mesh.get_local_rank("head"), mesh.get_local_rank("data")
    per, rows = H // hp, B // dp
    g = torch.Generator().manual_seed(7)
    kw = dict(l1_coefficient=l1, sparsity_loss_type=penalty, frequency_scale=scale, lp_coefficient=lp)
    for _ in range(3):
        x = (torch.randn(B, H, d, generator=g) * 1.5).to(torch.bfloat16)
        want = e1.step(x, lr, **kw)
        mine = x[dr * rows : (dr + 1) * rows, hr * per : (hr + 1) * per].contiguous()
        e2.step(mine, lr, **kw)
        # reconstruction loss: mean over tokens and this rank's heads -> mean over the head ranks is the single-process value
        l_rec = e2.last["l_rec"].clone()
        dist.all_reduce(l_rec, group=mesh.get_group("head"))
        assert torch.allclose(l_rec / hp, e1.last["l_rec"], rtol=1e-4), (l_rec / hp, e1.last["l_rec"])
        assert torch.allclose(e1.last["l0"], e2.last["l0"])
        if penalty == "tanh-quad":
            assert torch.allclose(e1.last["l_s"], e2.last["l_s"], rtol=1e-4)  # one global figure
        assert torch.isfinite(want)
    for name in ("W_D", "W_E", "b_E", "b_D"):
        whole = DimMap({"head": 0}).gather(getattr(sharded, name).data, mesh)
        assert torch.allclose(whole, getattr(single, name).data, atol=5e-6), name
    a, b = single.activation_function.log_jumprelu_threshold.data, sharded.activation_function.log_jumprelu_threshold.data
    assert torch.allclose(a, b, atol=5e-6)
    dist.barrier()


def _heads_tanh_lp_body():
    _head_parallel_body("tanh", 2e-3)


def _heads_quad_body():
    _head_parallel_body("tanh-quad", 0.0)


def _heads_and_replicas_body():
    _head_parallel_body("tanh-quad", 0.0, dims=(2, 2, 1))


@pytest.mark.parametrize("body", ["_heads_tanh_lp_body", "_heads_quad_body"])
def test_fused_crosscoder_step_with_heads_over_two_ranks_matches_one_process(body):
    from language_model_saes_b200.testing import distributed_test

    distributed_test(nproc_per_node=2, backend="gloo")(globals()[body])()


def test_fused_crosscoder_step_with_heads_and_replicas_on_four_ranks_matches_one_process():
    from language_model_saes_b200.testing import distributed_test

    distributed_test(nproc_per_node=4, backend="gloo")(_heads_and_replicas_body)()


def _sae_shards_body():
    """A JumpReLU SAE (tanh-quad penalty and the pre-activation penalty) with its features over two ranks against one process."""
    import torch.distributed as dist

    from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
    from language_model_saes_b200.parallel.mesh import DimMap, build_mesh

    d, F, B, lr = 64, 256, 96, 1e-3
    torch.manual_seed(0)
    cfg = SAEConfig(hook_point_in="h", hook_point_out="h", d_model=d, expansion_factor=F / d, act_fn="jumprelu", device="cpu", dtype=torch.float32,
                    norm_activation="inference")  # fmt: skip
    full = SparseAutoEncoder(cfg)
    full.init_parameters(encoder_uniform_bound=0.2, decoder_uniform_bound=0.2, init_log_jumprelu_threshold_value=-1.0)
    full.set_decoder_to_fixed_norm(1.0, True)
    full.init_encoder_with_decoder_transpose()
    single = copy.deepcopy(full)
    mesh = build_mesh("cpu", (1, 2), ("data", "model"))
    shard = SparseAutoEncoder(cfg.model_copy(), mesh)
    shard.load_full_state_dict(full.full_state_dict())
    e1, e2 = FusedCrosscoderStep(single, list_width=F), FusedCrosscoderStep(shard, list_width=F // 2)
    assert e2.tp == 2 and e2.F == F // 2 and e2.single
    g = torch.Generator().manual_seed(3)
    basis = torch.randn(10, d, generator=g)
    kw = dict(l1_coefficient=5e-2, sparsity_loss_type="tanh-quad", frequency_scale=0.05)
    for step in range(3):
        x = torch.randn(B, 10, generator=g) @ basis + 0.05 * torch.randn(B, d, generator=g)
        x = (x * (d**0.5 / x.norm(dim=-1).mean())).to(torch.bfloat16).unsqueeze(1)
        extra = dict(lp_coefficient=2e-3) if step == 2 else {}
        a, b = e1.step(x, lr, **kw, **extra), e2.step(x, lr, **kw, **extra)
        assert torch.allclose(a, b, rtol=1e-4), (a, b)
        for key in ("l_rec", "l_s", "l_p", "l0"):
            assert torch.allclose(e1.last[key].float(), e2.last[key].float(), rtol=1e-4, atol=1e-7), key
    maps = shard.dim_maps()
    for name, p in single.named_parameters():
        q = dict(shard.named_parameters())[name].data
        whole = maps[name].gather(q, mesh) if name in maps else q
        assert torch.allclose(whole, p.data, atol=5e-6), name
    dist.barrier()


def test_jumprelu_sae_with_feature_shards_matches_one_process():
    from language_model_saes_b200.testing import distributed_test

    distributed_test(nproc_per_node=2, backend="gloo")(_sae_shards_body)()


def _heads_and_shards_body():
    """Crosscoder: heads over two ranks x features over two ranks."""
    import torch.distributed as dist

    from language_model_saes_b200.parallel.mesh import build_mesh

    H, d, F, B, lr = 4, 64, 256, 96, 1e-3
    full = _model("cpu", H, d, F)
    single = copy.deepcopy(full)
    mesh = build_mesh("cpu", (2, 1, 2), ("head", "data", "model"))
    sharded = Crosscoder(full.cfg.model_copy(), mesh)
    sharded.load_full_state_dict(full.full_state_dict())
    e1, e2 = FusedCrosscoderStep(single, list_width=F), FusedCrosscoderStep(sharded, list_width=F // 2)
    assert e2.head_size == 2 and e2.tp == 2 and e2.H_l == 2 and e2.F == F // 2
    hr = mesh.get_local_rank("head")
    g = torch.Generator().manual_seed(7)
    kw = dict(l1_coefficient=3e-2, sparsity_loss_type="tanh")
    for _ in range(3):
        x = (torch.randn(B, H, d, generator=g) * 1.5).to(torch.bfloat16)
        e1.step(x, lr, **kw)
        e2.step(x[:, 2 * hr : 2 * hr + 2].contiguous(), lr, **kw)
        l_rec = e2.last["l_rec"].clone()
        dist.all_reduce(l_rec, group=mesh.get_group("head"))
        assert torch.allclose(l_rec / 2, e1.last["l_rec"], rtol=1e-4)
        assert torch.allclose(e1.last["l0"].float(), e2.last["l0"].float())
    maps = sharded.dim_maps()
    for name, p in single.named_parameters():
        whole = maps[name].gather(dict(sharded.named_parameters())[name].data, mesh)
        assert torch.allclose(whole, p.data, atol=5e-6), name
    dist.barrier()


def test_fused_crosscoder_step_with_heads_and_feature_shards_on_four_ranks_matches_one_process():
    from language_model_saes_b200.testing import distributed_test

    distributed_test(nproc_per_node=4, backend="gloo")(_heads_and_shards_body)()
