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


from language_model_saes_b200.testing import distributed_test  # noqa: E402


@distributed_test(nproc_per_node=2, backend="gloo")
def test_fused_clt_step_with_feature_shards_matches_one_process():
    """Features split over two gloo ranks: per-layer top-k merged over the shards from one exchange of all layers' lists,
    partial reconstructions summed over the shards; same losses and weights as the unsharded step."""
    import torch.distributed as dist

    from language_model_saes_b200.parallel.mesh import DimMap, build_mesh

    L, d, F, k, B, lr, steps = 3, 64, 256, 8, 64, 1e-3, 3
    full = _model("cpu", L, d, F, k, True)
    mesh = build_mesh("cpu", (1, 2), ("data", "model"))
    single = copy.deepcopy(full)
    sharded = CrossLayerTranscoder(full.cfg.model_copy(), mesh)
    sharded.load_full_state_dict(full.full_state_dict())
    e1, e2 = FusedCLTStep(single), FusedCLTStep(sharded)
    g = torch.Generator().manual_seed(1)
    for _ in range(steps):
        x = torch.randn(B, L, d, generator=g).to(torch.bfloat16)
        y = torch.randn(L, B, d, generator=g).to(torch.bfloat16)
        a, b = e1.step(x, y, k, lr), e2.step(x, y, k, lr)
        assert torch.allclose(a, b, rtol=1e-4), (a, b)
    # The partial reconstructions add up in another order than in one process; where that flips a bf16 rounding of the output
    # gradient, Adam's first steps (which normalise away the gradient's size) move a few weights by up to lr per step.
    def close(a, b):
        diff = (a - b).abs()
        return float(diff.mean()) < 2e-6 and float(diff.max()) <= 2.2 * lr * steps

    for t in range(L):
        assert close(DimMap({"model": 1}).gather(sharded.W_D[t].data, mesh), single.W_D[t].data), t
    assert close(DimMap({"model": 2}).gather(sharded.W_E.data, mesh), single.W_E.data)
    dist.barrier()


@distributed_test(nproc_per_node=2, backend="gloo")
def test_fused_clt_step_with_replicas_matches_one_process():
    """Tokens split over two gloo ranks: each replica encodes and decodes its own half, then both rebuild the same sparse
    updates from the gathered codes; same losses and weights as one process on the whole batch."""
    import torch.distributed as dist

    from language_model_saes_b200.parallel.mesh import build_mesh

    L, d, F, k, B, lr, steps = 3, 64, 256, 8, 64, 1e-3, 3
    full = _model("cpu", L, d, F, k, True)
    mesh = build_mesh("cpu", (2, 1), ("data", "model"))
    single = copy.deepcopy(full)
    replica = CrossLayerTranscoder(full.cfg.model_copy(), mesh)
    replica.load_full_state_dict(full.full_state_dict())
    e1, e2 = FusedCLTStep(single), FusedCLTStep(replica)
    assert e2.dp == 2
    r, half = dist.get_rank(), B // 2
    g = torch.Generator().manual_seed(1)
    for _ in range(steps):
        x = torch.randn(B, L, d, generator=g).to(torch.bfloat16)
        y = torch.randn(L, B, d, generator=g).to(torch.bfloat16)
        a = e1.step(x, y, k, lr)
        b = e2.step(x[r * half : (r + 1) * half], y[:, r * half : (r + 1) * half], k, lr)
        assert torch.allclose(a, b, rtol=1e-4), (a, b)
    for t in range(L):
        assert torch.allclose(replica.W_D[t].data, single.W_D[t].data, atol=1e-6), t
        assert torch.allclose(replica.b_D[t].data, single.b_D[t].data, atol=1e-6), t
    assert torch.allclose(replica.W_E.data, single.W_E.data, atol=1e-6)
    assert torch.allclose(replica.b_E.data, single.b_E.data, atol=1e-6)
    dist.barrier()


@distributed_test(nproc_per_node=4, backend="gloo")
def test_fused_clt_step_with_feature_shards_and_replicas_on_four_ranks_matches_one_process():
    import torch.distributed as dist

    from language_model_saes_b200.parallel.mesh import DimMap, build_mesh

    L, d, F, k, B, lr, steps = 3, 64, 256, 8, 64, 1e-3, 3
    full = _model("cpu", L, d, F, k, True)
    mesh = build_mesh("cpu", (2, 2), ("data", "model"))
    single = copy.deepcopy(full)
    sharded = CrossLayerTranscoder(full.cfg.model_copy(), mesh)
    sharded.load_full_state_dict(full.full_state_dict())
    e1, e2 = FusedCLTStep(single), FusedCLTStep(sharded)
    assert e2.tp == 2 and e2.dp == 2
    dr, half = mesh.get_local_rank("data"), B // 2
    g = torch.Generator().manual_seed(1)
    for _ in range(steps):
        x = torch.randn(B, L, d, generator=g).to(torch.bfloat16)
        y = torch.randn(L, B, d, generator=g).to(torch.bfloat16)
        a = e1.step(x, y, k, lr)
        b = e2.step(x[dr * half : (dr + 1) * half], y[:, dr * half : (dr + 1) * half], k, lr)
        assert torch.allclose(a, b, rtol=1e-4), (a, b)

    def close(a, b):  # see the feature-shard test: a flipped bf16 rounding moves a few weights by up to lr per step
        diff = (a - b).abs()
        return float(diff.mean()) < 2e-6 and float(diff.max()) <= 2.2 * lr * steps

    for t in range(L):
        assert close(DimMap({"model": 1}).gather(sharded.W_D[t].data, mesh), single.W_D[t].data), t
    assert close(DimMap({"model": 2}).gather(sharded.W_E.data, mesh), single.W_E.data)
    dist.barrier()


def _layertopk_model(k=12, gate=True):
    m = _model("cpu", 3, 64, 256, k, gate)
    m.cfg.act_fn = "layertopk"
    m.activation_function = m.activation_function_factory(m.device_mesh)
    return m


@pytest.mark.parametrize("gate", [True, False])
def test_fused_clt_step_with_layertopk_matches_autograd(gate, monkeypatch):
    """k codes per token over all layers together (not k per layer): selection, losses and parameters against the model."""
    L, d, F, k, B, lr, steps = 3, 64, 256, 12, 96, 1e-3, 4
    ref = _layertopk_model(k, gate)
    start = {n: p.detach().clone() for n, p in ref.named_parameters()}
    fused_model = copy.deepcopy(ref)
    monkeypatch.delenv("LMSAE_FUSED_LAYERTOPK", raising=False)
    assert not FusedCLTStep.supports(fused_model)[0]  # on request only, until it has run on a GPU
    monkeypatch.setenv("LMSAE_FUSED_LAYERTOPK", "1")
    assert FusedCLTStep.supports(fused_model)[0]
    engine = FusedCLTStep(fused_model)
    g = torch.Generator().manual_seed(1)
    basis = torch.randn(6, d, generator=g)
    opt = torch.optim.Adam(ref.parameters(), lr=lr)
    tokens = torch.zeros(B, dtype=torch.long)
    for step in range(steps):
        z = torch.randn(B, 6, generator=g)
        x = torch.stack([z @ basis * (1 + 0.1 * l) + 0.2 * torch.randn(B, d, generator=g) for l in range(L)], dim=1).to(torch.bfloat16)
        y = torch.stack([(z @ basis).roll(l + 1, dims=-1) + 0.2 * torch.randn(B, d, generator=g) for l in range(L)], dim=0).to(torch.bfloat16)
        batch = {h: x[:, l].float() for l, h in enumerate(ref.cfg.hook_points_in)} | {h: y[l].float() for l, h in enumerate(ref.cfg.hook_points_out)}
        batch["tokens"] = tokens
        opt.zero_grad()
        out = ref.compute_loss(batch, return_aux_data=True)
        if step == 0:  # the two models are still the same: the same codes, k per token in all, spread unevenly over the layers
            idx, act = engine.encode(x, k)
            assert idx.shape == (B, k)
            dense = torch.zeros(B, L * F)
            dense.scatter_(1, idx.clamp_min(0).long(), torch.where(idx >= 0, act, torch.zeros_like(act)))
            want = out["feature_acts"].detach().reshape(B, L * F)
            both = (dense != 0) & (want != 0)
            # (the engine's weights are rounded to bf16: a near-tie at the k-th place may fall the other way)
            assert int(((dense != 0) != (want != 0)).sum()) <= 0.02 * B * k
            assert torch.allclose(dense[both], want[both], atol=5e-2, rtol=2e-2)
            assert int((want != 0).sum(-1).max()) <= k and len(set((want.view(B, L, F) != 0).sum(-1).reshape(-1).tolist())) > 2
        out["loss"].backward()
        opt.step()
        got = engine.step(x, y, k, lr)
        assert torch.allclose(out["loss"].detach(), got, rtol=2e-3), (out["loss"], got)
    for name, p in ref.named_parameters():
        a, b = p.detach().float(), dict(fused_model.named_parameters())[name].detach().float()
        moved = (a - start[name].float()).abs().mean()
        assert float((a - b).abs().mean()) < 0.05 * float(moved) + 1e-7, name


@distributed_test(nproc_per_node=2, backend="gloo")
def test_fused_clt_step_with_layertopk_and_feature_shards_matches_one_process():
    import os

    import torch.distributed as dist

    from language_model_saes_b200.parallel.mesh import DimMap, build_mesh

    os.environ["LMSAE_FUSED_LAYERTOPK"] = "1"
    L, d, F, k, B, lr, steps = 3, 64, 256, 12, 64, 1e-3, 3
    full = _layertopk_model(k)
    mesh = build_mesh("cpu", (1, 2), ("data", "model"))
    single = copy.deepcopy(full)
    sharded = CrossLayerTranscoder(full.cfg.model_copy(), mesh)
    sharded.load_full_state_dict(full.full_state_dict())
    e1, e2 = FusedCLTStep(single), FusedCLTStep(sharded)
    assert e2.joint and e2.tp == 2
    g = torch.Generator().manual_seed(1)
    for _ in range(steps):
        x = torch.randn(B, L, d, generator=g).to(torch.bfloat16)
        y = torch.randn(L, B, d, generator=g).to(torch.bfloat16)
        i1, _ = e1.encode(x, k)
        i2, _ = e2.encode(x, k)
        n_mine = (i2 >= 0).sum().reshape(1)
        dist.all_reduce(n_mine)
        assert int(n_mine) == int((i1 >= 0).sum())  # the shards' kept codes add up to the single-process selection
        a, b = e1.step(x, y, k, lr), e2.step(x, y, k, lr)
        assert torch.allclose(a, b, rtol=1e-4), (a, b)

    def close(a, b):
        diff = (a - b).abs()
        return float(diff.mean()) < 2e-6 and float(diff.max()) <= 2.2 * lr * steps

    for t in range(L):
        assert close(DimMap({"model": 1}).gather(sharded.W_D[t].data, mesh), single.W_D[t].data), t
    assert close(DimMap({"model": 2}).gather(sharded.W_E.data, mesh), single.W_E.data)
    dist.barrier()


def _batch_level_model(act, k=6, gate=True):
    m = _model("cpu", 3, 64, 256, k, gate)
    m.cfg.act_fn = act
    m.activation_function = m.activation_function_factory(m.device_mesh)
    return m


@pytest.mark.parametrize("act", ["batchtopk", "batchlayertopk"])
def test_fused_clt_step_with_batch_level_selection_matches_autograd(act, monkeypatch):
    """k x batch codes per layer (batchtopk) or over all layers together (batchlayertopk), rows of uneven width."""
    L, d, F, k, B, lr, steps = 3, 64, 256, 6, 96, 1e-3, 4
    monkeypatch.setenv("LMSAE_FUSED_LAYERTOPK", "1")
    if act == "batchlayertopk":  # this toy data puts most codes of the whole model on a few tokens: wider lists than 8 k
        monkeypatch.setenv("LMSAE_BATCH_LIST_FACTOR", "32")
    ref = _batch_level_model(act, k)
    start = {n: p.detach().clone() for n, p in ref.named_parameters()}
    fused_model = copy.deepcopy(ref)
    assert FusedCLTStep.supports(fused_model)[0]
    engine = FusedCLTStep(fused_model)
    g = torch.Generator().manual_seed(1)
    basis = torch.randn(6, d, generator=g)
    opt = torch.optim.Adam(ref.parameters(), lr=lr)
    tokens = torch.zeros(B, dtype=torch.long)
    for step in range(steps):
        z = torch.randn(B, 6, generator=g)
        x = torch.stack([z @ basis * (1 + 0.1 * l) + 0.2 * torch.randn(B, d, generator=g) for l in range(L)], dim=1).to(torch.bfloat16)
        y = torch.stack([(z @ basis).roll(l + 1, dims=-1) + 0.2 * torch.randn(B, d, generator=g) for l in range(L)], dim=0).to(torch.bfloat16)
        batch = {h: x[:, l].float() for l, h in enumerate(ref.cfg.hook_points_in)} | {h: y[l].float() for l, h in enumerate(ref.cfg.hook_points_out)}
        batch["tokens"] = tokens
        opt.zero_grad()
        out = ref.compute_loss(batch, return_aux_data=True)
        if step == 0:
            idx, act_v = engine.encode(x, k)
            want = out["feature_acts"].detach().reshape(B, L * F)
            per_layer = (want.view(B, L, F) != 0).sum((0, 2))
            assert int((idx >= 0).sum()) == int((want != 0).sum()) == k * B * (1 if act == "batchlayertopk" else L)
            if act == "batchtopk":
                assert per_layer.tolist() == [k * B] * L
            assert len(set((want != 0).sum(-1).tolist())) > 3  # rows of uneven width
            dense = torch.zeros(B, L * F)
            dense.scatter_(1, idx.clamp_min(0).long(), torch.where(idx >= 0, act_v, torch.zeros_like(act_v)))
            assert int(((dense != 0) != (want != 0)).sum()) <= 0.02 * int((want != 0).sum())
        out["loss"].backward()
        opt.step()
        got = engine.step(x, y, k, lr)
        assert torch.allclose(out["loss"].detach(), got, rtol=3e-3), (out["loss"], got)
    assert int(engine.list_overflow) == 0
    for name, p in ref.named_parameters():
        a, b = p.detach().float(), dict(fused_model.named_parameters())[name].detach().float()
        moved = (a - start[name].float()).abs().mean()
        assert float((a - b).abs().mean()) < 0.06 * float(moved) + 1e-7, name


@distributed_test(nproc_per_node=2, backend="gloo")
def test_fused_clt_step_with_batchtopk_and_feature_shards_matches_one_process():
    import os

    import torch.distributed as dist

    from language_model_saes_b200.parallel.mesh import build_mesh

    os.environ["LMSAE_FUSED_LAYERTOPK"] = "1"
    L, d, F, k, B, lr = 3, 64, 256, 6, 64, 1e-3
    for act in ("batchtopk", "batchlayertopk"):
        full = _batch_level_model(act, k)
        mesh = build_mesh("cpu", (1, 2), ("data", "model"))
        single = copy.deepcopy(full)
        sharded = CrossLayerTranscoder(full.cfg.model_copy(), mesh)
        sharded.load_full_state_dict(full.full_state_dict())
        e1, e2 = FusedCLTStep(single), FusedCLTStep(sharded)
        g = torch.Generator().manual_seed(1)
        for _ in range(3):
            x = torch.randn(B, L, d, generator=g).to(torch.bfloat16)
            y = torch.randn(L, B, d, generator=g).to(torch.bfloat16)
            i1, _ = e1.encode(x, k)
            i2, _ = e2.encode(x, k)
            n_mine = (i2 >= 0).sum().reshape(1)
            dist.all_reduce(n_mine)
            assert int(n_mine) == int((i1 >= 0).sum()), act  # exactly k x batch codes (per layer) over the shards together
            a, b = e1.step(x, y, k, lr), e2.step(x, y, k, lr)
            # entries EQUAL to the (bf16) threshold are granted in (shard, row, column) order: with shards a handful of the
            # k x batch codes are other, equally large, entries than in one process
            assert torch.allclose(a, b, rtol=2e-3), (act, a, b)
    dist.barrier()
