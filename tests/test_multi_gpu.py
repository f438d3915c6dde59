"""Feature-sharded fused step on 2 GPUs: peer-memory kernels vs NCCL collectives vs one GPU; and the bounded
wait of the peer-flag kernels (a flag that nothing sets must end in a status code, not a hang)."""

import os

import pytest
import torch
import torch.distributed as dist

from language_model_saes_b200.testing import distributed_test

pytestmark = pytest.mark.gpu

needs2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")


def _full_model(dev, d=256, F=4096, k=16):
    from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder

    torch.manual_seed(0)
    cfg = SAEConfig(hook_point_in="h", hook_point_out="h", d_model=d, expansion_factor=F / d, act_fn="topk", top_k=k,
                    device=str(dev), dtype=torch.float32)  # fmt: skip
    sae = SparseAutoEncoder(cfg)
    sae.init_parameters(encoder_uniform_bound=0.06, decoder_uniform_bound=0.06)
    sae.set_decoder_to_fixed_norm(0.7, True)
    sae.init_encoder_with_decoder_transpose()
    sae.set_dataset_average_activation_norm({"h": d**0.5})
    return sae


@needs2
@distributed_test(nproc_per_node=2, backend="nccl")
def test_peer_memory_step_matches_nccl_and_single_gpu():
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from language_model_saes_b200.models.sae import SparseAutoEncoder
    from language_model_saes_b200.ops import sae_kernels as K
    from language_model_saes_b200.ops.fused_step import FusedTopKSAEStep
    from language_model_saes_b200.parallel.mesh import DimMap, build_mesh
    from language_model_saes_b200.parallel.symm import SymmComm

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    mesh = build_mesh("cuda", (1, 2), ("data", "model"))
    full = _full_model(dev)
    B, d, k, lr = 512, 256, 16, 1e-3
    g = torch.Generator(device=dev).manual_seed(3)
    xs = [(torch.randn(B, d, device=dev, generator=g) * 1.0).to(torch.bfloat16) for _ in range(4)]
    for x in xs:
        dist.broadcast(x, src=0)

    def run(model, comm):
        eng = FusedTopKSAEStep(model, comm=comm, overlap_chunks=2)
        out = torch.stack([eng.step(x, x, k, lr) for x in xs])
        eng.join()
        return out

    single = SparseAutoEncoder(full.cfg.model_copy())
    single.load_full_state_dict(full.full_state_dict())
    want = run(single, None)

    def shard():
        m = SparseAutoEncoder(full.cfg.model_copy(), mesh)
        m.load_full_state_dict(full.full_state_dict())
        return m

    m_nccl = shard()
    got_nccl = run(m_nccl, None)
    assert torch.allclose(got_nccl, want, rtol=2e-3), (got_nccl, want)
    W_ref = single.W_D.data
    W = DimMap({"model": 0}).gather(m_nccl.W_D.data, mesh)
    assert torch.allclose(W, W_ref, atol=2e-4), float((W - W_ref).abs().max())
    # peer-memory variants: fp32 partial rows (exact protocol check), bf16 partial rows (the default on the wire) and, where
    # the fabric offers a multicast mapping, the owner-side sum and the gradient all-gather through the switch
    variants = [("fp32", dict(partial_dtype=torch.float32, use_multicast=False), 2e-3, 2e-4),
                ("bf16", dict(partial_dtype=torch.bfloat16, use_multicast=False), 1e-2, None),
                ("multicast", dict(partial_dtype=torch.bfloat16, use_multicast=True), 1e-2, None)]  # fmt: skip
    for name, kw, rtol, w_atol in variants:
        comm = SymmComm(mesh.get_group("model"), dev, B, k, d, **kw)
        if name == "multicast" and not comm.use_multicast:
            print("no multicast mapping for this group: the multimem variant is not exercised here")
            continue
        m_p2p = shard()
        got_p2p = run(m_p2p, comm)
        K.check_status(dev)
        # the peer-memory path reports the loss of the rows each rank owns: average the two halves
        dist.all_reduce(got_p2p)
        got_p2p /= 2
        assert torch.allclose(got_p2p, want, rtol=rtol), (name, got_p2p, want)
        W = DimMap({"model": 0}).gather(m_p2p.W_D.data, mesh)
        if w_atol is not None:
            assert torch.allclose(W, W_ref, atol=w_atol), (name, float((W - W_ref).abs().max()))
        else:  # partial rows rounded to bf16: Adam's first steps move a weight by about lr whatever the gradient's size
            assert float((W - W_ref).abs().max()) <= 2.2 * lr * len(xs), (name, float((W - W_ref).abs().max()))
        waits = comm.stats.read(1500.0)
        assert set(waits) == {"candidates", "partial rows", "gradient rows"} and all(v["calls"] == len(xs) for v in waits.values()), waits
        # codes outside a training step, twice (metrics path): the candidate exchange alone, on its alternating zones
        eng_a, eng_b = FusedTopKSAEStep(m_p2p, comm=comm), FusedTopKSAEStep(m_p2p, comm=None)
        for x in xs[:2]:
            ia, aa, xa = eng_a.forward_dense(x, k)
            ib, ab, xb = eng_b.forward_dense(x, k)
            K.check_status(dev)
            assert torch.equal(ia.sort(dim=1).values, ib.sort(dim=1).values), name
            assert torch.allclose(xa, xb, atol=1e-3, rtol=1e-3), name
        # debug layouts (bounds-checked build or LMSAE_BUFFER_GUARDS=1): nothing wrote past a region of the step buffers
        dist.barrier()
        comm.check_guards()


@needs2
@distributed_test(nproc_per_node=2, backend="nccl")
def test_data_parallel_step_with_row_sharded_optimizer_state_matches_single_gpu():
    """Two replicas, each with half of the batch: rows exchanged by one peer-store kernel, each replica updates half of
    the feature rows and publishes the new bf16 rows, norms and biases to the other. Same losses and, after gathering
    the master rows, the same parameters and Adam moments as one GPU on the whole batch."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from language_model_saes_b200.models.sae import SparseAutoEncoder
    from language_model_saes_b200.ops import sae_kernels as K
    from language_model_saes_b200.ops.fused_step import FusedTopKSAEStep
    from language_model_saes_b200.parallel.mesh import build_mesh
    from language_model_saes_b200.parallel.symm import DataParallelComm

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    mesh = build_mesh("cuda", (2, 1), ("data", "model"))
    full = _full_model(dev)
    B, d, k, lr, F = 512, 256, 16, 1e-3, 4096
    g = torch.Generator(device=dev).manual_seed(3)
    xs = [(torch.randn(B, d, device=dev, generator=g) * 1.0).to(torch.bfloat16) for _ in range(4)]
    for x in xs:
        dist.broadcast(x, src=0)
    single = SparseAutoEncoder(full.cfg.model_copy())
    single.load_full_state_dict(full.full_state_dict())
    eng1 = FusedTopKSAEStep(single)
    want = torch.stack([eng1.step(x, x, k, lr, clip_grad_norm=(0.5 if i == 3 else 0.0)) for i, x in enumerate(xs)])

    half = B // 2
    for sharded in (True, False):
        m = SparseAutoEncoder(full.cfg.model_copy(), mesh)
        m.load_full_state_dict(full.full_state_dict())
        dp_comm = None
        if sharded:
            n = B
            zones = {"x": n * d * 2, "dxhat": n * d * 2, "idx": n * k * 4, "act": n * k * 4, "dact": n * k * 4}
            dp_comm = DataParallelComm(mesh.get_group("data"), dev, F, d, zones)
        eng = FusedTopKSAEStep(m, dp_comm=dp_comm)
        got = torch.stack([eng.step(x[rank * half : (rank + 1) * half], x[rank * half : (rank + 1) * half], k, lr,
                                    clip_grad_norm=(0.5 if i == 3 else 0.0)) for i, x in enumerate(xs)])  # fmt: skip
        K.check_status(dev)
        dist.all_reduce(got)
        got /= 2  # each replica reports the mean loss of its half of the batch
        assert torch.allclose(got, want, rtol=2e-3), (sharded, got, want)
        eng.sync_params()
        assert torch.allclose(m.W_D.data, single.W_D.data, atol=2e-4), (sharded, float((m.W_D.data - single.W_D.data).abs().max()))
        assert torch.allclose(m.W_E.data, single.W_E.data, atol=2e-4)
        assert torch.allclose(m.b_E.data, single.b_E.data, atol=2e-4) and torch.allclose(m.b_D.data, single.b_D.data, atol=2e-4)
        assert torch.allclose(eng.dec_norm, eng1.dec_norm, atol=2e-4)
        st, st1 = eng.optimizer_state(), eng1.optimizer_state()
        assert torch.allclose(st["W_D"]["exp_avg_sq"], st1["W_D"]["exp_avg_sq"], atol=1e-6, rtol=1e-2)
        if sharded:
            assert eng.state["W_D"][0].shape[0] == F // 2  # the moments of half of the rows only
            assert dp_comm.stats.read(1500.0)["data-parallel rows"]["calls"] == len(xs)

    # the same with the Aux-K loss: dead statistics over the global batch, auxiliary codes and their gradient rows exchanged too
    from language_model_saes_b200.ops.fused_step import AuxK

    k_aux = 32

    def run_aux(model, dp_comm, rows):
        eng = FusedTopKSAEStep(model, dp_comm=dp_comm)
        aux = AuxK(eng.F, k_aux=k_aux, coefficient=1 / 32, dead_threshold=B // 2, device=dev)
        out = []
        for x in xs[:3]:
            loss = eng.step(x[rows], x[rows], k, lr, aux=aux)
            out.append(torch.stack([loss, eng.last_aux_loss]))
        eng.sync_params()
        return eng, aux, torch.stack(out)

    single = SparseAutoEncoder(full.cfg.model_copy())
    single.load_full_state_dict(full.full_state_dict())
    _, aux1, want = run_aux(single, None, slice(0, B))
    assert float(want[:, 1].min()) > 0
    m = SparseAutoEncoder(full.cfg.model_copy(), mesh)
    m.load_full_state_dict(full.full_state_dict())
    n = B
    zones = {"x": n * d * 2, "dxhat": n * d * 2, "idx": n * k * 4, "act": n * k * 4, "dact": n * k * 4}
    _, aux2, got = run_aux(m, DataParallelComm(mesh.get_group("data"), dev, F, d, zones), slice(rank * half, (rank + 1) * half))
    K.check_status(dev)
    dist.all_reduce(got)
    got /= 2
    assert torch.allclose(got, want, rtol=3e-3), (got, want)
    assert torch.equal(aux2.tokens_since_last_activation, aux1.tokens_since_last_activation)
    assert torch.allclose(m.W_D.data, single.W_D.data, atol=2e-4), float((m.W_D.data - single.W_D.data).abs().max())


@needs2
@distributed_test(nproc_per_node=2, backend="nccl")
def test_auxk_step_with_feature_shards_matches_single_gpu():
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from language_model_saes_b200.models.sae import SparseAutoEncoder
    from language_model_saes_b200.ops import sae_kernels as K
    from language_model_saes_b200.ops.fused_step import AuxK, FusedTopKSAEStep
    from language_model_saes_b200.parallel.mesh import DimMap, build_mesh
    from language_model_saes_b200.parallel.symm import SymmComm

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    mesh = build_mesh("cuda", (1, 2), ("data", "model"))
    full = _full_model(dev)
    B, d, k, lr = 512, 256, 16, 1e-3
    g = torch.Generator(device=dev).manual_seed(5)
    xs = [(torch.randn(B, d, device=dev, generator=g) * 1.0).to(torch.bfloat16) for _ in range(3)]
    for x in xs:
        dist.broadcast(x, src=0)

    def run(model, comm, k_aux):
        eng = FusedTopKSAEStep(model, comm=comm)
        aux = AuxK(eng.F, k_aux=k_aux, coefficient=1 / 32, dead_threshold=B // 2, device=dev)  # dead = did not fire in the step
        out = []
        for x in xs:
            loss = eng.step(x, x, k, lr, aux=aux)
            out.append(torch.stack([loss, eng.last_aux_loss]))
        return torch.stack(out)

    for k_aux in (32, 96):  # 96: lists longer than the merge kernel's, merged with the plain-torch statement
        single = SparseAutoEncoder(full.cfg.model_copy())
        single.load_full_state_dict(full.full_state_dict())
        want = run(single, None, k_aux)
        assert float(want[:, 1].min()) > 0
        for use_comm in (False, True):
            m = SparseAutoEncoder(full.cfg.model_copy(), mesh)
            m.load_full_state_dict(full.full_state_dict())
            got = run(m, SymmComm(mesh.get_group("model"), dev, B, k, d) if use_comm else None, k_aux)
            K.check_status(dev)
            assert torch.allclose(got, want, rtol=3e-3), (k_aux, use_comm, got, want)
            W = DimMap({"model": 0}).gather(m.W_D.data, mesh)
            off = ((W - single.W_D.data).abs() > 2e-4).any(dim=1).float().mean()
            # k_aux > 64 selects on pre-activations stored in bf16, where equal values are common: which of several
            # equal candidates gets the last places depends on how the lists were split. The losses above agree (equal
            # values contribute equally), but Adam's first steps move every row that got any gradient by about lr, so
            # rows whose tied features differ end up lr apart: bounded by the steps taken, not by a rounding tolerance.
            if k_aux <= 64:
                assert float(off) == 0.0, (k_aux, use_comm, float(off))
            else:
                assert float((W - single.W_D.data).abs().max()) <= 2.2 * lr * len(xs), (k_aux, use_comm)


def test_peer_flag_wait_times_out_with_status_code():
    from language_model_saes_b200.ops import sae_kernels as K

    from language_model_saes_b200.parallel.symm import peer_table

    dev = torch.device("cuda", 0)
    buf = torch.zeros(4096, dtype=torch.uint8, device=dev)
    table = peer_table(1, 0, [buf.data_ptr()], 0, 1024, 2048, 3072, 3584)
    st = K.status_buffer(dev)
    st.zero_()
    K._ext().comm_wait(table, 0, 7, st)  # epoch 7 was never published
    torch.cuda.synchronize()
    # while the error is on record the update kernels leave parameters and moments alone
    p, g = torch.ones(64, device=dev), torch.ones(64, device=dev)
    m, v = torch.zeros(64, device=dev), torch.zeros(64, device=dev)
    K.adam_flat(p, g, m, v, 0.1, 0.9, 0.999, 1e-8, 1)
    assert float(p.sum()) == 64.0 and float(m.abs().sum()) == 0.0
    with pytest.raises(K.KernelStatusError, match="peer flag"):
        K.check_status(dev)
    # the context is still usable afterwards, and with the status cleared the update runs
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0
    K.adam_flat(p, g, m, v, 0.1, 0.9, 0.999, 1e-8, 1)
    assert float(p.sum()) < 64.0


@needs2
@distributed_test(nproc_per_node=2, backend="nccl")
def test_shuffle_all_to_all_is_the_seeded_global_permutation():
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from language_model_saes_b200.activation.processors.activation import CrossRankShuffler
    from language_model_saes_b200.ops import sae_kernels as K
    from language_model_saes_b200.parallel.mesh import build_mesh
    from language_model_saes_b200.parallel.symm import ShuffleComm

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    mesh = build_mesh("cuda", (2, 1), ("data", "model"))
    n, d = 1000, 256
    comm = ShuffleComm(mesh.get_group("data"), dev, rows_per_rank=1024, max_row_bytes=d * 2)
    for call in range(3):  # three calls: both landing buffers and their re-use
        x = (torch.arange(n, device=dev)[:, None] + 10_000 * rank + 100_000 * call).expand(n, d).to(torch.bfloat16).contiguous()
        y = comm.shuffle(x, seed=7 + call)
        K.check_status(dev)
        both_x = [torch.empty_like(x) for _ in range(2)]
        both_y = [torch.empty_like(y) for _ in range(2)]
        dist.all_gather(both_x, x)
        dist.all_gather(both_y, y)
        X, Y = torch.cat(both_x), torch.cat(both_y)
        perm = comm.permutation(n, 7 + call).to(dev)
        want = torch.empty_like(X)
        want[perm] = X
        assert torch.equal(Y, want)

    # through the activation buffer: uneven buffers, a tensor with 8-byte rows
    shuf = CrossRankShuffler(mesh, seed=3, capacity_rows=64)
    m_local = 40 + 8 * rank
    data = {"h": torch.randn(m_local, 64, device=dev), "tokens": torch.arange(m_local, device=dev) + 1000 * rank}
    data["h"][:, 0] = data["tokens"].float()
    out = shuf(data)
    K.check_status(dev)
    assert out["h"].shape == data["h"].shape and out["tokens"].shape == data["tokens"].shape
    assert torch.equal(out["h"][:, 0], out["tokens"].float())  # rows travel whole, all tensors with the same permutation
    assert torch.equal(out["tokens"][40:], data["tokens"][40:])  # rows beyond the common length stay
    mixed = [torch.empty(40, dtype=torch.long, device=dev) for _ in range(2)]
    dist.all_gather(mixed, out["tokens"][:40].contiguous())
    assert sorted(torch.cat(mixed).tolist()) == sorted(list(range(40)) + list(range(1000, 1040)))
    assert (out["tokens"][:40] >= 1000).any() and (out["tokens"][:40] < 1000).any()


@needs2
@distributed_test(nproc_per_node=2, backend="nccl")
def test_peer_broadcast_of_masked_cast_rows_and_cached_loader():
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import tempfile
    from pathlib import Path

    from safetensors.torch import save_file

    from language_model_saes_b200.activation.processors.cached_activation import CachedActivationLoader
    from language_model_saes_b200.ops import sae_kernels as K
    from language_model_saes_b200.parallel.mesh import build_mesh
    from language_model_saes_b200.parallel.symm import BroadcastComm

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    mesh = build_mesh("cuda", (1, 2), ("data", "model"))
    group = mesh.get_group("model")
    n, d = 3000, 512
    g = torch.Generator(device="cpu").manual_seed(5)
    for use_mc in (False, True):  # peer stores, then one store per 16 bytes through the NVSwitch multicast mapping
        comm = BroadcastComm(group, dev, max_rows=n, max_row_bytes=d * 4, use_multicast=use_mc)
        if use_mc and not comm.use_multicast:
            print("no multicast mapping for this group: the multimem variant is not exercised here")
            continue
        for call in range(5):  # both landing zones, their re-use, and both ranks as the sender
            src = call % 2
            rows_cpu = torch.randn(n - 100 * call, d, generator=g)
            keep_cpu = torch.rand(n - 100 * call, generator=g) > 0.25
            use_mask, out_dtype = call % 3 != 2, (torch.bfloat16 if call % 2 == 0 else torch.float32)
            rows = rows_cpu.to(dev) if rank == src else None
            keep = keep_cpu.to(dev) if (rank == src and use_mask) else None
            got = comm.broadcast_rows(src, d, out_dtype, rows, keep)
            K.check_status(dev)
            want = (rows_cpu[keep_cpu] if use_mask else rows_cpu).to(out_dtype).to(dev)
            assert torch.equal(got, want), (use_mc, call, got.shape, want.shape)

    # the cached-activation loader: rank 0 of the model group reads, rank 1 receives the same records
    root = Path(tempfile.gettempdir()) / "lmsae_peer_bcast_cache"
    if rank == 0:
        for hp in ("h0", "h1"):
            (root / hp).mkdir(parents=True, exist_ok=True)
            for c in range(3):
                gg = torch.Generator().manual_seed(100 * c + (hp == "h1"))
                save_file({"activation": torch.randn(4, 16, 64, generator=gg).to(torch.bfloat16),
                           "tokens": torch.arange(64).view(4, 16) + 1000 * c, "mask": torch.ones(4, 16, dtype=torch.bool),
                           "attention_mask": torch.ones(4, 16, dtype=torch.bool)}, str(root / hp / f"chunk-{c}.safetensors"))  # fmt: skip
    dist.barrier()
    dirs = {hp: root / hp for hp in ("h0", "h1")}
    pushed = list(CachedActivationLoader(dirs, device=str(dev), device_mesh=mesh, peer_broadcast=True).process())
    plain = list(CachedActivationLoader(dirs, device=str(dev)).process())
    K.check_status(dev)
    assert len(pushed) == len(plain) == 3
    for a, b in zip(pushed, plain):
        assert set(a) == set(b)
        for key in b:
            assert torch.equal(a[key], b[key]) if isinstance(b[key], torch.Tensor) else a[key] == b[key]


@needs2
@distributed_test(nproc_per_node=2, backend="nccl")
def test_head_parallel_crosscoder_sums_pre_activations_with_the_all_reduce_kernel():
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    from language_model_saes_b200.models.crosscoder import Crosscoder, CrosscoderConfig
    from language_model_saes_b200.ops import sae_kernels as K
    from language_model_saes_b200.parallel.mesh import build_mesh
    from language_model_saes_b200.parallel.symm import HeadSumComm

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    mesh = build_mesh("cuda", (2, 1, 1), ("head", "data", "model"))
    group = mesh.get_group("head")

    # the collective alone: every rank contributes its own heads, all ranks get the total
    M, heads, d, N = 256, 2, 128, 1024
    torch.manual_seed(10 + rank)
    x = torch.randn(M, heads * d, device=dev).to(torch.bfloat16)
    w = (torch.randn(heads * N, d, device=dev) / d**0.5).to(torch.bfloat16)
    bias = torch.randn(N, device=dev)
    local = bias + sum(x[:, h * d : (h + 1) * d].float() @ w[h * N : (h + 1) * N].float().T for h in range(heads))
    want = local.clone()
    dist.all_reduce(want)
    comm = HeadSumComm(group, dev, max_rows=M, n_cols=N)
    for call in range(4):  # both buffers twice; the ranks' bf16 partial results are summed in fp32 and stored as bf16
        got = comm.head_sum(x, w, bias, heads, N, torch.float32)
        K.check_status(dev)
        assert torch.allclose(got, want, atol=4e-2, rtol=1e-2), (call, float((got - want).abs().max()))

    # the model: fused against the all-reduce path, values and gradients
    def make(fused):
        torch.manual_seed(0)
        cfg = CrosscoderConfig(hook_points=["a", "b", "c", "e"], d_model=128, expansion_factor=8, act_fn="relu", device="cuda",
                               dtype=torch.bfloat16, norm_activation="inference", fused_head_sum=fused)  # fmt: skip
        m = Crosscoder(cfg, device_mesh=mesh)
        m.init_parameters(encoder_uniform_bound=0.1, decoder_uniform_bound=0.1, init_log_jumprelu_threshold_value=0.0)
        with torch.no_grad():
            m.W_E.mul_(1 + 0.1 * (torch.arange(2, device=dev) + 2 * rank).view(2, 1, 1))
        return m

    a, b = make(True), make(False)
    torch.manual_seed(100 + rank)
    x = torch.randn(256, 2, 128, device=dev, dtype=torch.bfloat16)
    fa, ha = a.encode(x, return_hidden_pre=True)
    fb, hb = b.encode(x, return_hidden_pre=True)
    K.check_status(dev)
    assert torch.allclose(ha.float(), hb.float(), atol=5e-2, rtol=5e-2)
    g = torch.randn_like(fa)
    (fa * g).sum().backward()
    (fb * g).sum().backward()

    def close(u, v):
        return float((u.float() - v.float()).norm() / v.float().norm()) < 0.05

    assert close(a.W_E.grad, b.W_E.grad) and close(a.b_E.grad, b.b_E.grad)


@needs2
@distributed_test(nproc_per_node=2, backend="nccl")
def test_in_place_all_reduce_kernel_and_head_parallel_fused_crosscoder():
    """The one-kernel in-place all-reduce of a bf16 matrix (NVSwitch multicast loads / stores where the fabric offers a
    mapping, peer loads / stores otherwise), and the fused crosscoder step with its heads split over two ranks against the
    generic autograd path on the same mesh."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import copy

    from language_model_saes_b200.models.crosscoder import Crosscoder, CrosscoderConfig
    from language_model_saes_b200.ops import sae_kernels as K
    from language_model_saes_b200.ops.fused_crosscoder import FusedCrosscoderStep
    from language_model_saes_b200.parallel.mesh import build_mesh
    from language_model_saes_b200.parallel.symm import AllReduceComm

    rank = dist.get_rank()
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    mesh = build_mesh("cuda", (2, 1, 1), ("head", "data", "model"))
    group = mesh.get_group("head")
    # the one-kernel all-gather of several tensors (data-parallel row exchange), peer stores and multicast stores
    from language_model_saes_b200.parallel.symm import DataParallelComm

    for use_mc in (False, True):
        torch.manual_seed(3 + rank)
        parts = {"x": torch.randn(96, 64, device=dev).to(torch.bfloat16), "idx": torch.randint(0, 999, (96, 8), device=dev, dtype=torch.int32),
                 "act": torch.randn(96, 8, device=dev)}  # fmt: skip
        dpc = DataParallelComm(group, dev, 64, 64, {n_: 2 * v.numel() * v.element_size() for n_, v in parts.items()}, use_multicast=use_mc)
        if use_mc and not dpc.use_multicast:
            continue
        for call in range(3):
            mine = {n_: (v + call).to(v.dtype) for n_, v in parts.items()}
            got = dpc.exchange(mine)
            K.check_status(dev)
            for n_, v in mine.items():
                want = [torch.empty_like(v) for _ in range(2)]
                dist.all_gather(want, v.contiguous())
                assert torch.equal(got[n_], torch.cat(want)), (use_mc, call, n_)

    rows, cols = 1000, 4096
    for use_mc in (False, True):
        comm = AllReduceComm(group, dev, rows, cols, use_multicast=use_mc)
        if use_mc and not comm.use_multicast:
            print("no multicast mapping for this group: the multimem variant is not exercised here")
            continue
        for call in range(3):  # both buffers and their re-use
            torch.manual_seed(10 * call + rank)
            mine = torch.randn(rows, cols, device=dev).to(torch.bfloat16)
            want = mine.float().clone()
            dist.all_reduce(want)
            comm.matrix(rows).copy_(mine)
            got = comm.all_reduce(rows)
            K.check_status(dev)
            assert torch.allclose(got.float(), want, atol=3e-2, rtol=2e-2), (use_mc, call, float((got.float() - want).abs().max()))

    # fused crosscoder step, 4 heads over 2 ranks, against autograd on the same mesh
    H, d, F, B, lr, steps = 4, 64, 2048, 512, 1e-3, 4
    torch.manual_seed(0)
    cfg = CrosscoderConfig(hook_points=[f"s{i}" for i in range(H)], d_model=d, expansion_factor=F / d, act_fn="jumprelu", device=str(dev),
                           dtype=torch.float32, norm_activation="inference")  # fmt: skip
    ref = Crosscoder(cfg, device_mesh=mesh)
    ref.init_parameters(encoder_uniform_bound=0.2, decoder_uniform_bound=0.2, init_log_jumprelu_threshold_value=-0.3)
    ref.set_decoder_to_fixed_norm(1.0, True)
    ref.init_encoder_with_decoder_transpose(1.0 / H)
    with torch.no_grad():
        ref.W_D.mul_(1 + 0.1 * (torch.arange(2, device=dev) + 2 * rank).view(2, 1, 1))
    fused_model = copy.deepcopy(ref)
    fused_model.device_mesh = mesh
    engine = FusedCrosscoderStep(fused_model, list_width=F)
    g = torch.Generator(device=dev).manual_seed(1)
    basis = torch.randn(8, d, device=dev, generator=g)
    opt = torch.optim.Adam(ref.parameters(), lr=lr)
    tokens = torch.zeros(B, dtype=torch.long, device=dev)
    ref_losses, fused_losses = [], []
    for _ in range(steps):
        z = torch.randn(B, 8, device=dev, generator=g)
        x = torch.stack([z @ basis * (1 + 0.2 * h) + 0.3 * torch.randn(B, d, device=dev, generator=g) for h in range(H)], dim=1)
        x = (x * (d**0.5 / x.norm(dim=-1).mean())).to(torch.bfloat16)
        dist.broadcast(x, src=0)
        mine = x[:, 2 * rank : 2 * rank + 2].contiguous()
        opt.zero_grad()
        batch = {f"s{2 * rank + h}": mine[:, h].float() for h in range(2)} | {"tokens": tokens}
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = ref.compute_loss(batch, sparsity_loss_type="tanh", l1_coefficient=3e-2, lp_coefficient=2e-3, return_aux_data=True)
        out["loss"].backward()
        thr = ref.activation_function.log_jumprelu_threshold
        dist.all_reduce(thr.grad, group=group)  # shared parameter: the trainer sums its gradient over the head ranks
        opt.step()
        ref_losses.append(float(out["loss"].detach()))
        local = engine.step(mine, lr, l1_coefficient=3e-2, lp_coefficient=2e-3)
        dist.all_reduce(local, group=group)
        fused_losses.append(float(local) / 2)
    K.check_status(dev)
    assert int(engine.list_overflow) == 0
    assert torch.allclose(torch.tensor(ref_losses), torch.tensor(fused_losses), rtol=3e-2), (ref_losses, fused_losses)
    a, b = ref.activation_function.log_jumprelu_threshold.detach(), fused_model.activation_function.log_jumprelu_threshold.detach()
    assert float((a - b).abs().mean()) < 0.3 * lr * steps, float((a - b).abs().mean())
