"""Multi-rank logic on CPU (gloo, 2 ranks): sharded models and the fused step's orchestration must reproduce
the single-process result."""

import pytest
import torch
import torch.distributed as dist

from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
from language_model_saes_b200.ops.fused_step import FusedTopKSAEStep
from language_model_saes_b200.parallel.mesh import DimMap, build_mesh
from language_model_saes_b200.testing import distributed_test


def _full_model(d=32, F=128, k=8):
    torch.manual_seed(0)
    cfg = SAEConfig(hook_point_in="h", hook_point_out="h", d_model=d, expansion_factor=F / d, act_fn="topk", top_k=k)
    sae = SparseAutoEncoder(cfg)
    sae.init_parameters(encoder_uniform_bound=0.3, decoder_uniform_bound=0.3)
    sae.set_decoder_to_fixed_norm(0.8, True)
    sae.init_encoder_with_decoder_transpose()
    with torch.no_grad():
        sae.b_E.normal_(0, 0.05)
        sae.b_D.normal_(0, 0.05)
    sae.set_dataset_average_activation_norm({"h": d**0.5})
    return sae


def _sharded_copy(full: SparseAutoEncoder, mesh) -> SparseAutoEncoder:
    m = SparseAutoEncoder(full.cfg.model_copy(), mesh)
    m.load_full_state_dict(full.full_state_dict())
    return m


def _data(B=64, d=32):
    g = torch.Generator().manual_seed(5)
    return torch.randn(B, d, generator=g) * 1.0


@distributed_test(nproc_per_node=2, backend="gloo")
def test_feature_sharded_forward_matches_single():
    mesh = build_mesh("cpu", (1, 2), ("data", "model"))
    full = _full_model()
    tp = _sharded_copy(full, mesh)
    x = _data()
    batch = {"h": x, "tokens": torch.zeros(x.shape[0], dtype=torch.long)}
    want = full.compute_loss(full.normalize_activations(batch))
    got = tp.compute_loss(tp.normalize_activations(batch))
    assert torch.allclose(want["loss"], got["loss"], rtol=1e-5)
    acts = DimMap({"model": 1}).gather(got["feature_acts"], mesh)
    assert torch.allclose(acts, want["feature_acts"], atol=1e-6)
    want["loss"].backward()
    got["loss"].backward()
    sl = DimMap({"model": 0}).local_slices(full.W_D.shape, mesh)
    assert torch.allclose(tp.W_D.grad, full.W_D.grad[sl], atol=1e-6)
    assert torch.allclose(tp.b_D.grad, full.b_D.grad, atol=1e-6)
    # round trip of the gathered state dict
    sd = tp.full_state_dict()
    assert torch.allclose(sd["W_E"], full.W_E) and sd["W_E"].shape == full.W_E.shape


def _run_fused(sae, xs, k, lr=1e-2):
    eng = FusedTopKSAEStep(sae)
    losses = [eng.step(x, x, k, lr) for x in xs]
    return eng, torch.stack(losses)


@distributed_test(nproc_per_node=2, backend="gloo")
def test_fused_step_feature_and_data_parallel_match_single():
    full = _full_model()
    xs = [(_data() + i).to(torch.bfloat16) for i in range(3)]
    ref = SparseAutoEncoder(full.cfg.model_copy())
    ref.load_full_state_dict(full.full_state_dict())
    _, want = _run_fused(ref, xs, 8)

    tp_mesh = build_mesh("cpu", (1, 2), ("data", "model"))
    tp = _sharded_copy(full, tp_mesh)
    _, got = _run_fused(tp, xs, 8)
    assert torch.allclose(got, want, rtol=1e-4), (got, want)
    W = DimMap({"model": 0}).gather(tp.W_D.data, tp_mesh)
    assert torch.allclose(W, ref.W_D.data, atol=1e-5)

    dp_mesh = build_mesh("cpu", (2, 1), ("data", "model"))
    dp = _sharded_copy(full, dp_mesh)
    r = dist.get_rank()
    half = xs[0].shape[0] // 2
    _, got_dp = _run_fused(dp, [x[r * half : (r + 1) * half] for x in xs], 8)
    mean = got_dp.clone()
    dist.all_reduce(mean)
    assert torch.allclose(mean / 2, want, rtol=1e-4)
    assert torch.allclose(dp.W_D.data, ref.W_D.data, atol=1e-5)
    assert torch.allclose(dp.W_E.data, ref.W_E.data, atol=1e-5)


def _moment_norm(eng) -> torch.Tensor:
    return torch.sqrt(sum(st[0].square().sum() for st in eng.state.values() if st is not None))


def _clip_case(make):
    """First Adam moments after one step are 0.1 x the (clipped) gradient: their norm shows the factor that was applied."""
    x = _data().to(torch.bfloat16)
    e0 = FusedTopKSAEStep(make())
    e0.step(x, x, 8, 1e-2)
    e2 = FusedTopKSAEStep(make())
    e2.step(x, x, 8, 1e-2, clip_grad_norm=1e9)  # a bound above the norm: measured, nothing scaled
    g = e2.last_grad_norm
    e1 = FusedTopKSAEStep(make())
    e1.step(x, x, 8, 1e-2, clip_grad_norm=float(g) / 4)
    return g, e0, e1, e2


def test_fused_step_clips_the_gradient_norm_like_the_generic_path():
    from language_model_saes_b200.optim import compute_grad_norm

    full = _full_model()

    def make():
        m = SparseAutoEncoder(full.cfg.model_copy())
        m.load_full_state_dict(full.full_state_dict())
        return m

    g, e0, e1, e2 = _clip_case(make)
    assert torch.allclose(e1.last_grad_norm, g, rtol=1e-5)
    assert torch.allclose(_moment_norm(e1), _moment_norm(e0) / 4, rtol=1e-3)  # clipped to a quarter of the norm
    assert torch.allclose(e2.WD, e0.WD) and torch.allclose(e2.bD, e0.bD)
    # the norm is the generic path's: |g|_2 / sqrt(non-zero entries) (the fused path rounds operands to bf16: loose tolerance)
    ref = make()
    x = _data().to(torch.bfloat16).float()
    ref.compute_loss({"h": x, "tokens": torch.zeros(x.shape[0], dtype=torch.long)})["loss"].backward()
    want = compute_grad_norm(ref.parameters())
    assert torch.allclose(g, want, rtol=5e-2), (g, want)


@distributed_test(nproc_per_node=2, backend="gloo")
def test_fused_step_clipping_feature_parallel_matches_single():
    full = _full_model()

    def single():
        m = SparseAutoEncoder(full.cfg.model_copy())
        m.load_full_state_dict(full.full_state_dict())
        return m

    g, _, e1, _ = _clip_case(single)
    mesh = build_mesh("cpu", (1, 2), ("data", "model"))
    gt, _, t1, _ = _clip_case(lambda: _sharded_copy(full, mesh))
    assert torch.allclose(gt, g, rtol=1e-4) and torch.allclose(t1.last_grad_norm, g, rtol=1e-4)  # sharded rows add up over the group, the decoder bias counts once
    W = DimMap({"model": 0}).gather(t1.WD, mesh)
    assert torch.allclose(W, e1.WD, atol=1e-5)


@distributed_test(nproc_per_node=2, backend="gloo")
def test_fused_batchtopk_step_feature_and_data_parallel_match_single():
    """Batch-level top-k on the fused path: feature shards share one threshold (and ration the ties between them), data
    shards agree on the width of their code lists; both reproduce the single-process run."""
    full = _full_model()
    full.cfg.act_fn = "batchtopk"
    xs = [(_data() + i).to(torch.bfloat16) for i in range(3)]
    ref = SparseAutoEncoder(full.cfg.model_copy())
    ref.load_full_state_dict(full.full_state_dict())
    eng, want = _run_fused(ref, xs, 8)
    assert eng.batch_level
    idx, _ = eng.encode(xs[0], 8)
    assert int((idx >= 0).sum()) == 8 * xs[0].shape[0]  # exactly k codes per token on average

    tp_mesh = build_mesh("cpu", (1, 2), ("data", "model"))
    tp = _sharded_copy(full, tp_mesh)
    # before any update: the shards together keep exactly k * batch codes, the same ones as one process except for which
    # of the entries EQUAL to the (bf16) threshold get the last places (one process grants them in row order, shards in
    # rank order; the reference's sort breaks such ties arbitrarily too)
    tp0 = _sharded_copy(full, tp_mesh)
    ref0 = SparseAutoEncoder(full.cfg.model_copy())
    ref0.load_full_state_dict(full.full_state_dict())
    idx_1, act_1 = FusedTopKSAEStep(ref0).encode(xs[0], 8)
    idx_l, act_l = FusedTopKSAEStep(tp0).encode(xs[0], 8)
    n = (idx_l >= 0).sum()
    dist.all_reduce(n)
    assert int(n) == 8 * xs[0].shape[0]
    F_l, r = tp0.W_D.shape[0], dist.get_rank()
    dense_1 = torch.zeros(xs[0].shape[0], 2 * F_l)
    rows = torch.arange(xs[0].shape[0])[:, None].expand_as(idx_1)
    dense_1[rows[idx_1 >= 0], idx_1[idx_1 >= 0].long()] = act_1[idx_1 >= 0]
    dense_l = torch.zeros(xs[0].shape[0], F_l)
    rows = torch.arange(xs[0].shape[0])[:, None].expand_as(idx_l)
    dense_l[rows[idx_l >= 0], idx_l[idx_l >= 0].long()] = act_l[idx_l >= 0]
    mine = dense_1[:, r * F_l : (r + 1) * F_l]
    differ = (mine != 0) != (dense_l != 0)
    assert int(differ.sum()) <= 8 and torch.equal(mine[~differ], dense_l[~differ])
    eng_tp, got = _run_fused(tp, xs, 8)
    assert torch.allclose(got, want, rtol=2e-2), (got, want)

    # data parallel: every replica thresholds its own half batch (k * local batch codes), as the reference does
    dp_mesh = build_mesh("cpu", (2, 1), ("data", "model"))
    dp = _sharded_copy(full, dp_mesh)
    r = dist.get_rank()
    half = xs[0].shape[0] // 2
    eng_dp, got_dp = _run_fused(dp, [x[r * half : (r + 1) * half] for x in xs], 8)
    assert torch.isfinite(got_dp).all()
    both = [torch.empty_like(dp.W_D.data) for _ in range(2)]
    dist.all_gather(both, dp.W_D.data.contiguous())
    assert torch.equal(both[0], both[1])  # replicas stay identical


@distributed_test(nproc_per_node=2, backend="gloo")
def test_fused_auxk_step_feature_parallel_matches_single():
    """Aux-K on the fused path with feature shards: the dead features' top-k runs over all shards, both reconstructions
    are summed over shards; losses, auxiliary losses and weights follow the single-process run. With ``dead_threshold``
    below one batch every feature that did not fire in the step is dead, on whichever shard it lives."""
    from language_model_saes_b200.ops.fused_step import AuxK

    full = _full_model()
    xs = [(_data() + i).to(torch.bfloat16) for i in range(3)]

    def run(sae):
        eng = FusedTopKSAEStep(sae)
        aux = AuxK(eng.F, k_aux=12, coefficient=1 / 8, dead_threshold=32, device="cpu")
        out = []
        for x in xs:
            loss = eng.step(x, x, 8, 1e-2, aux=aux)
            out.append(torch.stack([loss, eng.last_aux_loss]))
        return eng, aux, torch.stack(out)

    ref = SparseAutoEncoder(full.cfg.model_copy())
    ref.load_full_state_dict(full.full_state_dict())
    _, aux1, want = run(ref)
    assert float(want[:, 1].min()) > 0  # the auxiliary term is active in every step
    mesh = build_mesh("cpu", (1, 2), ("data", "model"))
    tp = _sharded_copy(full, mesh)
    eng, aux2, got = run(tp)
    assert torch.allclose(got, want, rtol=1e-4), (got, want)
    assert torch.allclose(DimMap({"model": 0}).gather(tp.W_D.data, mesh), ref.W_D.data, atol=1e-5)
    assert torch.allclose(DimMap({"model": 1}).gather(tp.W_E.data, mesh), ref.W_E.data, atol=1e-5)
    F_l, r = eng.F, dist.get_rank()
    assert torch.equal(aux2.tokens_since_last_activation, aux1.tokens_since_last_activation[r * F_l : (r + 1) * F_l])


def _run_fused_comm(sae, xs, k, comm, lr=1e-2):
    eng = FusedTopKSAEStep(sae, comm=comm)
    return eng, torch.stack([eng.step(x, x, k, lr) for x in xs])


@distributed_test(nproc_per_node=2, backend="gloo")
def test_peer_memory_protocol_on_the_host_matches_collectives():
    """The peer-buffer protocol of the fused step (stores into peers' buffers, epoch flags, bounded waits) run by the
    host over a shared-memory file: same losses and weights as the all-reduce path, over several steps (the buffers are
    re-used without a barrier), also when one rank publishes a flag late."""
    from language_model_saes_b200.parallel.host_transport import HostPeerComm
    from language_model_saes_b200.parallel.mesh import mesh_group
    from language_model_saes_b200.parallel.symm import PHASE_CAND, PHASE_PARTIAL

    full = _full_model()
    xs = [(_data() + i).to(torch.bfloat16) for i in range(4)]
    mesh = build_mesh("cpu", (1, 2), ("data", "model"))
    _, want = _run_fused(_sharded_copy(full, mesh), xs, 8)  # gloo all-gather / all-reduce between the shards
    late = {"delay_flag": (PHASE_PARTIAL, 0.2)} if dist.get_rank() == 1 else None
    comm = HostPeerComm(mesh_group(mesh, "model"), xs[0].shape[0], 8, 32, timeout_s=20.0, faults=late, partial_dtype=torch.float32)
    tp = _sharded_copy(full, mesh)
    eng, got = _run_fused_comm(tp, xs, 8, comm)
    assert comm.epochs[PHASE_PARTIAL] == len(xs)
    # each rank reports the loss of the rows it owns: the mean over ranks is the batch loss
    dist.all_reduce(got)
    assert torch.allclose(got / 2, want, rtol=1e-4), (got / 2, want)
    ref = _sharded_copy(full, mesh)
    ref_eng, _ = _run_fused(ref, xs, 8)
    assert torch.allclose(tp.W_D.data, ref.W_D.data, atol=1e-5) and torch.allclose(tp.W_E.data, ref.W_E.data, atol=1e-5)
    assert torch.allclose(tp.b_D.data, ref.b_D.data, atol=1e-5)
    # codes and reconstruction for metrics, twice in a row between training steps: the candidate exchange then runs
    # without the later phases of a step behind it (its landing zone alternates, its epoch advances per exchange)
    for x in xs[:2]:
        idx_a, act_a, xhat_a = eng.forward_dense(x, 8)
        idx_b, act_b, xhat_b = ref_eng.forward_dense(x, 8)
        assert torch.equal(idx_a.sort(dim=1).values, idx_b.sort(dim=1).values)
        assert torch.allclose(xhat_a, xhat_b, atol=1e-4)
    assert comm.epochs[PHASE_CAND] == len(xs) + 2
    more, more_ref = eng.step(xs[0], xs[0], 8, 1e-2), ref_eng.step(xs[0], xs[0], 8, 1e-2)
    dist.all_reduce(more)
    assert torch.allclose(more / 2, more_ref, rtol=1e-4)
    # partial rows in bf16 (the default on the wire): same protocol, reconstruction rounded like a bf16 all-reduce
    # ... on the debug layout: a guard band behind every region of the buffers; the steps leave all of them untouched
    comm16 = HostPeerComm(mesh_group(mesh, "model"), xs[0].shape[0], 8, 32, timeout_s=20.0, guards=True)
    assert [n for n, _ in comm16.lay["guards"]] == ["flags", "cand_val", "cand_idx", "partial", "dxhat"]
    _, got16 = _run_fused_comm(_sharded_copy(full, mesh), xs, 8, comm16)
    dist.all_reduce(got16)
    assert torch.allclose(got16 / 2, want, rtol=2e-2), (got16 / 2, want)
    comm16.check_guards()
    dist.barrier()
    # a store that runs one row past the end of the peer's gradient region is caught by that rank's check
    if dist.get_rank() == 0:
        end = comm16.lay["dxhat"] + xs[0].shape[0] * 32 * 2
        comm16.bufs[1][end : end + 64] = 0
    dist.barrier()
    if dist.get_rank() == 1:
        try:
            comm16.check_guards()
            raise AssertionError("the overrun went unnoticed")
        except RuntimeError as e:
            assert "dxhat" in str(e)
    else:
        comm16.check_guards()


@distributed_test(nproc_per_node=2, backend="gloo")
def test_peer_memory_protocol_reports_a_flag_that_never_arrives():
    """Rank 1 never publishes its partial-rows flag: rank 0's bounded wait runs out and its step raises
    ``CollectiveTimeout`` naming the phase and the silent rank; rank 1, whose own sources all arrived, finishes."""
    from language_model_saes_b200.ops.sae_kernels import CollectiveTimeout
    from language_model_saes_b200.parallel.host_transport import HostPeerComm
    from language_model_saes_b200.parallel.mesh import mesh_group
    from language_model_saes_b200.parallel.symm import PHASE_PARTIAL

    full = _full_model()
    x = _data().to(torch.bfloat16)
    mesh = build_mesh("cpu", (1, 2), ("data", "model"))
    rank = dist.get_rank()
    # rank 1 waits for rank 0's gradient flag, which rank 0 publishes only after its own wait has run out: give it longer
    comm = HostPeerComm(mesh_group(mesh, "model"), x.shape[0], 8, 32, timeout_s=1.0 if rank == 0 else 20.0,
                        faults={"drop_flag": PHASE_PARTIAL} if rank == 1 else None)  # fmt: skip
    sae = _sharded_copy(full, mesh)
    eng = FusedTopKSAEStep(sae, comm=comm)
    before = {n: p.detach().clone() for n, p in sae.named_parameters()}
    if rank == 0:
        with pytest.raises(CollectiveTimeout, match=r"phase 1 .*rank\(s\) \[1\]") as info:
            eng.step(x, x, 8, 1e-2)
        assert info.value.code == 5 and info.value.sources == [1]
        # the step gave up before its update: parameters and moments are those of before the step
        for n, p in sae.named_parameters():
            assert torch.equal(p.detach(), before[n]), n
        assert all(float(m.abs().sum()) == 0.0 for st in eng.state.values() if st is not None for m in st)
    else:
        assert torch.isfinite(eng.step(x, x, 8, 1e-2))


@distributed_test(nproc_per_node=2, backend="gloo")
def test_heartbeat_reports_a_rank_that_leaves_and_one_that_goes_silent():
    import time

    import torch.distributed as dist

    from language_model_saes_b200.parallel.health import Heartbeat, PeerLost, default_store

    rank = dist.get_rank()
    hb = Heartbeat(default_store(), rank, 2, timeout_s=30.0, prefix="t1")
    dist.barrier()  # (the two processes may have started seconds apart)
    hb.beat(0)
    dist.barrier()
    hb.check()  # both alive
    dist.barrier()  # rank 1 must not announce that it leaves before rank 0 has looked
    if rank == 1:
        hb.leave("ValueError: injected on the host")  # what Trainer.fit does in its exception handler
        dist.barrier()
    else:
        dist.barrier()
        with pytest.raises(PeerLost, match="rank 1: left: ValueError"):
            hb.check()
    # silence: rank 1 stops beating (it stays in the job, so the barriers below still work)
    hb2 = Heartbeat(default_store(), rank, 2, timeout_s=0.5, prefix="t2")
    hb2.beat(1)
    dist.barrier()
    if rank == 0:
        deadline = time.time() + 10
        while True:
            hb2.beat(2)
            try:
                hb2.check()
            except PeerLost as e:
                assert list(e.ranks) == [1] and "silent" in e.ranks[1]
                break
            assert time.time() < deadline, "the silent peer was never reported"
            time.sleep(0.1)
    dist.barrier()


def test_trainer_saves_a_failure_checkpoint_and_reports_kernel_status(tmp_path):
    import torch

    from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
    from language_model_saes_b200.trainer import Trainer, TrainerConfig, _LossReader

    cfg = SAEConfig(hook_point_in="in", hook_point_out="in", d_model=16, expansion_factor=2, act_fn="relu", device="cpu",
                    dtype=torch.float32, norm_activation="inference")  # fmt: skip
    sae = SparseAutoEncoder(cfg)
    sae.init_parameters(encoder_uniform_bound=0.3, decoder_uniform_bound=0.3, init_log_jumprelu_threshold_value=0.0)

    def stream():
        for i in range(10):
            if i == 4:
                raise OSError("disk went away")  # a host-side failure in the middle of the run
            yield {"in": torch.randn(8, 16), "tokens": torch.ones(8, dtype=torch.long)}

    tcfg = TrainerConfig(lr=1e-3, total_training_tokens=80, lr_warm_up_steps=0, n_checkpoints=0, log_frequency=100,
                         exp_result_path=str(tmp_path), checkpoint_on_failure=True, l1_coefficient=1e-4, sparsity_loss_type="power")  # fmt: skip
    trainer = Trainer(tcfg)
    with pytest.raises(OSError, match="disk went away"):
        trainer.fit(sae, stream())
    out = tmp_path / "failure" / "rank_0"
    state = torch.load(out / "trainer.pt", weights_only=False)
    assert state["cur_step"] == 4 and "optimizer" in state and (out / "local_state.pt").exists() and (out / "config.json").exists()
    # the status word that travels with the loss: nothing to report on CPU tensors
    assert _LossReader().push(torch.tensor(1.5)) == 1.5
