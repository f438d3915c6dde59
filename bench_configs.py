"""The benchmark configurations beyond the headline one, reached through ``bench.py --config N``.

    3  million-feature BatchTopK SAE: d_model 4096, d_sae 1 048 576, batch-level top-k of 64 x batch, batch 8192 tokens,
       Aux-K dead-feature loss with k_aux 512, data x feature parallel (2 x 4 on eight GPUs)
    4  crosscoder over model snapshots, head parallel (one snapshot per GPU): see ``run_crosscoder``
    5  cross-layer transcoder + low-rank sparse attention: see ``run_clt_lorsa``

Same output contract as ``bench.py`` (one JSON line from rank 0, device-timed ``value`` and an end-to-end number through
``Trainer.fit`` with pinned host batches), same two arms: ``--impl ours`` runs this package, ``--impl reference`` the
unmodified reference project from ``baseline/_ref`` through its own ``Trainer.fit``.
"""

from __future__ import annotations

import gc
import os
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))


def mesh_shape(world: int) -> tuple[int, int]:
    """(data, model) sizes for ``world`` GPUs: feature shards up to four ways, replicas beyond that. ``LMSAE_BENCH_MESH=AxB``
    overrides it."""
    env = os.environ.get("LMSAE_BENCH_MESH")
    if env:
        dp, tp = (int(v) for v in env.lower().split("x"))
        assert dp * tp == world, f"LMSAE_BENCH_MESH={env} does not multiply to {world} ranks"
        return dp, tp
    tp = min(world, 4)
    return world // tp, tp


C3 = dict(d_model=4096, expansion=256, top_k=64, batch=8192, lr=2e-4, k_aux=512, auxk=1 / 32, pool=4)


def _c3_scaled() -> dict:
    """Config 3, optionally with a smaller dictionary for machines whose memory cannot hold the full one on few GPUs
    (``LMSAE_BENCH_C3_EXPANSION``); the reported config names the size actually run."""
    c = dict(C3)
    c["expansion"] = int(os.environ.get("LMSAE_BENCH_C3_EXPANSION", c["expansion"]))
    return c


def c3_config(world: int, c: dict) -> dict:
    dp, tp = mesh_shape(world)
    return {"model": f"BatchTopK SAE d_model {c['d_model']}, d_sae {c['d_model'] * c['expansion']}, k {c['top_k']} x batch, "
                     f"Aux-K k_aux {c['k_aux']} coefficient 1/32 dead after 10 batches, Adam lr {c['lr']:g}, fp32 parameters, bf16 autocast",
            "global_batch": c["batch"], "seq_len": 1, "parallelism": f"dp{dp} x tp{tp}",
            "l2": f"inputs rotate through {c['pool']} batches > L2"}  # fmt: skip


def _batches(c: dict, n: int, rows: slice, seed: int = 1234):
    """The synthetic activations of bench.py (low-rank Gaussian plus noise, mean norm sqrt(d)) at this config's shape;
    every rank generates the same global batches and keeps its ``rows``."""
    import torch

    g = torch.Generator().manual_seed(seed)
    d, B = c["d_model"], c["batch"]
    A = torch.randn(256, d, generator=g)
    out = []
    for _ in range(n):
        z = torch.randn(B, 256, generator=g)
        x = z @ A + 0.1 * torch.randn(B, d, generator=g)
        x = x * (d**0.5 / x.norm(dim=-1).mean())
        out.append(x[rows].to(torch.bfloat16).contiguous().pin_memory())
    return out


def run_config3(args, bench) -> None:
    c = _c3_scaled()
    if args.impl == "reference":
        return _run_config3_reference(args, bench, c)
    import torch
    import torch.distributed as dist

    import language_model_saes_b200 as lm
    from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
    from language_model_saes_b200.ops import sae_kernels as K
    from language_model_saes_b200.trainer import Trainer, TrainerConfig

    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    assert world == args.gpus
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dp, tp = mesh_shape(world)
    mesh = None
    if world > 1:
        from language_model_saes_b200.parallel.mesh import build_mesh, mesh_local_rank

        dist.init_process_group("nccl", device_id=dev)
        mesh = build_mesh("cuda", (dp, tp), ("data", "model"))
        dp_rank = mesh_local_rank(mesh, "data")
    else:
        dp_rank = 0
    D, B = c["d_model"], c["batch"]
    B_l = B // dp
    hook = "blocks.16.hook_resid_post"
    torch.manual_seed(0)
    cfg = SAEConfig(hook_point_in=hook, hook_point_out=hook, d_model=D, expansion_factor=c["expansion"], act_fn="batchtopk",
                    top_k=c["top_k"], device=f"cuda:{local}", dtype=torch.float32)  # fmt: skip
    sae = SparseAutoEncoder(cfg, mesh)
    bound = 1.0 / D**0.5

    def init():
        """Both timed fits start from these parameters (same seed): a step's cost depends on the number of dead features."""
        torch.manual_seed(0)
        sae.init_parameters(encoder_uniform_bound=bound, decoder_uniform_bound=bound)
        sae.set_decoder_to_fixed_norm(1.0, force_exact=True)
        sae.init_encoder_with_decoder_transpose()

    init()
    sae.set_dataset_average_activation_norm({hook: D**0.5})
    host = _batches(c, c["pool"], slice(dp_rank * B_l, (dp_rank + 1) * B_l))
    tokens = torch.zeros(B_l, dtype=torch.long).pin_memory()
    mask = torch.ones(B_l, dtype=torch.bool).pin_memory()
    W, Ks = args.warmup, args.steps

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def fit(source, on_start, n_warm, n_steps):
        """One ``Trainer.fit`` over n_warm + n_steps batches; ``on_start`` fires when the first timed batch is drawn."""

        def stream():
            for i in range(n_warm + n_steps + 2):
                if i == n_warm + 1:  # the trainer keeps one batch in flight
                    on_start()
                yield {hook: source(i), "tokens": tokens, "mask": mask}

        with tempfile.TemporaryDirectory() as tmp:
            tcfg = TrainerConfig(total_training_tokens=(n_warm + n_steps) * B, lr=c["lr"], lr_warm_up_steps=0, lr_cool_down_steps=0,
                                 lr_scheduler_name="constant", log_frequency=1, skip_metrics_calculation=True, n_checkpoints=0,
                                 exp_result_path=tmp, k_warmup_steps=0, l1_coefficient=None, auxk_coefficient=c["auxk"],
                                 k_aux=c["k_aux"], dead_threshold=10 * B, prefetch_to_device=True)  # fmt: skip
            tr = current["trainer"] = Trainer(tcfg)
            tr.fit(sae, stream())
        return tr

    current: dict = {}

    # ---- device-timed: batches resident on the device, CUDA events around the timed steps ------------------------
    pool = [h.to(dev) for h in host]
    ev = {}
    sampler = bench.ClockSampler(local)

    def start_events():
        barrier()
        sampler.start()
        gc.collect()
        gc.disable()
        ev["l0"] = K.kernel_launch_count()
        ev["a"] = torch.cuda.Event(enable_timing=True)
        ev["a"].record()

    tr = fit(lambda i: pool[i % len(pool)], start_events, W, Ks)
    ev["b"] = torch.cuda.Event(enable_timing=True)
    ev["b"].record()
    barrier()
    gc.enable()
    clocks = sampler.stop()
    launches = K.kernel_launch_count() - ev["l0"]
    ms = ev["a"].elapsed_time(ev["b"])
    K.check_status(dev)
    fused = tr.fused is not None
    aux_cap = tr._fused_aux.capacity if tr._fused_aux is not None else None
    sharded_state = bool(fused and tr.fused.dp_comm is not None)
    del pool, tr
    torch.cuda.empty_cache()
    init()
    # ---- end to end: pinned host batches copied every step, loss read back every step ---------------------------
    wall = {}

    def start_wall():
        barrier()
        wall["t0"] = time.perf_counter()

    tr = fit(lambda i: host[i % len(host)], start_wall, W, Ks)
    barrier()
    e2e_ms = (time.perf_counter() - wall["t0"]) * 1e3
    final_loss = tr.last_loss
    aux_cap_e2e = tr._fused_aux.capacity if tr._fused_aux is not None else None
    # ---- where the time goes: a third fit from the same parameters with an event mark after every phase of the step ----
    phases = None
    if fused and os.environ.get("LMSAE_BENCH_PHASES", "1") == "1":
        del tr
        torch.cuda.empty_cache()
        init()
        pool = [h.to(dev) for h in host]
        tr = fit(lambda i: pool[i % len(pool)], lambda: current["trainer"].fused.start_phase_timing(), W, Ks)
        pt = tr.fused.phase_times()
        names = sorted(pt)
        vals = torch.tensor([pt[n] for n in names], device=dev, dtype=torch.float64)
        lo = vals.clone()
        if world > 1:
            dist.all_reduce(vals, op=dist.ReduceOp.MAX)
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        order_ = sorted(range(len(names)), key=lambda i: -float(vals[i]))
        phases = {names[i]: [round(float(lo[i]), 3), round(float(vals[i]), 3)] for i in order_}
    t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    if rank == 0:
        bench.emit({
            "metric": f"SAE train tokens/s (d{D} x {D * c['expansion']} BatchTopK k{c['top_k']}, Aux-K {c['k_aux']})",
            "value": Ks * B / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": Ks, "warmup": W, "ms_per_step": ms / Ks,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": c3_config(world, c), "clocks": clocks,
            "path": "Trainer.fit on the fused kernel path" if fused else "Trainer.fit on the generic autograd path",
            "optimizer_state_sharded_over_replicas": sharded_state, "auxk_dead_capacity": aux_cap, "auxk_dead_capacity_e2e": aux_cap_e2e,
            **({"phase_ms_min_max_over_ranks": phases} if phases else {}),
            "e2e": {"value": Ks * B / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / Ks,
                    "h2d_bytes_per_step": B * D * 2 // tp + world * B_l * 9, "d2h_bytes_per_step": 4 * world},
            "gpu_launches": launches, "final_loss": final_loss, "impl": "ours", "package": lm.__name__,
        })  # fmt: skip
    if world > 1:
        dist.destroy_process_group()


def _run_config3_reference(args, bench, c: dict) -> None:
    here = os.path.join(ROOT, "baseline")
    if not os.path.isdir(os.path.join(here, "_ref", "llamascopium")):
        bench.emit({"impl": "reference", "unavailable": "baseline/_ref is not installed"})
        return
    sys.path[:0] = [os.path.join(here, "_stubs"), os.path.join(here, "_ref")]
    try:
        import torch
        import torch.distributed as dist
        from llamascopium import SAEConfig, SparseAutoEncoder, Trainer, TrainerConfig
        from llamascopium.utils.distributed import DimMap
    except Exception as e:  # noqa: BLE001
        bench.emit({"impl": "reference", "unavailable": f"reference does not import here: {type(e).__name__}: {e}"[:300]})
        return
    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dp, tp = mesh_shape(world)
    mesh = None
    dp_rank = 0
    if world > 1:
        from torch.distributed.device_mesh import init_device_mesh

        dist.init_process_group("nccl", device_id=dev)
        mesh = init_device_mesh("cuda", (dp, tp), mesh_dim_names=("data", "model"))
        dp_rank = mesh.get_local_rank("data")
    D, B = c["d_model"], c["batch"]
    B_l = B // dp
    hook = "blocks.16.hook_resid_post"
    W, Ks = args.warmup, args.steps
    try:
        torch.manual_seed(0)
        cfg = SAEConfig(hook_point_in=hook, hook_point_out=hook, d_model=D, expansion_factor=c["expansion"], act_fn="batchtopk",
                        top_k=c["top_k"], device="cuda", dtype=torch.float32)  # fmt: skip
        sae = SparseAutoEncoder(cfg, device_mesh=mesh)
        bound = 1.0 / D**0.5

        def init():
            torch.manual_seed(0)
            sae.init_parameters(encoder_uniform_bound=bound, decoder_uniform_bound=bound)
            sae.set_decoder_to_fixed_norm(1.0, force_exact=True)
            sae.init_encoder_with_decoder_transpose()

        init()
        sae.set_dataset_average_activation_norm({hook: D**0.5})
        host = _batches(c, c["pool"], slice(dp_rank * B_l, (dp_rank + 1) * B_l))

        def wrap(t):
            return DimMap({"data": 0}).from_local(t, mesh) if mesh is not None else t

        tokens = torch.zeros(B_l, dtype=torch.long, device=dev)
        mask = torch.ones(B_l, dtype=torch.bool, device=dev)

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def fit_once(source, record):
            def stream():
                yield {hook: wrap(source(0).float()), "tokens": wrap(tokens), "mask": wrap(mask)}
                for i in range(W + Ks + 1):
                    if i == W:
                        barrier()
                        record("start")
                    yield {hook: wrap(source(i).float()), "tokens": wrap(tokens), "mask": wrap(mask)}

            with tempfile.TemporaryDirectory() as tmp:
                tcfg = TrainerConfig(total_training_tokens=(W + Ks) * B, lr=c["lr"], lr_scheduler_name="constant", log_frequency=10**9,
                                     skip_metrics_calculation=True, n_checkpoints=0, exp_result_path=tmp, k_warmup_steps=0,
                                     l1_coefficient=None, amp_dtype=torch.bfloat16, auxk_coefficient=c["auxk"], k_aux=c["k_aux"],
                                     dead_threshold=10 * B)  # fmt: skip
                Trainer(tcfg).fit(sae, stream())
            barrier()
            record("end")

        pool = [h.to(dev) for h in host]
        ev = {}

        def rec(name):
            ev[name] = torch.cuda.Event(enable_timing=True)
            ev[name].record()

        sampler = bench.ClockSampler(local)
        sampler.start()
        fit_once(lambda i: pool[i % len(pool)], rec)
        clocks = sampler.stop()
        torch.cuda.synchronize()
        ms = ev["start"].elapsed_time(ev["end"])
        del pool
        torch.cuda.empty_cache()
        init()
        wall = {}
        fit_once(lambda i: host[i % len(host)].to(dev, non_blocking=True), lambda n: wall.__setitem__(n, time.perf_counter()))
        e2e_ms = (wall["end"] - wall["start"]) * 1e3
    except Exception as e:  # noqa: BLE001  (e.g. the dense [batch, d_sae] tensors of the reference do not fit this many GPUs)
        if rank == 0:
            bench.emit({"impl": "reference", "unavailable": f"the reference failed on this configuration: {type(e).__name__}: {str(e)[:200]}",
                        "config": c3_config(world, c)})  # fmt: skip
        if world > 1:
            dist.destroy_process_group()
        return
    t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    if rank == 0:
        bench.emit({
            "impl": "reference",
            "metric": f"SAE train tokens/s (d{D} x {D * c['expansion']} BatchTopK k{c['top_k']}, Aux-K {c['k_aux']})",
            "value": Ks * B / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": Ks, "warmup": W, "ms_per_step": ms / Ks,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": c3_config(world, c), "clocks": clocks,
            "path": "llamascopium.Trainer.fit(SparseAutoEncoder batchtopk), skip_metrics_calculation=True",
            "e2e": {"value": Ks * B / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / Ks,
                    "h2d_bytes_per_step": B_l * D * 2, "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "note": "library kernels only (cuBLAS / ATen / NCCL); third-party import stand-ins in baseline/_stubs",
        })  # fmt: skip
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------------------
# Generic harness for configurations 4 and 5: both arms drive ``Trainer.fit`` of their own package on the same synthetic
# stream, first with device-resident batches (CUDA events) and then with pinned host batches (wall clock).
# ---------------------------------------------------------------------------------------------------------------------
def _arm(impl: str):
    """Imports of one arm: (package module, wrap(tensor, mesh) for batch entries, mesh builder)."""
    if impl == "reference":
        here = os.path.join(ROOT, "baseline")
        if not os.path.isdir(os.path.join(here, "_ref", "llamascopium")):
            raise RuntimeError("baseline/_ref is not installed")
        sys.path[:0] = [os.path.join(here, "_stubs"), os.path.join(here, "_ref")]
        import llamascopium as pkg
        from llamascopium.utils.distributed import DimMap
        from torch.distributed.device_mesh import init_device_mesh

        def wrap(t, mesh, names):
            return DimMap({"data": 0}).from_local(t, mesh[names] if names else mesh) if mesh is not None else t

        return pkg, wrap, lambda shape, names: init_device_mesh("cuda", shape, mesh_dim_names=names)
    import language_model_saes_b200 as pkg
    from language_model_saes_b200.parallel.mesh import build_mesh

    return pkg, (lambda t, mesh, names: t), lambda shape, names: build_mesh("cuda", shape, names)


def _snapshot(sae):
    """Copies of the dictionary's parameters. Both timed fits of an arm start from them, so that the end-to-end fit
    repeats the trajectory of the device-timed one (the cost of a step depends on the state: number of dead features, of
    codes above a threshold) instead of continuing where it stopped."""
    return [p.detach().clone() for p in sae.parameters()]


def _restore(sae, snap) -> None:
    import torch

    with torch.no_grad():
        for p, s in zip(sae.parameters(), snap):
            p.copy_(s)


def _timed_fits(bench, args, world, rank, local, tokens_per_step, make_trainer, sae, stream_of, pools, result: dict) -> None:
    """``stream_of(source, on_start)`` yields batches; ``pools = (device batches, host batches)``. Fills ``result`` with
    ms / e2e_ms (max over ranks) and clocks. Three fits from the same parameters: an untimed one, the device-timed one and
    the end-to-end one."""
    import torch
    import torch.distributed as dist

    snap = _snapshot(sae)

    dev = torch.device("cuda", local)
    W, Ks = args.warmup, args.steps

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    ev = {}
    sampler = bench.ClockSampler(local)

    def start_events():
        barrier()
        sampler.start()
        gc.collect()
        gc.disable()
        ev["a"] = torch.cuda.Event(enable_timing=True)
        ev["a"].record()

    # an untimed fit first: communicators, symmetric buffers, lazily loaded kernels and the caching allocator are set up
    # once per process, and a host that stalls in one of them inside the timed steps makes every peer's kernels wait
    make_trainer().fit(sae, stream_of(pools[0], lambda: None))
    _restore(sae, snap)
    make_trainer().fit(sae, stream_of(pools[0], start_events))
    ev["b"] = torch.cuda.Event(enable_timing=True)
    ev["b"].record()
    barrier()
    gc.enable()
    result["clocks"] = sampler.stop()
    ms = ev["a"].elapsed_time(ev["b"])
    wall = {}

    def start_wall():
        barrier()
        wall["t0"] = time.perf_counter()

    _restore(sae, snap)
    del snap
    tr = make_trainer()
    tr.fit(sae, stream_of(pools[1], start_wall))
    barrier()
    e2e_ms = (time.perf_counter() - wall["t0"]) * 1e3
    t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    result["ms"], result["e2e_ms"] = t.tolist()
    result["final_loss"] = getattr(tr, "last_loss", None)


def _emit(bench, impl, metric, config, world, args, tokens_per_step, res, h2d, extra=None):
    Ks = args.steps
    rec = {"metric": metric, "value": Ks * tokens_per_step / (res["ms"] / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": Ks,
           "warmup": args.warmup, "ms_per_step": res["ms"] / Ks, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
           "dtype": "bf16", "data": "synthetic", "config": config, "clocks": res.get("clocks"),
           "e2e": {"value": Ks * tokens_per_step / (res["e2e_ms"] / 1e3), "unit": "tokens/s", "ms_per_step": res["e2e_ms"] / Ks,
                   "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * world},
           "final_loss": res.get("final_loss"), "impl": impl}  # fmt: skip
    rec.update(extra or {})
    bench.emit(rec)


C4 = dict(d_model=768, expansion=128, heads=8, batch=4096, lr=2e-4, pool=4, init_log_threshold=None)


def _crosscoder_batches(c: dict, n: int, head_ids: list[int], seed: int = 99):
    """Per-snapshot activations with shared structure: x_h = z (A + 0.3 dA_h) + eps, mean norm sqrt(d), bf16, pinned.
    Every rank draws the same z; a rank keeps the heads it owns."""
    import torch

    g = torch.Generator().manual_seed(seed)
    d, B, H = c["d_model"], c["batch"], c["heads"]
    A = torch.randn(256, d, generator=g)
    dA = torch.randn(H, 256, d, generator=g)
    out = []
    for _ in range(n):
        z = torch.randn(B, 256, generator=g)
        noise = torch.randn(H, B, d, generator=g)
        rec = {}
        for h in head_ids:
            x = z @ (A + 0.3 * dA[h]) + 0.1 * noise[h]
            rec[h] = (x * (d**0.5 / x.norm(dim=-1).mean())).to(torch.bfloat16).contiguous().pin_memory()
        out.append(rec)
    return out


def run_config4(args, bench) -> None:
    """Crosscoder over 8 model snapshots (Pythia-160M-shaped residuals, d_model 768), shared latent of 98304 features,
    JumpReLU, batch 4096 tokens, head parallel: the 8 heads are spread over the GPUs (one each on eight)."""
    import torch
    import torch.distributed as dist

    c = dict(C4)
    impl = args.impl
    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    assert c["heads"] % world == 0, "the number of GPUs must divide the 8 heads"
    config = {"model": f"Crosscoder {c['heads']} heads, d_model {c['d_model']}, d_sae {c['d_model'] * c['expansion']}, JumpReLU "
                       "(threshold exp(1.2), encoder = decoder^T / heads, window 2.0, tanh sparsity loss 1e-3), Adam lr 2e-4, fp32 parameters, bf16 autocast",
              "global_batch": c["batch"], "seq_len": 1, "parallelism": f"head{world}", "l2": "inputs rotate through 4 batches"}  # fmt: skip
    metric = f"Crosscoder train tokens/s ({c['heads']} heads x d{c['d_model']} -> {c['d_model'] * c['expansion']} JumpReLU)"
    try:
        pkg, wrap, build = _arm(impl)
    except Exception as e:  # noqa: BLE001
        bench.emit({"impl": impl, "unavailable": f"{type(e).__name__}: {e}"[:300]})
        return
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    mesh = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        mesh = build((1, world, 1), ("data", "head", "model"))
    H, D, B = c["heads"], c["d_model"], c["batch"]
    hooks = [f"snapshot{h}.blocks.6.hook_resid_post" for h in range(H)]
    per = H // world
    mine = list(range(rank * per, (rank + 1) * per))
    try:
        torch.manual_seed(0)
        kw = dict(hook_points=hooks, d_model=D, expansion_factor=c["expansion"], act_fn="jumprelu", device="cuda" if impl == "reference" else f"cuda:{local}",
                  dtype=torch.float32)  # fmt: skip
        if impl == "ours" and os.environ.get("LMSAE_BENCH_FUSED_HEAD_SUM", "1") == "1" and world > 1:
            kw["fused_head_sum"] = True
        cfg = pkg.CrosscoderConfig(**kw)
        sae = pkg.SparseDictionary.from_config(cfg, device_mesh=mesh) if hasattr(pkg, "SparseDictionary") else None
        bound = 1.0 / D**0.5
        # encoder = decoder^T / heads and a threshold of exp(1.2): a few dozen features per token pass at the start
        sae.init_parameters(encoder_uniform_bound=bound, decoder_uniform_bound=bound, init_log_jumprelu_threshold_value=1.2)
        sae.set_decoder_to_fixed_norm(1.0, force_exact=True)
        sae.init_encoder_with_decoder_transpose(1.0 / H)
        sae.set_dataset_average_activation_norm({hp: D**0.5 for hp in hooks})
        host = _crosscoder_batches(c, c["pool"], mine)
        tokens_h = torch.zeros(B, dtype=torch.long).pin_memory()
        pool_dev = [{h: v.to(dev) for h, v in rec.items()} for rec in host]
        tokens_d = tokens_h.to(dev)
        mask_h = torch.ones(B, dtype=torch.bool).pin_memory()
        mask_d = mask_h.to(dev)
        W, Ks = args.warmup, args.steps
        lead = 1 if impl == "reference" else 0  # the reference consumes one batch while sizing its schedule

        def stream_of(source, on_start):
            on_device = source is pool_dev

            def gen():
                for i in range(lead + W + Ks + 2):
                    if i == lead + W + (0 if impl == "reference" else 1):
                        on_start()
                    rec = source[i % len(source)]
                    out = {hooks[h]: (v if (on_device or impl == "ours") else v.to(dev, non_blocking=True)) for h, v in rec.items()}
                    if impl == "reference":
                        out = {k: v.float() for k, v in out.items()}
                    out["tokens"] = tokens_d if (on_device or impl == "reference") else tokens_h
                    # (the reference's trainer wants a mask in the batch that sizes its schedule, and its crosscoder loss
                    # rejects a per-token mask afterwards: it gets the all-true mask in that first batch only)
                    if impl == "ours" or i == 0:
                        out["mask"] = mask_d if (on_device or impl == "reference") else mask_h
                    yield out

            return gen()

        def make_trainer():
            tmp = tempfile.mkdtemp()
            extra = dict(prefetch_to_device=True, lr_warm_up_steps=0, lr_cool_down_steps=0) if impl == "ours" else dict(amp_dtype=torch.bfloat16)
            tcfg = pkg.TrainerConfig(total_training_tokens=(W + Ks) * B, lr=c["lr"], lr_scheduler_name="constant",
                                     log_frequency=1 if impl == "ours" else 10**9, skip_metrics_calculation=True, n_checkpoints=0,
                                     exp_result_path=tmp, k_warmup_steps=0, l1_coefficient=1e-3, l1_coefficient_warmup_steps=1,
                                     sparsity_loss_type="tanh", **extra)  # fmt: skip
            return pkg.Trainer(tcfg)

        res: dict = {}
        _timed_fits(bench, args, world, rank, local, B, make_trainer, sae, stream_of, (pool_dev, host), res)
    except Exception as e:  # noqa: BLE001
        import traceback

        if rank == 0:
            bench.emit({"impl": impl, "unavailable": f"{type(e).__name__}: {str(e)[:300]}", "config": config,
                        "trace": traceback.format_exc()[-800:]})  # fmt: skip
        if world > 1:
            dist.destroy_process_group()
        return
    if rank == 0:
        _emit(bench, impl, metric, config, world, args, B, res, h2d=per * B * D * 2 + B * 8,
              extra={"path": "Trainer.fit(Crosscoder)", "gpu_launches": _launches(impl)})  # fmt: skip
    if world > 1:
        dist.destroy_process_group()


def _launches(impl: str) -> int:
    if impl != "ours":
        return 0
    from language_model_saes_b200.ops import sae_kernels as K

    return K.kernel_launch_count()


C5 = dict(d_model=768, layers=12, clt_expansion=32, clt_k=64, lorsa_heads=8192, lorsa_qk=64, d_qk=64, lorsa_k=128, seq=1024,
          batch_tokens=2048, lr=2e-4, pool=3)  # fmt: skip


def _layer_batches(c: dict, n: int, keys: list[str], shape: tuple[int, ...], seed: int):
    """Correlated synthetic activations for several hook points of one model (shared latent z, one mixing matrix per
    hook point), mean norm sqrt(d), bf16, pinned."""
    import torch

    g = torch.Generator().manual_seed(seed)
    d = c["d_model"]
    A = torch.randn(len(keys), 128, d, generator=g)
    out = []
    for _ in range(n):
        z = torch.randn(*shape, 128, generator=g)
        rec = {}
        for i, k in enumerate(keys):
            x = z @ A[i] + 0.1 * torch.randn(*shape, d, generator=g)
            rec[k] = (x * (d**0.5 / x.norm(dim=-1).mean())).to(torch.bfloat16).contiguous().pin_memory()
        out.append(rec)
    return out


def run_config5(args, bench) -> None:
    """Cross-layer transcoder (12 layers x 24576 features, TopK 64 per layer) and low-rank sparse attention (8192 OV heads
    in 64 QK groups of head dimension 64, TopK 128) on a Pythia-160M-shaped model (d_model 768), 2048 tokens per step as two
    sequences of 1024, features / heads sharded over the GPUs. Both dictionaries train on every batch, one after the
    other; the reported value is tokens over the sum of the two step times, and both parts are listed."""
    import torch
    import torch.distributed as dist

    c = dict(C5)
    impl = args.impl
    world, rank, local = (int(os.environ.get(k, d)) for k, d in (("WORLD_SIZE", "1"), ("RANK", "0"), ("LOCAL_RANK", "0")))
    config = {"model": f"CLT {c['layers']} layers x {c['d_model'] * c['clt_expansion']} features TopK {c['clt_k']} + Lorsa {c['lorsa_heads']} OV heads, "
                       f"{c['lorsa_qk']} QK groups d_qk {c['d_qk']}, TopK {c['lorsa_k']}; d_model {c['d_model']}, Adam lr 2e-4, fp32 parameters, bf16 autocast",
              "global_batch": c["batch_tokens"], "seq_len": c["seq"], "parallelism": f"tp{world}", "l2": "inputs rotate through 3 batches"}  # fmt: skip
    metric = "CLT + Lorsa train tokens/s (Pythia-160M shape)"
    try:
        pkg, wrap, build = _arm(impl)
    except Exception as e:  # noqa: BLE001
        bench.emit({"impl": impl, "unavailable": f"{type(e).__name__}: {e}"[:300]})
        return
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    mesh = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        mesh = build((1, world), ("data", "model"))
    D, L, T, S = c["d_model"], c["layers"], c["batch_tokens"], c["seq"]
    W, Ks = args.warmup, args.steps
    lead = 1 if impl == "reference" else 0
    device_name = "cuda" if impl == "reference" else f"cuda:{local}"
    parts: dict[str, dict] = {}
    try:
        ins = [f"blocks.{i}.ln2.hook_normalized" for i in range(L)]
        outs = [f"blocks.{i}.hook_mlp_out" for i in range(L)]
        jobs = []
        clt_kw = dict(hook_points_in=ins, hook_points_out=outs, d_model=D, expansion_factor=c["clt_expansion"], act_fn="topk",
                      top_k=c["clt_k"], device=device_name, dtype=torch.float32)  # fmt: skip
        if impl == "ours" and os.environ.get("LMSAE_BENCH_CLT_CSR", "1") == "1":
            clt_kw["decode_with_csr"] = True
        jobs.append(("clt", pkg.CLTConfig(**clt_kw), ins + outs, (T,), 7))
        lorsa_kw = dict(hook_point_in="blocks.6.ln1.hook_normalized", hook_point_out="blocks.6.hook_attn_out", d_model=D,
                        expansion_factor=c["lorsa_heads"] / D, n_qk_heads=c["lorsa_qk"], d_qk_head=c["d_qk"], rotary_dim=c["d_qk"],
                        n_ctx=S, act_fn="topk", top_k=c["lorsa_k"], device=device_name, dtype=torch.float32)  # fmt: skip
        if impl == "ours" and os.environ.get("LMSAE_BENCH_ATTN", "") in ("library", "tensor_core"):
            lorsa_kw["attention_kernel"] = os.environ["LMSAE_BENCH_ATTN"]
        jobs.append(("lorsa", pkg.LorsaConfig(**lorsa_kw), ["blocks.6.ln1.hook_normalized", "blocks.6.hook_attn_out"], (T // S, S), 8))
        only = os.environ.get("LMSAE_BENCH_C5_PARTS")  # "clt" or "lorsa": run one of the two parts (for launch lists)
        if only:
            jobs = [j for j in jobs if j[0] in only.split(",")]
        for name, cfg, keys, shape, seed in jobs:
            torch.manual_seed(0)
            sae = pkg.SparseDictionary.from_config(cfg, device_mesh=mesh)
            bound = 1.0 / D**0.5
            sae.init_parameters(encoder_uniform_bound=bound, decoder_uniform_bound=bound)
            if hasattr(sae, "set_dataset_average_activation_norm"):
                sae.set_dataset_average_activation_norm({k: D**0.5 for k in keys})
            host = _layer_batches(c, c["pool"], keys, shape, seed)
            pool_dev = [{k: v.to(dev) for k, v in rec.items()} for rec in host]
            tok_h = torch.zeros(*shape, dtype=torch.long).pin_memory()
            tok_d = tok_h.to(dev)
            mask_h = torch.ones(*shape, dtype=torch.bool).pin_memory()
            mask_d = mask_h.to(dev)

            def stream_of(source, on_start, pool_dev=pool_dev, keys=keys, tok_h=tok_h, tok_d=tok_d, mask_h=mask_h, mask_d=mask_d):
                on_device = source is pool_dev

                def gen():
                    for i in range(lead + W + Ks + 2):
                        if i == lead + W + (0 if impl == "reference" else 1):
                            on_start()
                        rec = source[i % len(source)]
                        if impl == "reference":
                            out = {k: wrap((v if on_device else v.to(dev, non_blocking=True)).float(), mesh, None) for k, v in rec.items()}
                            out["tokens"] = wrap(tok_d, mesh, None)
                            out["mask"] = wrap(mask_d, mesh, None)
                        else:
                            out = dict(rec)
                            out["tokens"] = tok_d if on_device else tok_h
                            out["mask"] = mask_d if on_device else mask_h
                        yield out

                return gen()

            def make_trainer():
                tmp = tempfile.mkdtemp()
                extra = dict(prefetch_to_device=True, lr_warm_up_steps=0, lr_cool_down_steps=0) if impl == "ours" else dict(amp_dtype=torch.bfloat16)
                tcfg = pkg.TrainerConfig(total_training_tokens=(W + Ks) * T, lr=c["lr"], lr_scheduler_name="constant",
                                         log_frequency=1 if impl == "ours" else 10**9, skip_metrics_calculation=True, n_checkpoints=0,
                                         exp_result_path=tmp, k_warmup_steps=0, l1_coefficient=None, **extra)  # fmt: skip
                return pkg.Trainer(tcfg)

            res: dict = {}
            _timed_fits(bench, args, world, rank, local, T, make_trainer, sae, stream_of, (pool_dev, host), res)
            parts[name] = res
            del sae, pool_dev, host
            torch.cuda.empty_cache()
    except Exception as e:  # noqa: BLE001
        import traceback

        if rank == 0:
            bench.emit({"impl": impl, "unavailable": f"{type(e).__name__}: {str(e)[:300]}", "config": config,
                        "trace": traceback.format_exc()[-1200:], "finished_parts": {k: v["ms"] / Ks for k, v in parts.items()}})  # fmt: skip
        if world > 1:
            dist.destroy_process_group()
        return
    if rank == 0:
        both = {"ms": sum(p["ms"] for p in parts.values()), "e2e_ms": sum(p["e2e_ms"] for p in parts.values()),
                "clocks": next(iter(parts.values()))["clocks"], "final_loss": list(parts.values())[-1].get("final_loss")}  # fmt: skip
        _emit(bench, impl, metric, config, world, args, T, both, h2d=(2 * L + 2) * T * D * 2 // 1,
              extra={"path": "Trainer.fit(CrossLayerTranscoder), then Trainer.fit(LowRankSparseAttention)", "gpu_launches": _launches(impl),
                     "parts_ms_per_step": {k: {"device_timed": v["ms"] / Ks, "e2e": v["e2e_ms"] / Ks} for k, v in parts.items()}})  # fmt: skip
    if world > 1:
        dist.destroy_process_group()
