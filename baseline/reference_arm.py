"""`bench.py --impl reference`: the unmodified reference project driven through its own public API.

The reference (installed under ``baseline/_ref``) is imported with stand-ins for the third-party packages it
needs at import time but that are absent here (``baseline/_stubs``); its own sources are untouched. The arm
builds the reference ``SparseAutoEncoder`` + ``Trainer`` for the benchmark configuration and calls
``Trainer.fit`` on a synthetic activation stream: once with device-resident inputs (device-timed ``value``) and
once with pinned host inputs copied every step (``e2e``). None of this repository's models, kernels or engine
is on that path.
"""

from __future__ import annotations

import os
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))


def run_reference(args, emit, synthetic_batches, ClockSampler, c):
    ref_dir = os.path.join(HERE, "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "llamascopium")):
        emit({"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --target baseline/_ref failed or was not run)"})
        return
    sys.path[:0] = [os.path.join(HERE, "_stubs"), ref_dir]
    try:
        import torch
        import torch.distributed as dist
        from llamascopium import SAEConfig, SparseAutoEncoder, Trainer, TrainerConfig
        from llamascopium.utils.distributed import DimMap
    except Exception as e:  # noqa: BLE001
        emit({"impl": "reference", "unavailable": f"reference does not import here: {type(e).__name__}: {e}"[:300]})
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    mesh = None
    if world > 1:
        from torch.distributed.device_mesh import init_device_mesh

        dist.init_process_group("nccl", device_id=dev)
        mesh = init_device_mesh("cuda", (1, world), mesh_dim_names=("data", "model"))

    D, B, k = c["d_model"], c["batch"], c["top_k"]
    hook = "blocks.16.hook_resid_post"
    torch.manual_seed(0)
    cfg = SAEConfig(hook_point_in=hook, hook_point_out=hook, d_model=D, expansion_factor=c["expansion"], act_fn="topk",
                    top_k=k, device="cuda", dtype=torch.float32)  # fmt: skip
    sae = SparseAutoEncoder(cfg, device_mesh=mesh)
    bound = 1.0 / D**0.5
    sae.init_parameters(encoder_uniform_bound=bound, decoder_uniform_bound=bound)
    sae.set_decoder_to_fixed_norm(1.0, force_exact=True)
    sae.init_encoder_with_decoder_transpose()
    sae.set_dataset_average_activation_norm({hook: D**0.5})

    host = synthetic_batches(c["pool"])
    W, K = args.warmup, args.steps

    def wrap(t):
        return DimMap({"data": 0}).from_local(t, mesh) if mesh is not None else t

    tokens = torch.zeros(B, dtype=torch.long, device=dev)
    mask = torch.ones(B, dtype=torch.bool, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def fit_once(source, record):
        """source(i) -> activation tensor on the device for step i. The reference consumes one batch while
        sizing its schedule, hence the extra leading batch."""

        def stream():
            yield {hook: wrap(source(0).float()), "tokens": wrap(tokens), "mask": wrap(mask)}
            for i in range(W + K + 1):
                if i == W:
                    barrier()
                    record("start")
                yield {hook: wrap(source(i).float()), "tokens": wrap(tokens), "mask": wrap(mask)}

        with tempfile.TemporaryDirectory() as tmp:
            tcfg = TrainerConfig(total_training_tokens=(W + K) * B, lr=c["lr"], lr_scheduler_name="constant",
                                 log_frequency=10**9, skip_metrics_calculation=True, n_checkpoints=0, exp_result_path=tmp,
                                 k_warmup_steps=0, l1_coefficient=None, amp_dtype=torch.bfloat16)  # fmt: skip
            Trainer(tcfg).fit(sae, stream())
        barrier()
        record("end")

    # (a) device-resident inputs, CUDA events
    pool = [h.to(dev) for h in host]
    ev = {}

    def rec_events(name):
        ev[name] = torch.cuda.Event(enable_timing=True)
        ev[name].record()
        ev[name + "_wall"] = time.perf_counter()

    sampler = ClockSampler(local)
    sampler.start()
    fit_once(lambda i: pool[i % len(pool)], rec_events)
    clocks = sampler.stop()
    torch.cuda.synchronize()
    ms = ev["start"].elapsed_time(ev["end"])
    del pool
    torch.cuda.empty_cache()

    # (b) pinned host inputs copied every step
    wall = {}
    fit_once(lambda i: host[i % len(host)].to(dev, non_blocking=True), lambda name: wall.__setitem__(name, time.perf_counter()))
    e2e_ms = (wall["end"] - wall["start"]) * 1e3

    t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    if rank == 0:
        emit({
            "impl": "reference", "metric": "SAE train tokens/s (d4096 x 131072 TopK k50)", "value": K * B / (ms / 1e3),
            "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": c["config"], "path": "llamascopium.Trainer.fit(SparseAutoEncoder), skip_metrics_calculation=True",
            "clocks": clocks,
            "e2e": {"value": K * B / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / K,
                    "h2d_bytes_per_step": B * D * 2, "d2h_bytes_per_step": 4},
            "gpu_launches": 0, "note": "library kernels only (cuBLAS / ATen / NCCL); third-party import stand-ins in baseline/_stubs",
        })  # fmt: skip
    if world > 1:
        dist.destroy_process_group()
