"""Headline benchmark: SAE training tokens/s, d_model 4096 x d_sae 131072 TopK(k=50), batch 4096, bf16 compute.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--config 3|4|5]

One rank per GPU (launched through torch.distributed.run for N > 1); the dictionary is feature-sharded N ways
("model" mesh dimension) and the global batch stays 4096 tokens, so scaling is strong. Prints ONE JSON line on
rank 0. ``value`` is the device-timed training throughput (CUDA events around exactly K steps, max over
ranks, inputs rotated through a pool of device batches larger than L2); ``e2e`` is the same metric measured
through the public ``Trainer.fit`` call with every step's batch copied from pinned host memory and the loss
read back to the host each step.
"""

from __future__ import annotations

import argparse
import gc
import json
import os
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D_MODEL, EXPANSION, TOP_K, BATCH, LR = 4096, 32, 50, 4096, 2e-4
POOL = 8  # distinct synthetic batches: 8 x 32 MiB bf16 = 256 MiB > 126 MB L2


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4, 5],
                    help="benchmark configuration: 2 = the headline TopK SAE (default); 3, 4, 5: see bench_configs.py")
    return ap.parse_args()


from language_model_saes_b200.utils.clocks import ClockSampler  # noqa: E402


def synthetic_batches(n: int, seed: int = 1234):
    """x = z A + eps with z ~ N(0, I_256), A a seeded 256 x 4096 Gaussian, eps ~ N(0, 0.1^2), rescaled to a mean
    norm of sqrt(4096); bf16, pinned host memory. Every rank generates the same batches."""
    import torch

    g = torch.Generator().manual_seed(seed)
    A = torch.randn(256, D_MODEL, generator=g)
    out = []
    for _ in range(n):
        z = torch.randn(BATCH, 256, generator=g)
        x = z @ A + 0.1 * torch.randn(BATCH, D_MODEL, generator=g)
        x = x * (D_MODEL**0.5 / x.norm(dim=-1).mean())
        out.append(x.to(torch.bfloat16).pin_memory())
    return out


def emit(rec: dict):
    print(json.dumps(rec), flush=True)


def bench_config(world: int) -> dict:
    """The benchmark configuration as both arms report it (identical keys and values)."""
    return {"model": f"TopK SAE d_model {D_MODEL}, d_sae {D_MODEL * EXPANSION}, k {TOP_K}, Adam lr {LR:g}, fp32 parameters, bf16 autocast",
            "global_batch": BATCH, "seq_len": 1, "parallelism": f"tp{world}",
            "l2": f"inputs rotate through {POOL} batches ({POOL * BATCH * D_MODEL * 2 >> 20} MiB) > L2; weights 2 x 2.1 GB"}  # fmt: skip


def measured_peaks() -> dict:
    """Roofline denominators measured on this pool (MEASURED_PEAKS.json beside this file), else the stated fallback."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops_sustained"], "nvlink_gbs": 770.0, "source": "measured"}
    except Exception:  # noqa: BLE001
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1400.0, "nvlink_gbs": 770.0, "source": "fallback"}


def roofline(phases: dict, world: int, partial_itemsize: int) -> dict:
    """Achieved fraction of the roofline of every fused phase of the step: bound = the slowest of its FLOPs at the
    measured tensor throughput, its NVLink bytes (per rank and direction) at the measured peer-copy rate, and its local
    memory bytes at the measured copy bandwidth; fraction = bound / measured phase time (max over ranks)."""
    pk = measured_peaks()
    F_l, B, d, k, N = D_MODEL * EXPANSION // world, BATCH, D_MODEL, TOP_K, world
    far = (N - 1) / N
    model = {
        "encoder_gemm_topk": {"flops": 2.0 * B * d * F_l, "hbm": F_l * d * 2 + B * d * 2},
        "local_merge_push": {"nvlink": B * k * 8 * (N - 1), "hbm": B * 4 * 64 * 8},
        "decode_reduce_loss": {"nvlink": far * B * d * partial_itemsize + far * B * d * 2,
                               "hbm": B * (k / N) * d * 2 + 2 * B * d * partial_itemsize + B * d * 2 / N},
        "dact": {"hbm": B * (k / N + 1) * d * 2},
        "sparse_grad_adam": {"hbm": 26.0 * 2 * F_l * d},
    }  # fmt: skip
    out = {}
    for name, m in model.items():
        if name not in phases:
            continue
        t = phases[name][1]
        bounds = {"tensor": m.get("flops", 0) / (pk["bf16_tflops"] * 1e12) * 1e3,
                  "nvlink": m.get("nvlink", 0) / (pk["nvlink_gbs"] * 1e9) * 1e3,
                  "hbm": m.get("hbm", 0) / (pk["hbm_gbs"] * 1e9) * 1e3}  # fmt: skip
        which = max(bounds, key=bounds.get)
        out[name] = {"ms": round(t, 4), "bound_ms": round(bounds[which], 4), "bound_by": which,
                     "frac_of_" + pk["source"]: round(bounds[which] / t, 3) if t > 0 else None}  # fmt: skip
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    import language_model_saes_b200 as lm
    from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
    from language_model_saes_b200.ops import sae_kernels as K
    from language_model_saes_b200.ops.fused_step import FusedTopKSAEStep
    from language_model_saes_b200.trainer import Trainer, TrainerConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    mesh = None
    if world > 1:
        from language_model_saes_b200.parallel.mesh import build_mesh

        dist.init_process_group("nccl", device_id=dev)
        mesh = build_mesh("cuda", (1, world), ("data", "model"))

    torch.manual_seed(0)
    cfg = SAEConfig(hook_point_in="blocks.16.hook_resid_post", hook_point_out="blocks.16.hook_resid_post",
                    d_model=D_MODEL, expansion_factor=EXPANSION, act_fn="topk", top_k=TOP_K,
                    device=f"cuda:{local}", dtype=torch.float32)  # fmt: skip
    sae = SparseAutoEncoder(cfg, mesh)
    bound = 1.0 / D_MODEL**0.5
    sae.init_parameters(encoder_uniform_bound=bound, decoder_uniform_bound=bound)
    sae.set_decoder_to_fixed_norm(1.0, force_exact=True)
    sae.init_encoder_with_decoder_transpose()
    sae.set_dataset_average_activation_norm({cfg.hook_point_in: D_MODEL**0.5})

    host = synthetic_batches(POOL)
    tokens = torch.zeros(BATCH, dtype=torch.long).pin_memory()
    mask = torch.ones(BATCH, dtype=torch.bool).pin_memory()
    W, Ksteps = args.warmup, args.steps

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed kernel path --------------------------------------------------------------------
    comm = None
    if world > 1 and os.environ.get("LMSAE_BENCH_NCCL", "0") != "1":
        from language_model_saes_b200.parallel.symm import SymmComm

        comm = SymmComm(mesh.get_group("model"), dev, BATCH, TOP_K, D_MODEL,
                        partial_dtype=torch.float32 if os.environ.get("LMSAE_PARTIAL_FP32", "0") == "1" else torch.bfloat16)
    engine = FusedTopKSAEStep(sae, betas=(0.9, 0.999), comm=comm)
    pool = [h.to(dev) for h in host]
    for i in range(W):
        engine.step(pool[i % POOL], pool[i % POOL], TOP_K, LR)
    engine.join()  # the update of a step runs on its own stream: fold it back before timing starts
    K.check_status(dev)
    if comm is not None:
        comm.stats.reset()
    sampler = ClockSampler(local)
    sampler.start()
    gc.collect()
    gc.disable()  # no collector pauses on any rank inside the timed region (a stalled rank stalls its peers' flag waits)
    barrier()
    launches0 = K.kernel_launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # one more event after every step (a marker in the stream, no synchronisation): the spread of the per-step times
    # shows whether a slow average comes from every step or from a few stalls
    marks_ev = [torch.cuda.Event(enable_timing=True) for _ in range(Ksteps)]
    start.record()
    t_issue0 = time.perf_counter()
    for i in range(Ksteps):
        loss = engine.step(pool[(W + i) % POOL], pool[(W + i) % POOL], TOP_K, LR)
        marks_ev[i].record()
    engine.join()  # ... and before it stops: the last step's update is inside the timed region
    end.record()
    host_issue_ms = (time.perf_counter() - t_issue0) * 1e3 / Ksteps  # host time to enqueue one step (no synchronisation)
    barrier()
    gc.enable()
    launches = K.kernel_launch_count() - launches0
    clocks = sampler.stop()
    ms = start.elapsed_time(end)
    per_step = torch.tensor([a.elapsed_time(b) for a, b in zip([start] + marks_ev[:-1], marks_ev)], device=dev, dtype=torch.float64)
    K.check_status(dev)
    final_loss = float(loss)
    # time the kernels of the timed steps spent in bounded waits for their peers' flags (device counters, block 0 of every
    # waiting kernel), converted with the SM clock sampled during the region: the communication the step could not hide
    exposed = None
    if comm is not None:
        waits = comm.stats.read(float(clocks.get("sm_mhz") or clocks.get("sm_max_mhz") or 1965.0))
        ex = torch.tensor([sum(v["ms"] for v in waits.values()) / Ksteps] + [waits.get(n, {"ms": 0.0})["ms"] / Ksteps for n in ("candidates", "partial rows", "gradient rows")],
                          device=dev, dtype=torch.float64)  # fmt: skip
        dist.all_reduce(ex, op=dist.ReduceOp.MAX)
        exposed = {"total": round(float(ex[0]), 4), "candidates": round(float(ex[1]), 4), "partial_rows": round(float(ex[2]), 4),
                   "gradient_rows": round(float(ex[3]), 4)}  # fmt: skip
    partial_itemsize = comm.partial_dtype.itemsize if comm is not None else 4
    step_multicast = bool(comm is not None and comm.use_multicast)
    phases = None
    if os.environ.get("LMSAE_BENCH_PHASES", "1") == "1":  # diagnostics, after and outside the timed region
        engine.start_phase_timing()
        for i in range(Ksteps):
            engine.step(pool[i % POOL], pool[i % POOL], TOP_K, LR)
        pt = engine.phase_times()
        names = list(pt)
        vals = torch.tensor([pt[n] for n in names], device=dev, dtype=torch.float64)
        lo = vals.clone()
        if world > 1:
            dist.all_reduce(vals, op=dist.ReduceOp.MAX)
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        phases = {n: [round(a, 4), round(b, 4)] for n, a, b in zip(names, lo.tolist(), vals.tolist())}  # [min, max] over ranks
    collectives = "none" if world == 1 else ("nccl" if comm is None else
                                             "fused peer-memory kernels, " + ("multimem through the switch" if step_multicast else "peer loads/stores")
                                             + (", bf16 partial rows" if partial_itemsize == 2 else ", fp32 partial rows"))  # fmt: skip
    del engine, pool, comm
    torch.cuda.empty_cache()

    # ---- end to end through Trainer.fit --------------------------------------------------------------
    marks: dict[str, float] = {}

    # The trainer keeps one batch in flight (its host->device copy overlaps the previous step), so batch W + 1 is
    # drawn from the stream just before step W is launched: the clock starts there and covers steps W .. W + K - 1.
    def stream():
        for i in range(W + Ksteps + 2):
            if i == W + 1:
                barrier()
                marks["t0"] = time.perf_counter()
            yield {cfg.hook_point_in: host[i % POOL], "tokens": tokens, "mask": mask}

    with tempfile.TemporaryDirectory() as tmp:
        tcfg = TrainerConfig(total_training_tokens=(W + Ksteps) * BATCH, lr=LR, lr_warm_up_steps=0, lr_cool_down_steps=0,
                             lr_scheduler_name="constant", log_frequency=1, skip_metrics_calculation=True,
                             n_checkpoints=0, exp_result_path=tmp, k_warmup_steps=0, l1_coefficient=None,
                             prefetch_to_device=True)  # fmt: skip
        trainer = Trainer(tcfg)
        trainer.fit(sae, stream())
        barrier()
        marks["t1"] = time.perf_counter()
    e2e_s = marks["t1"] - marks["t0"]

    t = torch.tensor([ms, e2e_s * 1e3], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = t.tolist()
    if world > 1:
        dist.all_reduce(per_step, op=dist.ReduceOp.MAX)
    step_ms = {"min": round(float(per_step.min()), 4), "median": round(float(per_step.median()), 4),
               "max": round(float(per_step.max()), 4), "slowest_step": int(per_step.argmax())}  # fmt: skip
    if rank == 0:
        value = Ksteps * BATCH / (ms / 1e3)
        emit({
            "metric": "SAE train tokens/s (d4096 x 131072 TopK k50)", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": Ksteps, "warmup": W, "ms_per_step": ms / Ksteps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": bench_config(world), "collectives": collectives,
            "clocks": clocks,
            "e2e": {"value": Ksteps * BATCH / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / Ksteps,
                    # every rank copies 1/N of the activation rows (then NVLink all-gather) and the whole token-id vector
                    "h2d_bytes_per_step": BATCH * D_MODEL * 2 + world * BATCH * 9, "d2h_bytes_per_step": 4 * world,
                    "api": "Trainer.fit(sae, stream of pinned host batches): copy of batch i+1 overlaps step i, each rank copies "
                           "1/N of the rows over PCIe and all-gathers them over NVLink; the loss of every step is copied to pinned host memory "
                           "on every rank and read one step later, so the host runs one step ahead of the device"},
            "gpu_launches": launches, "host_issue_ms_per_step": round(host_issue_ms, 4), "step_ms": step_ms, **({"phase_ms_min_max_over_ranks": phases, "roofline": roofline(phases, world, partial_itemsize)} if phases else {}),
            **({"exposed_comm_ms_per_step": exposed["total"], "exposed_comm_ms_per_step_by_phase": exposed} if exposed else {"exposed_comm_ms_per_step": 0.0}),
            "final_loss": final_loss, "impl": "ours",
            "package": lm.__name__,
        })  # fmt: skip
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.config != 2:
        import bench_configs

        getattr(bench_configs, f"run_config{args.config}")(args, sys.modules[__name__])
        return
    if args.impl == "reference":
        from baseline.reference_arm import run_reference

        run_reference(args, emit, synthetic_batches, ClockSampler,
                      dict(d_model=D_MODEL, expansion=EXPANSION, top_k=TOP_K, batch=BATCH, lr=LR, pool=POOL,
                           config=bench_config(int(os.environ.get("WORLD_SIZE", "1")))))
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
