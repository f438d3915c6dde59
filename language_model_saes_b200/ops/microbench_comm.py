"""Micro-benchmarks of the peer-memory collectives against the NCCL calls they replace, on 2 to 8 GPUs of one node:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m language_model_saes_b200.ops.microbench_comm --case all

Cases: ``shuffle`` (seeded row all-to-all of the activation buffer, ``ShuffleComm`` vs ``all_to_all_single`` after a
local gather), ``bcast`` (masked + cast row broadcast of cached activations, ``BroadcastComm`` vs boolean index + cast +
``broadcast``), ``headsum`` (crosscoder pre-activation sum: head-summing GEMM into a symmetric buffer + one-kernel all-reduce, ``HeadSumComm``
vs ``einsum`` + ``all_reduce``), ``allreduce``
(in-place sum of a bf16 [4096, 98304] matrix in one kernel, ``AllReduceComm`` with and without the NVSwitch multicast
mapping, vs ``all_reduce``),
``rows`` (the five tensors of a data-parallel step in one kernel, ``DataParallelComm.exchange`` vs five
``all_gather_into_tensor`` calls). ``bcast``, ``allreduce`` and ``rows`` run twice where the group has a multicast
mapping: through the NVSwitch (``multimem``) and by plain peer loads / stores.

Every time is taken on the device with CUDA events after warm-up and is the MAX over ranks; every JSON line carries the
SM clock, power and throttle reasons sampled on rank 0 while the case ran. NVLink bytes are counted per rank and
direction; the link fraction is against the measured peer-copy rate of 770 GB/s.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..utils.clocks import ClockSampler
from . import sae_kernels as K

LINK_GBS = 770.0


def _time(fn, iters: int, warmup: int, min_seconds: float) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    total, n = 0.0, 0
    while n < iters or total < min_seconds * 1e3:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # also keeps the ranks' loop counts in step
        total += float(t)
        n += 1
    return total / n


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all", help="all | shuffle | bcast | headsum | allreduce | rows")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--min-seconds", type=float, default=0.5)
    a = ap.parse_args(argv)
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD
    want = lambda c: a.case in ("all", c)  # noqa: E731

    def run(name, ours, ref, link_bytes, **extra):
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        t_o = _time(ours, a.iters, a.warmup, a.min_seconds)
        t_r = _time(ref, a.iters, a.warmup, a.min_seconds)
        K.check_status(dev)
        if rank == 0:
            print(json.dumps({"case": name, "world": world, "ms_ours": round(t_o, 4), "ms_nccl_path": round(t_r, 4),
                              "speedup": round(t_r / t_o, 2), "nvlink_mb_per_rank": round(link_bytes / 1e6, 1),
                              "fraction_of_link_rate": round(link_bytes / (t_o * 1e-3) / (LINK_GBS * 1e9), 3), **extra,
                              "clocks": sampler.stop()}), flush=True)  # fmt: skip

    from ..parallel import symm

    if want("shuffle"):
        n, d = 32768, 4096  # rows per rank of a bf16 activation buffer (256 MiB per rank)
        x = torch.randn(n, d, device=dev).to(torch.bfloat16)
        comm = symm.ShuffleComm(group, dev, rows_per_rank=n, max_row_bytes=d * 2)
        perm = comm.permutation(n, 11)
        dest = perm[rank * n : (rank + 1) * n].to(dev)
        owner = torch.div(dest, n, rounding_mode="floor")
        order = torch.argsort(owner, stable=True)
        counts = torch.bincount(owner, minlength=world).tolist()
        recv_counts = [torch.zeros(1, dtype=torch.long, device=dev) for _ in range(world)]
        dist.all_to_all(recv_counts, [torch.tensor([c], device=dev) for c in counts])
        recv_counts = [int(c) for c in recv_counts]
        recv = torch.empty(sum(recv_counts), d, dtype=torch.bfloat16, device=dev)

        def nccl_path():  # gather rows by destination rank, exchange, (the final placement by slot is left out: in its favour)
            send = x[order]
            dist.all_to_all_single(recv, send, recv_counts, counts)

        run("shuffle_rows_all_to_all_32768x4096_bf16", lambda: comm.shuffle(x, 11, perm=perm), nccl_path,
            link_bytes=n * d * 2 * (world - 1) / world)  # fmt: skip
        del comm, x, recv

    if want("bcast"):
        n, d = 65536, 4096  # one chunk of cached fp32 activations, a quarter of the tokens masked out, cast to bf16
        src_rows = torch.randn(n, d, device=dev) if rank == 0 else None
        keep = (torch.rand(n, device=dev) > 0.25) if rank == 0 else None
        count = torch.zeros(1, dtype=torch.long, device=dev)
        landing = torch.empty(n, d, dtype=torch.bfloat16, device=dev)

        def nccl_path():
            if rank == 0:
                rows = src_rows[keep].to(torch.bfloat16)
                count.fill_(rows.shape[0])
            dist.broadcast(count, src=0)
            m = int(count)
            if rank == 0:
                landing[:m].copy_(rows)
            dist.broadcast(landing[:m], src=0)

        for use_mc in (True, False):
            comm = symm.BroadcastComm(group, dev, max_rows=n, max_row_bytes=d * 2, use_multicast=use_mc)
            if use_mc and not comm.use_multicast:
                continue
            # bytes the sender puts on its link: once through the switch, once per peer otherwise
            run(f"broadcast_masked_cast_rows_65536x4096_fp32_to_bf16_{'multimem' if use_mc else 'peer_stores'}",
                lambda: comm.broadcast_rows(0, d, torch.bfloat16, src_rows, keep), nccl_path,
                link_bytes=0.75 * n * d * 2 * (1 if use_mc else world - 1))  # fmt: skip
            del comm
        del src_rows, landing

    if want("headsum"):
        M, heads, d, N = 4096, max(1, 8 // world), 768, 98304  # the crosscoder of 8 snapshots, heads spread over the ranks
        x = torch.randn(M, heads * d, device=dev).to(torch.bfloat16)
        w = (torch.randn(heads * N, d, device=dev) / d**0.5).to(torch.bfloat16)
        bias = torch.zeros(N, device=dev)
        comm = symm.HeadSumComm(group, dev, M, N)
        x3, w3 = x.view(M, heads, d), w.view(heads, N, d)

        def nccl_path():
            s = torch.einsum("bhd,hfd->bf", x3, w3)
            dist.all_reduce(s)

        run(f"crosscoder_head_sum_M4096_{heads}heads_per_rank_d768_F98304", lambda: comm.head_sum(x, w, bias, heads, N, torch.bfloat16),
            nccl_path, link_bytes=M * N * 4 * (world - 1) / world + M * N * 2 * (world - 1) / world,
            tflops_ours_per_rank=None)  # fmt: skip
        del comm, x, w

    if want("allreduce"):
        M, N = 4096, 98304  # the crosscoder's summed pre-activations
        mine = torch.randn(M, N, device=dev).to(torch.bfloat16)
        ref_buf = mine.clone()
        for use_mc in (True, False):
            comm = symm.AllReduceComm(group, dev, M, N, use_multicast=use_mc)
            if use_mc and not comm.use_multicast:
                continue
            comm.matrix(M).copy_(mine)
            # (the kernel sums in place: repeated calls keep summing the same buffer, values are irrelevant for the timing)
            run(f"all_reduce_bf16_4096x98304_one_kernel_{'multimem' if comm.use_multicast else 'peer_loads_stores'}",
                lambda: comm.all_reduce(M), lambda: dist.all_reduce(ref_buf), link_bytes=M * N * 2 * (world - 1) / world)
            del comm
        del mine, ref_buf

    if want("rows"):
        B, d, k = 4096, 4096, 64  # rows of one replica: x, d x_hat (bf16) and the three code tensors
        t = {"x": torch.randn(B, d, device=dev).to(torch.bfloat16), "dxhat": torch.randn(B, d, device=dev).to(torch.bfloat16),
             "idx": torch.randint(0, 1 << 17, (B, k), device=dev, dtype=torch.int32), "act": torch.randn(B, k, device=dev),
             "dact": torch.randn(B, k, device=dev)}  # fmt: skip
        zones = {n_: v.numel() * v.element_size() * world for n_, v in t.items()}
        outs = {n_: torch.empty(world * v.shape[0], *v.shape[1:], dtype=v.dtype, device=dev) for n_, v in t.items()}

        def nccl_path():
            for n_, v in t.items():
                dist.all_gather_into_tensor(outs[n_], v)

        per_rank = sum(v.numel() * v.element_size() for v in t.values())
        for use_mc in (True, False):
            comm = symm.DataParallelComm(group, dev, 1024, d, zones, use_multicast=use_mc)
            if use_mc and not comm.use_multicast:
                continue
            # bytes every rank RECEIVES (the side that bounds an all-gather through the switch)
            run(f"data_parallel_row_exchange_5_tensors_B4096_d4096_k64_{'multimem' if use_mc else 'peer_stores'}",
                lambda: comm.exchange(t), nccl_path, link_bytes=per_rank * (world - 1))
            del comm
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
