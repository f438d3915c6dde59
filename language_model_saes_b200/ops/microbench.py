"""Micro-benchmarks of the sm_100a kernels: ``python -m language_model_saes_b200.ops.microbench --case all``.

Each case is timed with CUDA events on the launching stream after warm-up, with a synchronise on both
sides; between timed iterations a buffer larger than L2 is written so that every iteration starts with a
cold L2. A case is repeated until ``--min-seconds`` of timed work have accumulated, while a thread samples the SM
clock, power and throttle reasons of the GPU. Prints one JSON object per case: ms (best / mean), achieved TFLOP/s or
GB/s, the fraction of the measured peak when a peaks file is given, and the clock record.

The ``comm_*`` cases run the fused compute + collective kernels of the feature-sharded step as a group of ONE rank
(the peer table points at this GPU's own buffer): same kernels and code paths as between GPUs, which is what a
single-GPU profiler capture can look at.
"""

from __future__ import annotations

import argparse
import json

import torch

from ..utils.clocks import ClockSampler
from . import sae_kernels as K

MIN_SECONDS = 0.0


def _timeit(fn, iters: int, warmup: int, flush: torch.Tensor | None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    while len(ts) < iters or sum(ts) < MIN_SECONDS * 1e3:
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    return min(ts), sum(ts) / len(ts)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all", help="all | cublas | hidden | hidden3 | hidden_pair | topk | topk_pair | merge | decode | csc | adam")
    ap.add_argument("--M", type=int, default=4096)
    ap.add_argument("--N", type=int, default=16384, help="dictionary size on this GPU")
    ap.add_argument("--K", type=int, default=4096, help="d_model")
    ap.add_argument("--k", type=int, default=50)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--peaks", default=None, help="JSON file with hbm_gbs and bf16_tflops")
    ap.add_argument("--min-seconds", type=float, default=0.0, help="repeat every case until this much timed work has accumulated")
    a = ap.parse_args(argv)
    global MIN_SECONDS
    MIN_SECONDS = a.min_seconds

    dev = torch.device("cuda")
    peaks = json.load(open(a.peaks)) if a.peaks else {}
    flush = None if a.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    M, F, d, k = a.M, a.N, a.K, a.k
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(M, d, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(F, d, device=dev, generator=g) / d**0.5).to(torch.bfloat16)
    b = torch.zeros(F, device=dev)
    gate = torch.ones(F, device=dev)
    flops = 2.0 * M * d * F
    want = lambda c: a.case in ("all", c)  # noqa: E731

    def timed(fn):
        sampler = ClockSampler(torch.cuda.current_device())
        sampler.start()
        t = _timeit(fn, a.iters, a.warmup, flush)
        return (*t, sampler.stop())

    def report(name, t, flops=None, bytes_=None):
        rec = {"case": name, "M": M, "N": F, "K": d, "k": k, "ms_best": round(t[0], 4), "ms_mean": round(t[1], 4)}
        if len(t) > 2:
            rec["clocks"] = t[2]
        if flops is not None:
            rec["tflops"] = round(flops / t[0] / 1e9, 1)
            if "bf16_tflops" in peaks:
                rec["frac_of_measured_cublas"] = round(rec["tflops"] / peaks["bf16_tflops"], 3)
        if bytes_ is not None:
            rec["gbs"] = round(bytes_ / t[0] / 1e6, 1)
            if "hbm_gbs" in peaks:
                rec["frac_of_measured_hbm"] = round(rec["gbs"] / peaks["hbm_gbs"], 3)
        print(json.dumps(rec), flush=True)

    if want("cublas"):
        report("cublas_matmul", timed(lambda: x @ w.t()), flops=flops)
    if want("hidden"):
        report("encoder_gemm_write_h", timed(lambda: K.encoder_hidden(x, w, b)), flops=flops)
    if want("hidden3"):
        H3 = torch.empty(M, F, dtype=torch.bfloat16, device=dev)
        st = K.status_buffer(dev)
        fn3 = lambda: K._ext().encoder_gemm(x, w, b, None, 1 | 4, 0, K.choose_splits(M, F), H3, None, None, st, 0, False, 0)  # noqa: E731
        report("encoder_gemm_write_h_3stages", timed(fn3), flops=flops)
        del H3
    if want("hidden_pair"):
        report("encoder_gemm_write_h_pair", timed(lambda: K.encoder_hidden(x, w, b, pair=True)), flops=flops)
    if want("topk_pair") and k <= 64:
        report(
            "encoder_gemm_fused_topk_pair",
            timed(lambda: K.encoder_topk_candidates(x, w, b, gate, k, pair=True)),
            flops=flops,
        )
    if want("topk") and k <= 64:
        report(
            "encoder_gemm_fused_topk",
            timed(lambda: K.encoder_topk_candidates(x, w, b, gate, k)),
            flops=flops,
        )
    K.check_status(dev)
    if a.case in ("cublas", "hidden", "hidden3", "topk", "hidden_pair", "topk_pair"):
        return
    if a.case.startswith("comm"):
        return _comm_cases(a, timed, report, x, w, b, gate, dev)
    kk = min(k, 64)
    cv, ci, _ = K.encoder_topk_candidates(x, w, b, gate, kk)
    if want("merge"):
        report("topk_merge", timed(lambda: K.topk_merge(cv, ci, kk, gate)))
    idx, act = K.topk_merge(cv, ci, kk, gate)
    loss = torch.zeros(1, device=dev)
    if want("decode"):
        report(
            "sparse_decode_loss_dact",
            timed(lambda: K.sparse_decode_loss(idx, act, w, None, x, None, 2.0 / M, loss)),
            bytes_=2.0 * M * kk * d * 2,
        )
    dx, dv, _ = K.sparse_decode_loss(idx, act, w, None, x, None, 2.0 / M, loss)
    groups = K.FeatureGroups(F, M * kk, dev)
    if want("csc"):
        report("csc_build", timed(lambda: groups.build(idx)))
    groups.build(idx)
    if want("adam"):
        WD = torch.randn(F, d, device=dev)
        WE = torch.randn(F, d, device=dev)
        st = [torch.zeros(F, d, device=dev) for _ in range(4)]
        bE = torch.zeros(F, device=dev)
        sb = [torch.zeros(F, device=dev) for _ in range(2)]
        WDb = torch.empty(F, d, dtype=torch.bfloat16, device=dev)
        WEb = torch.empty_like(WDb)
        dn = torch.empty(F, device=dev)
        fn = lambda: K.sparse_grad_adam(  # noqa: E731
            groups, act, dv, x, dx, WD, st[0], st[1], WDb, WE, st[2], st[3], WEb, bE, sb[0], sb[1], dn, None, None,
            1e-4, 0.9, 0.999, 1e-8, 2,
        )  # fmt: skip
        report("sparse_grad_adam", timed(fn), bytes_=2.0 * F * d * 26)


def _comm_cases(a, timed, report, x, w, b, gate, dev):
    """The fused compute + collective kernels of the feature-sharded step over a one-rank group: candidate merge with
    the push epilogue, merge over shards with the in-kernel wait, decode with the reduce-scatter epilogue, owner-side
    reduction + loss + gradient all-gather, code gradient with the in-kernel wait. ``--case comm`` runs all of them;
    ``comm_decode`` only the decode / reduce pair."""
    from ..parallel.symm import PHASE_CAND, PHASE_DXHAT, PHASE_PARTIAL, WaitStats, _NUM_PHASES, peer_table, step_buffer_layout

    M, F, d = x.shape[0], w.shape[0], x.shape[1]
    k = min(a.k, 64)
    lay = step_buffer_layout(M, 1, k, d, 2)
    buf = torch.zeros(lay["nbytes"], dtype=torch.uint8, device=dev)
    stats = WaitStats(dev)
    done = torch.zeros(1, dtype=torch.int32, device=dev)
    st = K.status_buffer(dev)
    ext = K._ext()
    epochs = [0] * _NUM_PHASES

    def table(parity=0):
        off = parity * lay["cand_stride"]
        return peer_table(1, 0, [buf.data_ptr()], lay["flags"], lay["cand_val"] + off, lay["cand_idx"] + off, lay["partial"],
                          lay["dxhat"], 0, stats.buf.data_ptr())  # fmt: skip

    def view(off, shape, dtype):
        n = dtype.itemsize
        for s_ in shape:
            n *= s_
        return buf[off : off + n].view(dtype).view(*shape)

    cv, ci, C = K.encoder_topk_candidates(x, w, b, gate, k)
    out_i = torch.empty(M, k, dtype=torch.int32, device=dev)
    out_v = torch.empty(M, k, dtype=torch.float32, device=dev)
    loss = torch.zeros(1, device=dev)

    def merge_pair():
        epochs[PHASE_CAND] += 1
        e = epochs[PHASE_CAND]
        ext.topk_merge(cv, ci, M, C, k, None, 0, C, True, None, None, 1, table(e & 1), e, done, st)
        off = (e & 1) * lay["cand_stride"]
        ext.topk_merge(view(lay["cand_val"] + off, (M, k), torch.float32), view(lay["cand_idx"] + off, (M, k), torch.int32), M, k, k,
                       gate, 0, k, False, out_i, out_v, 2, table(e & 1), e, None, st)  # fmt: skip

    def decode_pair():
        epochs[PHASE_PARTIAL] += 1
        epochs[PHASE_DXHAT] += 1
        ext.comm_decode_scatter(table(), out_i, out_v, w, 1, False, True, epochs[PHASE_PARTIAL], done)
        ext.comm_reduce_loss_push(table(), M, d, x, None, None, 2.0 / M, loss, None, 1, False, epochs[PHASE_PARTIAL],
                                  epochs[PHASE_DXHAT], done, st)  # fmt: skip

    dval = torch.empty(M, k, dtype=torch.float32, device=dev)

    def dact():
        ext.sparse_dact(out_i, w, view(lay["dxhat"], (M, d), torch.bfloat16), dval, table(), epochs[PHASE_DXHAT], st)

    merge_pair()
    if a.case in ("comm", "comm_merge"):
        report("comm_merge_push_then_merge_shards_world1", timed(merge_pair))
    decode_pair()
    if a.case in ("comm", "comm_decode"):
        report("comm_decode_scatter_then_reduce_loss_push_world1", timed(decode_pair), bytes_=1.0 * M * k * d * 2 + 4.0 * M * d * 2)
    if a.case in ("comm", "comm_dact"):
        report("comm_dact_with_wait_world1", timed(dact), bytes_=1.0 * M * (k + 1) * d * 2)
    K.check_status(dev)


if __name__ == "__main__":
    main()
