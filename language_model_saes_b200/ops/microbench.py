"""Micro-benchmarks of the sm_100a kernels: ``python -m language_model_saes_b200.ops.microbench --case all``.

Each case is timed with CUDA events on the launching stream after warm-up, with a synchronise on both
sides; between timed iterations a buffer larger than L2 is written so that every iteration starts with a
cold L2. Prints one JSON object per case: ms (best / mean), achieved TFLOP/s or GB/s, and the fraction of
the measured peak when a peaks file is given.
"""

from __future__ import annotations

import argparse
import json

import torch

from . import sae_kernels as K


def _timeit(fn, iters: int, warmup: int, flush: torch.Tensor | None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
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
    a = ap.parse_args(argv)

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

    def report(name, t, flops=None, bytes_=None):
        rec = {"case": name, "M": M, "N": F, "K": d, "k": k, "ms_best": round(t[0], 4), "ms_mean": round(t[1], 4)}
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
        report("cublas_matmul", _timeit(lambda: x @ w.t(), a.iters, a.warmup, flush), flops=flops)
    if want("hidden"):
        report("encoder_gemm_write_h", _timeit(lambda: K.encoder_hidden(x, w, b), a.iters, a.warmup, flush), flops=flops)
    if want("hidden3"):
        H3 = torch.empty(M, F, dtype=torch.bfloat16, device=dev)
        st = K.status_buffer(dev)
        fn3 = lambda: K._ext().encoder_gemm(x, w, b, None, 1 | 4, 0, K.choose_splits(M, F), H3, None, None, st, 0, False)  # noqa: E731
        report("encoder_gemm_write_h_3stages", _timeit(fn3, a.iters, a.warmup, flush), flops=flops)
        del H3
    if want("hidden_pair"):
        report("encoder_gemm_write_h_pair", _timeit(lambda: K.encoder_hidden(x, w, b, pair=True), a.iters, a.warmup, flush), flops=flops)
    if want("topk_pair") and k <= 64:
        report(
            "encoder_gemm_fused_topk_pair",
            _timeit(lambda: K.encoder_topk_candidates(x, w, b, gate, k, pair=True), a.iters, a.warmup, flush),
            flops=flops,
        )
    if want("topk") and k <= 64:
        report(
            "encoder_gemm_fused_topk",
            _timeit(lambda: K.encoder_topk_candidates(x, w, b, gate, k), a.iters, a.warmup, flush),
            flops=flops,
        )
    K.check_status(dev)
    if a.case in ("cublas", "hidden", "hidden3", "topk", "hidden_pair", "topk_pair"):
        return
    kk = min(k, 64)
    cv, ci, _ = K.encoder_topk_candidates(x, w, b, gate, kk)
    if want("merge"):
        report("topk_merge", _timeit(lambda: K.topk_merge(cv, ci, kk, gate), a.iters, a.warmup, flush))
    idx, act = K.topk_merge(cv, ci, kk, gate)
    loss = torch.zeros(1, device=dev)
    if want("decode"):
        report(
            "sparse_decode_loss_dact",
            _timeit(lambda: K.sparse_decode_loss(idx, act, w, None, x, None, 2.0 / M, loss), a.iters, a.warmup, flush),
            bytes_=2.0 * M * kk * d * 2,
        )
    dx, dv, _ = K.sparse_decode_loss(idx, act, w, None, x, None, 2.0 / M, loss)
    groups = K.FeatureGroups(F, M * kk, dev)
    if want("csc"):
        report("csc_build", _timeit(lambda: groups.build(idx), a.iters, a.warmup, flush))
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
        report("sparse_grad_adam", _timeit(fn, a.iters, a.warmup, flush), bytes_=2.0 * F * d * 26)


if __name__ == "__main__":
    main()
