"""Micro-benchmarks of the kernels behind the other dictionary families and the batch-level selections, each against
the library path it replaces: ``python -m language_model_saes_b200.ops.microbench_families --case all``.

Timing as in ``ops.microbench``: CUDA events on the launching stream after warm-up, a synchronise on both sides, and
a buffer larger than L2 written between timed iterations. One JSON object per line.
"""

from __future__ import annotations

import argparse
import json

import torch
import torch.nn.functional as F

from . import attention as A
from . import clt_kernels as CK
from . import sae_kernels as K
from . import select_kernels as S
from ..utils.clocks import ClockSampler
from . import microbench as _mb
from .microbench import _timeit


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all", help="all | attn | attn_fwd | batchtopk | batchtopk_step | clt | clt_adam | compact | headsum")
    ap.add_argument("--attn-shape", default="4,1024,64,64,128", help="batch,seq,heads,d_qk,d_v of the attention cases")
    ap.add_argument("--clt-layers", type=int, default=12, help="source layers of the clt_adam case (rows = layers x 24576)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--min-seconds", type=float, default=1.0, help="repeat every timed case until this much timed work has accumulated")
    a = ap.parse_args(argv)
    _mb.MIN_SECONDS = a.min_seconds
    dev = torch.device("cuda")
    # one clock record per report: SM clock (median under load), power, throttle reasons since the previous report
    sampler = [ClockSampler(torch.cuda.current_device())]
    sampler[0].start()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    want = lambda c: a.case in ("all", c)  # noqa: E731

    def report(name, ours, ref, **extra):
        rec = {"case": name, "ms_ours": round(ours[0], 4), "ms_reference_path": round(ref[0], 4),
               "speedup": round(ref[0] / ours[0], 2), **extra, "clocks": sampler[0].stop()}  # fmt: skip
        print(json.dumps(rec), flush=True)
        sampler[0] = ClockSampler(torch.cuda.current_device())
        sampler[0].start()

    if want("attn") or a.case == "attn_fwd":
        # default: low-rank sparse attention at d_sae 8192: 64 QK heads of width 64, OV groups of 128, 4 x 1024 tokens
        b, s, h, dqk, dv = (int(t) for t in a.attn_shape.split(","))
        q, k = (torch.randn(b, s, h, dqk, device=dev, dtype=torch.bfloat16).requires_grad_() for _ in range(2))
        v = torch.randn(b, s, h, dv, device=dev, dtype=torch.bfloat16).requires_grad_()
        do = torch.randn(b, s, h, dv, device=dev, dtype=torch.bfloat16)
        scale = dqk**-0.5

        def sdpa():
            return F.scaled_dot_product_attention(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3),
                                                  scale=scale, is_causal=True).permute(0, 2, 1, 3)  # fmt: skip

        def train(fn):
            out = fn()
            out.backward(do)
            q.grad = k.grad = v.grad = None

        flops_fwd = 2.0 * b * h * s * s * (dqk + dv) / 2  # causal: half of the score matrix
        with torch.no_grad():
            t_o = _timeit(lambda: A.causal_attention_fwd(q, k, v, scale), a.iters, a.warmup, flush)
            t_r = _timeit(sdpa, a.iters, a.warmup, flush)
        tag = f"b{b}_s{s}_h{h}_dqk{dqk}_dv{dv}"
        with torch.no_grad():  # the kernel alone, operands already laid out (values transposed to [b, h, d_v, s])
            vt = v.detach().permute(0, 2, 3, 1).contiguous()
            out = torch.empty(b, s, h, dv, dtype=torch.bfloat16, device=dev)
            lse = torch.empty(b, h, s, dtype=torch.float32, device=dev)
            st = K.status_buffer(dev)
            qd, kd = q.detach(), k.detach()
            t_k = _timeit(lambda: K._ext().attn_fwd(qd, kd, vt, out, lse, scale, st), a.iters, a.warmup, flush)
            t_t = _timeit(lambda: v.detach().permute(0, 2, 3, 1).contiguous(), a.iters, a.warmup, flush)
        print(json.dumps({"case": f"attention_fwd_kernel_only_{tag}", "ms_kernel": round(t_k[0], 4), "ms_value_transpose": round(t_t[0], 4),
                          "tflops_kernel": round(flops_fwd / t_k[0] / 1e9, 1)}), flush=True)  # fmt: skip
        report(f"attention_fwd_{tag}", t_o, t_r, tflops_ours=round(flops_fwd / t_o[0] / 1e9, 1),
               tflops_reference_path=round(flops_fwd / t_r[0] / 1e9, 1))  # fmt: skip
        if a.case != "attn_fwd":
            t_o = _timeit(lambda: train(lambda: A.causal_attention(q, k, v, scale)), a.iters, a.warmup, flush)
            t_r = _timeit(lambda: train(sdpa), a.iters, a.warmup, flush)
            report(f"attention_fwd_bwd_{tag}", t_o, t_r, tflops_ours=round(3.5 * flops_fwd / t_o[0] / 1e9, 1))
        K.check_status(dev)
        del q, k, v, do

    if want("batchtopk"):
        for dtype in (torch.float32, torch.bfloat16):
            B, N, k = 4096, 32768, 50
            x = torch.randn(B, N, device=dev).relu_().to(dtype)
            t_o = _timeit(lambda: S.positive_topk(x, k * B, (0, 1)), a.iters, a.warmup, flush)
            from ..utils.math import topk

            t_r = _timeit(lambda: topk(x, k=k * B, dim=(0, 1), abs=True), max(2, a.iters // 2), 1, flush)
            report(f"batchtopk_mask_4096x32768_k50_{str(dtype).split('.')[-1]}", t_o, t_r,
                   gbs_ours=round(x.numel() * x.element_size() * 4 / t_o[0] / 1e6, 1))  # fmt: skip
            del x

    if want("clt"):
        B, L, Fd, d, k = 4096, 12, 8192, 768, 32
        w16 = [(torch.randn(t + 1, Fd, d, device=dev) / d**0.5).to(torch.bfloat16) for t in range(L)]
        acts = torch.zeros(B, L * Fd, device=dev, dtype=torch.bfloat16)
        cols = torch.randint(0, L * Fd, (B, k * L), device=dev)
        acts.scatter_(1, cols, torch.rand(B, k * L, device=dev).to(torch.bfloat16) + 0.1)
        acts = acts.view(B, L, Fd)
        idx, val = S.dense_rows_to_sparse(acts.view(B, L * Fd))

        def dense():
            return torch.stack([torch.einsum("blf,lfd->bd", acts[:, : t + 1], w16[t]) for t in range(L)])

        t_o = _timeit(lambda: CK.clt_decode(idx, val, w16, None, torch.bfloat16), a.iters, a.warmup, flush)
        t_r = _timeit(dense, a.iters, a.warmup, flush)
        report("clt_decode_fanout_B4096_L12_F8192_d768_k32perlayer", t_o, t_r)
        t_c = _timeit(lambda: S.dense_rows_to_sparse(acts.view(B, L * Fd)), a.iters, a.warmup, flush)
        print(json.dumps({"case": "row_compact_4096x98304_bf16", "ms_ours": round(t_c[0], 4),
                          "gbs": round(acts.numel() * 2 * 2 / t_c[0] / 1e6, 1)}), flush=True)  # fmt: skip
        dy = torch.randn(L, B, d, device=dev).to(torch.bfloat16)
        t_g = _timeit(lambda: (CK.clt_dact(idx, w16, dy), CK.clt_wgrad(idx, val, dy, L, Fd)), a.iters, a.warmup, flush)
        print(json.dumps({"case": "clt_backward_dact_wgrad", "ms_ours": round(t_g[0], 4)}), flush=True)
        del w16, acts, dy

    if want("clt_adam"):
        # decoder-side sparse gradient + Adam of a cross-layer transcoder's last target layer: 12 source layers x 24576
        # features, rows of 768 columns, 64 codes per token and source layer on 2048 tokens (5.3 codes per feature)
        B, L, Fd, d, k = 2048, a.clt_layers, 24576, 768, 64
        n_feat = L * Fd
        idx = torch.cat([torch.randint(0, Fd, (B, k), device=dev, dtype=torch.int32) + l * Fd for l in range(L)], dim=1).contiguous()
        act = torch.rand(B, L * k, device=dev)
        dy = torch.randn(B, d, device=dev).to(torch.bfloat16)
        W = torch.randn(n_feat, d, device=dev) / d**0.5
        m, v = torch.zeros_like(W), torch.zeros_like(W)
        W16 = W.to(torch.bfloat16)
        acc = torch.zeros(n_feat, device=dev)
        groups = K.FeatureGroups(n_feat, idx.numel(), dev).build(idx)
        step = [0]

        def decoder_side():
            step[0] += 1
            K.sparse_grad_adam(groups, act, act, dy, dy, W, m, v, W16, None, None, None, None, None, None, None, None, None, None,
                               2e-4, 0.9, 0.999, 1e-8, step[0], True, norm_sq_accum=acc)  # fmt: skip

        t = _timeit(decoder_side, a.iters, a.warmup, flush)
        gbs = n_feat * d * 26 / t[0] / 1e6
        print(json.dumps({"case": f"sparse_grad_adam_decoder_side_{n_feat}x768_5codes_per_feature", "ms_ours": round(t[0], 4), "gbs": round(gbs, 1),
                          "fraction_of_measured_copy": round(gbs / 6547.2, 3), "clocks": sampler[0].stop()}), flush=True)  # fmt: skip
        sampler[0] = ClockSampler(torch.cuda.current_device())
        sampler[0].start()
        del W, m, v, W16

    if want("compact"):
        n, d = 1 << 20, 1024
        src = torch.randn(n, d, device=dev)
        keep = torch.rand(n, device=dev) > 0.1
        t_o = _timeit(lambda: S.compact_rows(src, keep, torch.bfloat16), a.iters, a.warmup, flush)
        t_r = _timeit(lambda: src[keep].to(torch.bfloat16), a.iters, a.warmup, flush)
        report("mask_compact_cast_1Mx1024_fp32_to_bf16", t_o, t_r, gbs_ours=round(n * d * 0.9 * 6 / t_o[0] / 1e6, 1))
        del src

    if want("batchtopk_step"):
        # one training step of a BatchTopK SAE: the fused kernel sequence against autograd + torch.optim.Adam on the same model
        import copy

        from ..models.sae import SAEConfig, SparseAutoEncoder
        from .fused_step import FusedTopKSAEStep

        d, expansion, k, B, lr = 4096, 8, 50, 4096, 2e-4
        cfg = SAEConfig(hook_point_in="h", hook_point_out="h", d_model=d, expansion_factor=expansion, act_fn="batchtopk", top_k=k,
                        device="cuda", dtype=torch.float32)  # fmt: skip
        ref = SparseAutoEncoder(cfg)
        ref.init_parameters(encoder_uniform_bound=d**-0.5, decoder_uniform_bound=d**-0.5)
        ref.set_decoder_to_fixed_norm(1.0, True)
        ref.init_encoder_with_decoder_transpose()
        ref.set_dataset_average_activation_norm({"h": d**0.5})
        fused_model = copy.deepcopy(ref)
        fused_model.activation_function = fused_model.activation_function_factory(None)
        engine = FusedTopKSAEStep(fused_model)
        x = torch.randn(B, d, device=dev).to(torch.bfloat16)
        tokens = torch.zeros(B, dtype=torch.long, device=dev)
        opt = torch.optim.Adam(ref.parameters(), lr=lr)

        def generic():
            opt.zero_grad(set_to_none=True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = ref.compute_loss({"h": x.float(), "tokens": tokens})["loss"]
            loss.backward()
            opt.step()

        t_o = _timeit(lambda: engine.step(x, x, k, lr), a.iters, a.warmup, flush)
        t_r = _timeit(generic, a.iters, a.warmup, flush)
        report(f"batchtopk_sae_train_step_d{d}_F{d * expansion}_k{k}_B{B}", t_o, t_r, tokens_per_s_ours=round(B / t_o[0] * 1e3))
        K.check_status(dev)
        del ref, fused_model, engine, opt

    if want("headsum"):
        from ..parallel.symm import HeadSumComm

        M, heads, d, N = 4096, 4, 768, 24576
        x = torch.randn(M, heads * d, device=dev).to(torch.bfloat16)
        w = (torch.randn(heads * N, d, device=dev) / d**0.5).to(torch.bfloat16)
        bias = torch.zeros(N, device=dev)
        comm = HeadSumComm(None, dev, M, N)
        t_o = _timeit(lambda: comm.head_sum(x, w, bias, heads, N, torch.bfloat16), a.iters, a.warmup, flush)
        x3, w3 = x.view(M, heads, d), w.view(heads, N, d)
        t_r = _timeit(lambda: torch.einsum("bhd,hfd->bhf", x3, w3).sum(1), a.iters, a.warmup, flush)
        report("crosscoder_head_sum_gemm_M4096_4heads_d768_F24576", t_o, t_r,
               tflops_ours=round(2.0 * M * heads * d * N / t_o[0] / 1e9, 1))  # fmt: skip
        K.check_status(dev)


    sampler[0].stop()


if __name__ == "__main__":
    main()
