"""The fused TopK-SAE training step driven directly, timed with CUDA events.

    python examples/fused_step_throughput.py --d-model 4096 --expansion 32 --k 50 --batch 4096
"""

import argparse

import torch

from language_model_saes_b200 import SAEConfig, SparseAutoEncoder
from language_model_saes_b200.ops import sae_kernels as K
from language_model_saes_b200.ops.fused_step import FusedTopKSAEStep


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--expansion", type=int, default=32)
    ap.add_argument("--k", type=int, default=50)
    ap.add_argument("--batch", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=20)
    a = ap.parse_args()
    hp = "h"
    cfg = SAEConfig(hook_point_in=hp, hook_point_out=hp, d_model=a.d_model, expansion_factor=a.expansion, act_fn="topk", top_k=a.k,
                    device="cuda", dtype=torch.float32)  # fmt: skip
    sae = SparseAutoEncoder(cfg)
    sae.init_parameters(encoder_uniform_bound=a.d_model**-0.5, decoder_uniform_bound=a.d_model**-0.5)
    sae.set_decoder_to_fixed_norm(1.0, force_exact=True)
    sae.init_encoder_with_decoder_transpose()
    engine = FusedTopKSAEStep(sae)
    batches = [torch.randn(a.batch, a.d_model, device="cuda").to(torch.bfloat16) for _ in range(8)]  # more than the L2 holds
    for i in range(3):
        engine.step(batches[i], batches[i], a.k, 2e-4)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for i in range(a.steps):
        loss = engine.step(batches[i % 8], batches[i % 8], a.k, 2e-4)
    engine.join()
    end.record()
    torch.cuda.synchronize()
    K.check_status(torch.device("cuda"))
    ms = start.elapsed_time(end) / a.steps
    print(f"{ms:.3f} ms/step, {a.batch / ms * 1e3:,.0f} tokens/s, loss {float(loss):.4f}, {K.kernel_launch_count()} kernel launches in total")


if __name__ == "__main__":
    main()
