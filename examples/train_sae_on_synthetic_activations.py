"""Train a TopK (or BatchTopK) SAE on synthetic activations with ``Trainer.fit``.

    python examples/train_sae_on_synthetic_activations.py [--act batchtopk] [--d-model 1024] [--expansion 16]

On a CUDA device with fp32 parameters this runs on the fused kernel path (five kernels per step, no dense
``[batch, d_sae]`` tensor); pass ``--generic`` to force the autograd path for comparison.
"""

import argparse
import tempfile
import time

import torch

from language_model_saes_b200 import SAEConfig, SparseAutoEncoder, Trainer, TrainerConfig


def stream(n_steps: int, batch: int, d_model: int, device: str, rank: int = 64):
    """Low-rank structure + noise, so that there is something to learn."""
    g = torch.Generator(device=device).manual_seed(0)
    basis = torch.randn(rank, d_model, device=device, generator=g)
    for _ in range(n_steps):
        codes = torch.relu(torch.randn(batch, rank, device=device, generator=g))
        x = codes @ basis + 0.05 * torch.randn(batch, d_model, device=device, generator=g)
        yield {"blocks.0.hook_resid_post": x, "tokens": torch.ones(batch, dtype=torch.long, device=device)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--act", default="topk", choices=["topk", "batchtopk"])
    ap.add_argument("--d-model", type=int, default=1024)
    ap.add_argument("--expansion", type=int, default=16)
    ap.add_argument("--k", type=int, default=32)
    ap.add_argument("--batch", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--generic", action="store_true")
    a = ap.parse_args()
    device = "cuda" if torch.cuda.is_available() else "cpu"
    hp = "blocks.0.hook_resid_post"
    cfg = SAEConfig(hook_point_in=hp, hook_point_out=hp, d_model=a.d_model, expansion_factor=a.expansion, act_fn=a.act, top_k=a.k,
                    device=device, dtype=torch.float32)  # fmt: skip
    sae = SparseAutoEncoder(cfg)
    bound = a.d_model**-0.5
    sae.init_parameters(encoder_uniform_bound=bound, decoder_uniform_bound=bound)
    sae.set_decoder_to_fixed_norm(1.0, force_exact=True)
    sae.init_encoder_with_decoder_transpose()
    sae.set_dataset_average_activation_norm({hp: a.d_model**0.5})
    with tempfile.TemporaryDirectory() as out:
        trainer = Trainer(TrainerConfig(total_training_tokens=a.steps * a.batch, lr=4e-4, lr_warm_up_steps=20, log_frequency=50,
                                        n_checkpoints=0, exp_result_path=out, l1_coefficient=None, k_warmup_steps=0,
                                        use_fused_kernels=not a.generic))  # fmt: skip
        t0 = time.time()
        trainer.fit(sae, stream(a.steps + 1, a.batch, a.d_model, device))
        if device == "cuda":
            torch.cuda.synchronize()
        dt = time.time() - t0
    print(f"{a.steps} steps, {a.steps * a.batch / dt:,.0f} tokens/s, last loss {trainer.last_loss}, fused path: {trainer.fused is not None}")


if __name__ == "__main__":
    main()
