"""Train a TopK SAE from an activation cache.

    python examples/train_topk_sae_from_cache.py
    torchrun --nproc-per-node 8 examples/train_topk_sae_from_cache.py --model-parallel 8   # dictionary split over 8 GPUs

With ``model_parallel_size > 1`` every rank holds 1/N of the dictionary; on the fused path the top-k candidates, the
partial reconstructions and the reconstruction gradient cross NVLink from inside the compute kernels.
"""

import argparse

import torch

from language_model_saes_b200 import (
    ActivationFactoryActivationsSource,
    ActivationFactoryConfig,
    InitializerConfig,
    SAEConfig,
    TrainerConfig,
    TrainSAESettings,
    train_sae,
)
from language_model_saes_b200.activation.factory import ActivationFactoryTarget
from language_model_saes_b200.activation.processors.activation import BufferShuffleConfig

ap = argparse.ArgumentParser()
ap.add_argument("--model-parallel", type=int, default=1)
ap.add_argument("--data-parallel", type=int, default=1)
args = ap.parse_args()

hook = "blocks.6.hook_resid_post"
settings = TrainSAESettings(
    sae=SAEConfig(hook_point_in=hook, hook_point_out=hook, d_model=768, expansion_factor=32, act_fn="topk", top_k=50,
                  dtype=torch.float32, device="cuda"),  # fmt: skip
    sae_name="pythia-160m-L6R-32x-topk50",
    sae_series="examples",
    initializer=InitializerConfig(grid_search_init_norm=True, init_encoder_with_decoder_transpose=True),
    trainer=TrainerConfig(total_training_tokens=800_000_000, lr=4e-4, lr_warm_up_steps=5000, initial_k=768 / 2, k_warmup_steps=0.1,
                          log_frequency=1000, n_checkpoints=5, exp_result_path="results/pythia-160m-L6R-32x-topk50"),  # fmt: skip
    activation_factory=ActivationFactoryConfig(
        sources=[ActivationFactoryActivationsSource(name="cache", path="activations/pythia-160m", device="cuda", num_workers=4,
                                                    peer_broadcast=args.model_parallel > 1)],  # fmt: skip
        target=ActivationFactoryTarget.ACTIVATIONS_1D,
        hook_points=[hook],
        batch_size=4096,
        buffer_size=4096 * 16,
        buffer_shuffle=BufferShuffleConfig(perm_seed=42, generator_device="cuda", cross_rank=args.data_parallel > 1),
    ),
    model_parallel_size=args.model_parallel,
    data_parallel_size=args.data_parallel,
)

if __name__ == "__main__":
    train_sae(settings)
