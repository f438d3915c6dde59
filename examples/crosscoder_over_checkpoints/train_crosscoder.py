"""Train one crosscoder over the snapshots' caches.

    torchrun --nproc-per-node 8 examples/crosscoder_over_checkpoints/train_crosscoder.py --size 160m --layer 6 \
        --head-parallel 8 --lr 5e-5 --l1-coefficient 0.3 --jumprelu-lr-factor 0.1 --expansion-factor 32 --batch-size 2048
"""

import os

import torch
from common import D_MODEL, arguments, cache_dir

from language_model_saes_b200 import (
    ActivationFactoryActivationsSource,
    ActivationFactoryConfig,
    CrosscoderConfig,
    InitializerConfig,
    TrainCrosscoderSettings,
    TrainerConfig,
    train_crosscoder,
)
from language_model_saes_b200.activation.factory import ActivationFactoryTarget

if __name__ == "__main__":
    args = arguments(head_parallel=dict(type=int, default=1), lr=dict(type=float, default=5e-5), l1_coefficient=dict(type=float, default=0.3),
                     jumprelu_lr_factor=dict(type=float, default=0.1), expansion_factor=dict(type=int, default=32),
                     batch_size=dict(type=int, default=2048), total_tokens=dict(type=int, default=800_000_000),
                     sparsity_loss_type=dict(default="tanh-quad", choices=["tanh", "tanh-quad", "power"]),
                     init_encoder_factor=dict(type=float, default=1.0))  # fmt: skip
    n, ranks = len(args.steps), args.head_parallel
    assert n % ranks == 0, "the snapshots must split evenly over the head-parallel ranks"
    per_rank = n // ranks
    # heads are named "<snapshot>/<hook point>"; rank r of the head dimension reads the caches of its own snapshots only
    heads = [f"{step}/{args.hook}" for step in args.steps]
    factories = [
        ActivationFactoryConfig(
            sources=[ActivationFactoryActivationsSource(name="cache", device="cuda", dtype=torch.bfloat16, num_workers=4, prefetch=4,
                                                        path={h: os.path.join(cache_dir(args, h.split("/")[0], "1d"), args.hook)
                                                              for h in heads[r * per_rank : (r + 1) * per_rank]})],
            target=ActivationFactoryTarget.ACTIVATIONS_1D, hook_points=heads[r * per_rank : (r + 1) * per_rank], batch_size=args.batch_size,
        ) for r in range(ranks)
    ]  # fmt: skip
    name = f"pythia-{args.size}-L{args.layer}R-{n}snapshots-{args.expansion_factor}x-lr{args.lr}-l1c{args.l1_coefficient}"
    train_crosscoder(TrainCrosscoderSettings(
        sae=CrosscoderConfig(hook_points=heads, d_model=D_MODEL[args.size], expansion_factor=args.expansion_factor, act_fn="jumprelu",
                             jumprelu_threshold_window=4.0, dtype=torch.float32, device="cuda"),
        initializer=InitializerConfig(grid_search_init_norm=True, init_encoder_with_decoder_transpose_factor=args.init_encoder_factor,
                                      init_log_jumprelu_threshold_value=-2.0),
        trainer=TrainerConfig(lr=args.lr, initial_k=None, l1_coefficient=args.l1_coefficient, sparsity_loss_type=args.sparsity_loss_type,
                              jumprelu_lr_factor=args.jumprelu_lr_factor, total_training_tokens=args.total_tokens, log_frequency=1000,
                              n_checkpoints=5, exp_result_path=os.path.join(args.root, "results", name), amp_dtype=torch.bfloat16),
        activation_factories=factories, sae_name=name, sae_series="crosscoder-over-checkpoints",
    ))  # fmt: skip
