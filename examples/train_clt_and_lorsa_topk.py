"""Train a cross-layer transcoder or a low-rank sparse attention dictionary (Lorsa) on activations computed on the fly.

    python examples/train_clt_and_lorsa_topk.py --family clt
    torchrun --nproc-per-node 8 examples/train_clt_and_lorsa_topk.py --family lorsa --model-parallel 8

Both settings meet the conditions of the fused kernel steps (TopK, Adam, fp32 parameters with bf16 compute, no sparsity
penalty): `Trainer` logs "fused ... kernel path" when it takes them. With ``--model-parallel N`` the dictionary (the
features of every layer, or the OV heads with their QK heads) is split over N GPUs.
"""

import argparse
import math

import torch

from language_model_saes_b200 import (
    ActivationFactoryConfig,
    ActivationFactoryDatasetSource,
    CLTConfig,
    DatasetConfig,
    InitializerConfig,
    LanguageModelConfig,
    LorsaConfig,
    TrainCLTSettings,
    TrainerConfig,
    TrainLorsaSettings,
    train_clt,
    train_lorsa,
)
from language_model_saes_b200.activation.factory import ActivationFactoryTarget

ap = argparse.ArgumentParser()
ap.add_argument("--family", choices=["clt", "lorsa"], default="clt")
ap.add_argument("--model-parallel", type=int, default=1)
ap.add_argument("--data-parallel", type=int, default=1)
args = ap.parse_args()

D, LAYERS, CTX = 768, 12, 1024
common = dict(
    model=LanguageModelConfig(model_name="EleutherAI/pythia-160m", device="cuda", dtype="bfloat16"),
    model_name="pythia-160m",
    datasets={"SlimPajama-3B": DatasetConfig(dataset_name_or_path="Hzfinfdu/SlimPajama-3B")},
    model_parallel_size=args.model_parallel,
    data_parallel_size=args.data_parallel,
    sae_series="examples",
)

if args.family == "clt":
    hooks_in = [f"blocks.{i}.ln2.hook_normalized" for i in range(LAYERS)]
    hooks_out = [f"blocks.{i}.hook_mlp_out" for i in range(LAYERS)]
    settings = TrainCLTSettings(
        # features of layer i read the residual stream before MLP i and write to the outputs of MLPs i .. 11
        sae=CLTConfig(hook_points_in=hooks_in, hook_points_out=hooks_out, d_model=D, expansion_factor=32, act_fn="topk", top_k=64,
                      dtype=torch.float32, device="cuda"),
        sae_name="pythia-160m-clt-32x-topk64",
        initializer=InitializerConfig(grid_search_init_norm=False, init_encoder_with_decoder_transpose=False,
                                      encoder_uniform_bound=1 / math.sqrt(D), decoder_uniform_bound=1 / math.sqrt(D * 32 * LAYERS)),
        trainer=TrainerConfig(lr=2e-4, total_training_tokens=800_000_000, log_frequency=1000, n_checkpoints=0,
                              exp_result_path="results/pythia-160m-clt-32x-topk64", amp_dtype=torch.bfloat16),
        activation_factory=ActivationFactoryConfig(
            sources=[ActivationFactoryDatasetSource(name="SlimPajama-3B")], target=ActivationFactoryTarget.ACTIVATIONS_1D,
            hook_points=hooks_in + hooks_out, batch_size=4096, buffer_size=4096 * 4, context_size=CTX, model_batch_size=32),
        **common,
    )  # fmt: skip
else:
    hook_in, hook_out = "blocks.6.ln1.hook_normalized", "blocks.6.hook_attn_out"
    settings = TrainLorsaSettings(
        # 6144 rank-1 OV heads in 48 groups, each group sharing one QK head of width 64; Pythia rotates the first quarter of a
        # head's channels, in the half-split layout
        sae=LorsaConfig(hook_point_in=hook_in, hook_point_out=hook_out, d_model=D, expansion_factor=8, n_qk_heads=48, d_qk_head=64,
                        rotary_dim=64 // 4, rotary_adjacent_pairs=False, rotary_base=10_000, n_ctx=CTX, act_fn="topk", top_k=64,
                        dtype=torch.float32, device="cuda"),
        sae_name="pythia-160m-L6-lorsa-8x-topk64",
        initializer=InitializerConfig(grid_search_init_norm=False, init_encoder_with_decoder_transpose=False,
                                      decoder_uniform_bound=1 / math.sqrt(D), encoder_uniform_bound=1 / math.sqrt(D * 8)),
        # whole sequences per step ([batch, context, d_model]): total_training_tokens counts sequences x context
        trainer=TrainerConfig(lr=2e-4, initial_k=64, total_training_tokens=800_000_000, log_frequency=1000, n_checkpoints=0,
                              exp_result_path="results/pythia-160m-L6-lorsa-8x-topk64", amp_dtype=torch.bfloat16),
        activation_factory=ActivationFactoryConfig(
            sources=[ActivationFactoryDatasetSource(name="SlimPajama-3B")], target=ActivationFactoryTarget.ACTIVATIONS_2D,
            hook_points=[hook_in, hook_out], batch_size=32, buffer_size=None, context_size=CTX, model_batch_size=32),
        **common,
    )  # fmt: skip

if __name__ == "__main__":
    (train_clt if args.family == "clt" else train_lorsa)(settings)
