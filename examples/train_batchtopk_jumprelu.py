"""BatchTopK training (the k * batch largest gated pre-activations of a batch are kept, on the fused kernel path on a GPU),
then conversion of the result to JumpReLU thresholds estimated from activations.

    python examples/train_batchtopk_jumprelu.py train
    python examples/train_batchtopk_jumprelu.py convert      # cross-layer transcoders only, as in the reference project
"""

import sys

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
from language_model_saes_b200.runners import ConvertTopKToJumpReLUSettings, PretrainedSAE, convert_topk_to_jumprelu

hook = "blocks.6.hook_resid_post"
factory = ActivationFactoryConfig(
    sources=[ActivationFactoryActivationsSource(name="cache", path="activations/pythia-160m", device="cuda")],
    target=ActivationFactoryTarget.ACTIVATIONS_1D, hook_points=[hook], batch_size=4096, buffer_size=4096 * 16,
)  # fmt: skip
out = "results/pythia-160m-L6R-32x-batchtopk50"

train = TrainSAESettings(
    sae=SAEConfig(hook_point_in=hook, hook_point_out=hook, d_model=768, expansion_factor=32, act_fn="batchtopk", top_k=50,
                  dtype=torch.float32, device="cuda"),  # fmt: skip
    sae_name="pythia-160m-L6R-32x-batchtopk50", sae_series="examples",
    initializer=InitializerConfig(grid_search_init_norm=True),
    trainer=TrainerConfig(total_training_tokens=800_000_000, lr=4e-4, auxk_coefficient=None, exp_result_path=out),
    activation_factory=factory,
)  # fmt: skip

convert = ConvertTopKToJumpReLUSettings(
    sae=PretrainedSAE(pretrained_name_or_path=out, device="cuda", dtype=torch.float32),
    sae_name="pythia-160m-clt-jumprelu", sae_series="examples", activation_factory=factory, exp_result_path=out + "-jumprelu",
)  # fmt: skip

if __name__ == "__main__":
    convert_topk_to_jumprelu(convert) if sys.argv[1:] == ["convert"] else train_sae(train)
