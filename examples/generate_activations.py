"""Write an activation cache: run a language model over a dataset and store the hooked activations per hook point.

    python examples/generate_activations.py            # one GPU
    torchrun --nproc-per-node 8 examples/generate_activations.py   # eight data-parallel writers (one shard each)
"""

from language_model_saes_b200 import DatasetConfig, GenerateActivationsSettings, LanguageModelConfig, generate_activations
from language_model_saes_b200.activation.factory import ActivationFactoryTarget

settings = GenerateActivationsSettings(
    model=LanguageModelConfig(model_name="EleutherAI/pythia-160m", device="cuda", dtype="bfloat16"),
    model_name="pythia-160m",
    dataset=DatasetConfig(dataset_name_or_path="Skylion007/openwebtext", is_dataset_on_disk=False),
    dataset_name="openwebtext",
    hook_points=[f"blocks.{layer}.hook_resid_post" for layer in (3, 6)],
    output_dir="activations/pythia-160m",
    target=ActivationFactoryTarget.ACTIVATIONS_2D,  # [samples, context, d_model] chunks with tokens and masks
    total_tokens=100_000_000,
    context_size=1024,
    model_batch_size=32,
    batch_size=32,  # samples per record handed to the writer
    n_samples_per_chunk=16,
    num_workers=4,  # writer threads
    format="safetensors",
)

if __name__ == "__main__":
    generate_activations(settings)
