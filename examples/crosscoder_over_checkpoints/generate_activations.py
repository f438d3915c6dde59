"""Activation caches of every snapshot: token-level and shuffled for training (``--target 1d``), whole contexts for the
analysis (``--target 2d``).

    torchrun --nproc-per-node 8 examples/crosscoder_over_checkpoints/generate_activations.py --size 160m --layer 6 --target 1d
"""

import os

from common import arguments, cache_dir

from language_model_saes_b200 import BufferShuffleConfig, DatasetConfig, GenerateActivationsSettings, LanguageModelConfig, generate_activations
from language_model_saes_b200.activation.factory import ActivationFactoryTarget

if __name__ == "__main__":
    args = arguments(target=dict(default="1d", choices=["1d", "2d"]), total_tokens=dict(type=int, default=800_000_000),
                     dataset=dict(default="~/data/SlimPajama-3B", help="a dataset saved with save_to_disk()"),
                     models=dict(default="~/models", help="<models>/pythia-<size>/<step> holds every snapshot's weights"))  # fmt: skip
    for step in args.steps:
        one_d = args.target == "1d"
        generate_activations(GenerateActivationsSettings(
            # one folder per snapshot, e.g. from `huggingface-cli download EleutherAI/pythia-160m --revision step1000 --local-dir ...`
            model=LanguageModelConfig(model_name=f"EleutherAI/pythia-{args.size}", device="cuda", dtype="bfloat16",
                                      model_from_pretrained_path=os.path.join(os.path.expanduser(args.models), f"pythia-{args.size}", step)),
            model_name=f"pythia-{args.size}-{step}",
            dataset=DatasetConfig(dataset_name_or_path=os.path.expanduser(args.dataset), is_dataset_on_disk=True),
            dataset_name="SlimPajama-3B",
            hook_points=[args.hook],
            output_dir=cache_dir(args, step, args.target),
            target=ActivationFactoryTarget.ACTIVATIONS_1D if one_d else ActivationFactoryTarget.ACTIVATIONS_2D,
            total_tokens=args.total_tokens,
            context_size=1024,
            model_batch_size=32,
            batch_size=2048 * 16 if one_d else 16,
            # the same seed for every snapshot: row i of every cache is the same token, which a crosscoder needs
            buffer_size=2048 * 200 if one_d else None,
            buffer_shuffle=BufferShuffleConfig(perm_seed=42) if one_d else None,
            n_samples_per_chunk=None if one_d else 16,
            num_workers=4,
            format="safetensors",
        ))  # fmt: skip
