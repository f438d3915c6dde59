"""Per-feature statistics and top activating contexts of a trained crosscoder, into the embedded database.

    python examples/crosscoder_over_checkpoints/analyze_crosscoder.py --name <name printed by train_crosscoder.py>
    MONGO_URI=file://$HOME/crosscoder/store MONGO_DB=mechinterp uvicorn language_model_saes_b200.server.app:app --port 24577
"""

import os

import torch
from common import arguments, cache_dir

from language_model_saes_b200 import (
    ActivationFactoryActivationsSource,
    ActivationFactoryConfig,
    AnalyzeCrosscoderSettings,
    FeatureAnalyzerConfig,
    MongoDBConfig,
    analyze_crosscoder,
)
from language_model_saes_b200.activation.factory import ActivationFactoryTarget
from language_model_saes_b200.runners import PretrainedSAE

if __name__ == "__main__":
    args = arguments(name=dict(required=True), batch_size=dict(type=int, default=16), total_tokens=dict(type=int, default=100_000_000))
    heads = [f"{step}/{args.hook}" for step in args.steps]
    factory = ActivationFactoryConfig(
        sources=[ActivationFactoryActivationsSource(name="cache", device="cuda", dtype=torch.bfloat16, num_workers=4, prefetch=4,
                                                    path={h: os.path.join(cache_dir(args, h.split("/")[0], "2d"), args.hook) for h in heads})],
        target=ActivationFactoryTarget.ACTIVATIONS_2D, hook_points=heads, batch_size=args.batch_size,
    )  # fmt: skip
    analyze_crosscoder(AnalyzeCrosscoderSettings(
        sae=PretrainedSAE(pretrained_name_or_path=os.path.join(args.root, "results", args.name), device="cuda", dtype=torch.float32),
        sae_name=args.name, sae_series="crosscoder-over-checkpoints",
        activation_factories=[factory],  # one factory: all heads on one rank (one per head-parallel rank otherwise)
        analyzer=FeatureAnalyzerConfig(total_analyzing_tokens=args.total_tokens),
        mongo=MongoDBConfig(mongo_uri=f"file://{os.path.join(args.root, 'store')}", mongo_db="mechinterp"),
    ))  # fmt: skip
