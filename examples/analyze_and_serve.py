"""Feature analysis into the embedded file store, then how to browse it.

    python examples/analyze_and_serve.py
    MONGO_URI=file://$PWD/store MONGO_DB=mechinterp uvicorn language_model_saes_b200.server.app:app --port 24577
    # open http://127.0.0.1:24577/ui/

A ``mongodb://`` URI works the same way (the reference project's database layout).
"""

import os

from language_model_saes_b200 import (
    ActivationFactoryActivationsSource,
    ActivationFactoryConfig,
    AnalyzeSAESettings,
    FeatureAnalyzerConfig,
    MongoDBConfig,
    analyze_sae,
)
from language_model_saes_b200.activation.factory import ActivationFactoryTarget
from language_model_saes_b200.runners import PretrainedSAE

hook = "blocks.6.hook_resid_post"
settings = AnalyzeSAESettings(
    sae=PretrainedSAE(pretrained_name_or_path="results/pythia-160m-L6R-32x-topk50", device="cuda"),
    sae_name="pythia-160m-L6R-32x-topk50",
    sae_series="examples",
    activation_factory=ActivationFactoryConfig(
        sources=[ActivationFactoryActivationsSource(name="cache", path="activations/pythia-160m", device="cuda")],
        target=ActivationFactoryTarget.ACTIVATIONS_2D,  # whole contexts: the analyzer keeps top-activating samples
        hook_points=[hook],
        batch_size=16,
    ),
    analyzer=FeatureAnalyzerConfig(total_analyzing_tokens=20_000_000),
    mongo=MongoDBConfig(mongo_uri=f"file://{os.getcwd()}/store", mongo_db="mechinterp"),
)

if __name__ == "__main__":
    analyze_sae(settings)
