"""The interpretation runner end to end against the local file store: a trained dictionary is analysed into the store, a fake
chat service explains its features, and the explanations land on the feature records; features that never fired or are already
explained are left alone (runners/autointerp.py:20-129 of the reference project)."""

import asyncio
import json

import torch
from conftest import tiny_lm_config

from language_model_saes_b200.activation.factory import ActivationFactoryConfig, ActivationFactoryDatasetSource, ActivationFactoryTarget
from language_model_saes_b200.analysis import FeatureAnalyzerConfig
from language_model_saes_b200.analysis.autointerp import AutoInterpConfig
from language_model_saes_b200.config import DatasetConfig
from language_model_saes_b200.database import MongoClient, MongoDBConfig
from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
from language_model_saes_b200.runners import AnalyzeSAESettings, PretrainedSAE, analyze_sae
from language_model_saes_b200.runners.autointerp import AutoInterpSettings, async_auto_interp

HOOK = "blocks.1.hook_resid_post"


class _Chat:
    """``client.chat.completions.create`` of the OpenAI async interface."""

    def __init__(self):
        self.n_explanations = 0
        self.chat = self.completions = self

    async def create(self, model, messages, **kwargs):
        system, user = messages[0]["content"], messages[1]["content"]
        if "evaluation_results" in system:
            content = json.dumps({"steps": [], "evaluation_results": [True] * user.count("Example ")})
        else:
            self.n_explanations += 1
            content = json.dumps({"steps": [], "final_explanation": f"explanation {self.n_explanations}", "activation_consistency": 4, "complexity": 2})
        msg = type("M", (), {"content": content})
        return type("R", (), {"choices": [type("C", (), {"message": msg})]})


def test_explanations_are_written_to_the_features_that_fired(tiny_lm_workspace, tmp_path):
    mongo_cfg = MongoDBConfig(mongo_uri=f"file://{tmp_path / 'db'}", mongo_db="interp")
    store = MongoClient(mongo_cfg)
    lm_cfg = tiny_lm_config(tiny_lm_workspace)
    ds_cfg = DatasetConfig(dataset_name_or_path=str(tiny_lm_workspace / "data"), is_dataset_on_disk=True)
    store.add_dataset("toy", ds_cfg)
    store.add_model("tiny", lm_cfg)
    torch.manual_seed(0)
    sae = SparseAutoEncoder(SAEConfig(hook_point_in=HOOK, hook_point_out=HOOK, d_model=16, expansion_factor=2, act_fn="topk", top_k=4,
                                      norm_activation="inference"))  # fmt: skip
    sae.init_parameters(encoder_uniform_bound=0.5, decoder_uniform_bound=0.5)
    sae.save_pretrained(tmp_path / "sae")
    sae.cfg.save_hyperparameters(tmp_path / "sae")
    store.create_sae("toy-sae", "ser", str(tmp_path / "sae"), sae.cfg, model_name="tiny")
    analyze_sae(AnalyzeSAESettings(
        sae=PretrainedSAE(pretrained_name_or_path=str(tmp_path / "sae"), device="cpu", dtype=torch.float32), sae_name="toy-sae", sae_series="ser",
        activation_factory=ActivationFactoryConfig(sources=[ActivationFactoryDatasetSource(name="toy")], target=ActivationFactoryTarget.ACTIVATIONS_2D,
                                                   hook_points=[HOOK], batch_size=4, context_size=16, model_batch_size=4, num_workers=0),
        model_name="tiny", datasets={"toy": None}, analyzer=FeatureAnalyzerConfig(total_analyzing_tokens=16 * 32), mongo=mongo_cfg,
        device_type="cpu", amp_dtype=torch.bfloat16,
    ))  # fmt: skip
    fired = [i for i in range(32) if store.get_feature("toy-sae", "ser", i).analyses[0].act_times > 0]
    silent = [i for i in range(32) if i not in fired]
    assert len(fired) >= 4
    store.update_feature("toy-sae", fired[0], {"interpretation": {"text": "kept as it was"}}, "ser")

    chat = _Chat()
    settings = AutoInterpSettings(sae_name="toy-sae", sae_series="ser", model=lm_cfg, model_name="tiny", mongo=mongo_cfg, max_workers=3,
                                  auto_interp=AutoInterpConfig(n_activating_examples=3, n_non_activating_examples=3, detection_n_examples=2,
                                                               fuzzing_n_examples=2, max_length=16))  # fmt: skip
    asyncio.run(async_auto_interp(settings, client=chat))
    texts = {i: (store.get_feature("toy-sae", "ser", i).interpretation or {}).get("text") for i in range(32)}
    assert texts[fired[0]] == "kept as it was"
    assert all(texts[i] is not None and texts[i].startswith("explanation ") for i in fired[1:])
    assert all(texts[i] is None for i in silent)
    assert chat.n_explanations == len(fired) - 1
    # a second run finds nothing left to do; naming features limits the work
    asyncio.run(async_auto_interp(settings, client=chat))
    assert chat.n_explanations == len(fired) - 1
    again = settings.model_copy(update={"features": fired[:2], "auto_interp": settings.auto_interp.model_copy(update={"overwrite_existing": True})})
    asyncio.run(async_auto_interp(again, client=chat))
    assert chat.n_explanations == len(fired) + 1
    assert store.get_feature("toy-sae", "ser", fired[0]).interpretation["text"].startswith("explanation ")
