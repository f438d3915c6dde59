"""The runners end to end on CPU with a tiny random GPT-2 and a word-level tokenizer saved to a temp directory:
generate activations -> train an SAE on the cache -> analyze -> direct logit attribution -> evaluate."""

import json
import pickle
from pathlib import Path

import pytest
import torch

from language_model_saes_b200.activation.factory import ActivationFactoryActivationsSource, ActivationFactoryConfig, ActivationFactoryTarget
from language_model_saes_b200.analysis import DirectLogitAttributorConfig, FeatureAnalyzerConfig
from language_model_saes_b200.config import DatasetConfig
from language_model_saes_b200.evaluator import EvalConfig
from language_model_saes_b200.initializer import InitializerConfig
from language_model_saes_b200.models.sae import SAEConfig
from language_model_saes_b200.runners import (
    AnalyzeSAESettings,
    CheckActivationConsistencySettings,
    DirectLogitAttributeSettings,
    EvaluateSAESettings,
    GenerateActivationsSettings,
    PretrainedSAE,
    TrainSAESettings,
    analyze_sae,
    check_activation_consistency,
    direct_logit_attribute,
    evaluate_sae,
    generate_activations,
    train_sae,
)
from language_model_saes_b200.trainer import TrainerConfig

from conftest import tiny_lm_config

HOOK = "blocks.1.hook_resid_post"


@pytest.fixture()
def workspace(tiny_lm_workspace, tmp_path):
    return tiny_lm_workspace, tmp_path


def _lm(root):
    return tiny_lm_config(root)


def test_pipeline_generate_train_analyze_evaluate(workspace):
    src, root = workspace
    acts = root / "acts"
    generate_activations(GenerateActivationsSettings(
        model=_lm(src), model_name="tiny", dataset=DatasetConfig(dataset_name_or_path=str(src / "data"), is_dataset_on_disk=True),
        dataset_name="toy", hook_points=[HOOK], output_dir=str(acts), total_tokens=16 * 64, context_size=16,
        model_batch_size=4, batch_size=4, device_type="cpu", format="safetensors",
    ))  # fmt: skip
    chunks = sorted((acts / HOOK).glob("*.safetensors"))
    assert len(chunks) >= 4
    check_activation_consistency(CheckActivationConsistencySettings(paths={HOOK: acts / HOOK}, device="cpu"))

    def factory(target, batch_size):
        return ActivationFactoryConfig(
            sources=[ActivationFactoryActivationsSource(name="toy", path=str(acts), device="cpu", num_workers=0, prefetch=None)],
            target=target, hook_points=[HOOK], batch_size=batch_size, num_workers=0,
        )  # fmt: skip

    out = root / "sae"
    train_sae(TrainSAESettings(
        sae=SAEConfig(hook_point_in=HOOK, hook_point_out=HOOK, d_model=16, expansion_factor=4, act_fn="topk", top_k=4,
                      device="cpu", dtype=torch.float32),
        sae_name="toy-sae", sae_series="test", initializer=InitializerConfig(),
        trainer=TrainerConfig(lr=1e-3, total_training_tokens=512, log_frequency=4, eval_frequency=10**6, n_checkpoints=0,
                              lr_warm_up_steps=2, exp_result_path=str(out), amp_dtype=torch.float32, l1_coefficient=None),
        activation_factory=factory(ActivationFactoryTarget.ACTIVATIONS_1D, 32), device_type="cpu",
    ))  # fmt: skip
    assert (out / "config.json").exists() and (out / "sae_weights.safetensors").exists()
    assert json.loads((out / "config.json").read_text())["sae_type"] == "sae"

    pre = PretrainedSAE(pretrained_name_or_path=str(out), device="cpu", dtype=torch.float32)
    analysis_dir = root / "analysis"
    analyze_sae(AnalyzeSAESettings(
        sae=pre, sae_name="toy-sae", sae_series="test", activation_factory=factory(ActivationFactoryTarget.ACTIVATIONS_2D, 4),
        analyzer=FeatureAnalyzerConfig(total_analyzing_tokens=16 * 16, ignore_token_ids=[1]), output_dir=analysis_dir,
        device_type="cpu", amp_dtype=torch.float32,
    ))  # fmt: skip
    pkl = analysis_dir / "toy-sae" / "test" / "default_analysis_64_features.pkl"
    assert pkl.exists()
    with open(pkl, "rb") as f:
        records = pickle.load(f)
    assert [r["feature_idx"] for r in records] == list(range(64))
    assert sum(r["act_times"] for r in records) > 0
    fired = next(r for r in records if r["act_times"] > 0)
    top = fired["samplings"][0]
    assert top["name"] == "top_activations" and len(top["context_idx"]) > 0 and top["dataset_name"][0] == "toy"

    direct_logit_attribute(DirectLogitAttributeSettings(
        sae=pre, sae_name="toy-sae", sae_series="test", model=_lm(src), model_name="tiny",
        direct_logit_attributor=DirectLogitAttributorConfig(top_k=3), analysis_file=pkl, device_type="cpu",
    ))  # fmt: skip
    with open(pkl, "rb") as f:
        records = pickle.load(f)
    assert len(records[0]["logits"]["top_positive"]) == 3 and len(records[0]["logits"]["top_negative"]) == 3
    assert records[0]["logits"]["top_positive"][0]["logit"] >= records[0]["logits"]["top_positive"][1]["logit"]
    assert isinstance(records[0]["logits"]["top_positive"][0]["token"], str)

    metrics = evaluate_sae(EvaluateSAESettings(
        sae=pre, sae_name="toy-sae", sae_series="test", activation_factory=factory(ActivationFactoryTarget.ACTIVATIONS_1D, 32),
        eval=EvalConfig(total_eval_tokens=128), device_type="cpu",
    ))  # fmt: skip
    assert any("explained_variance" in k for k in metrics) and any("l0" in k.lower() for k in metrics)
    l0 = next(v for k, v in metrics.items() if k.lower().endswith("l0"))
    assert abs(l0 - 4) < 1e-3


from language_model_saes_b200.testing import distributed_test  # noqa: E402


@distributed_test(nproc_per_node=2, backend="gloo")
def test_sweep_trains_two_dictionaries_on_one_shared_stream():
    """Two sweep members (one gloo rank each) train dictionaries with different k from ONE activation stream: member 0
    builds the factory and broadcasts every batch; member 1 is even given a source path that does not exist, which it
    never opens (runners/train.py:1179-1338 of the reference project replicates one stream over the sweep dimension)."""
    import tempfile

    import torch.distributed as dist

    from conftest import build_tiny_lm
    from language_model_saes_b200.runners import SweepSAESettings, sweep_sae
    from language_model_saes_b200.runners.train import SweepingItem

    rank = dist.get_rank()
    box = [None]
    if rank == 0:
        root = Path(tempfile.mkdtemp(prefix="lmsae_sweep_"))
        src = build_tiny_lm(root / "lm")
        generate_activations(GenerateActivationsSettings(
            model=_lm(src), model_name="tiny", dataset=DatasetConfig(dataset_name_or_path=str(src / "data"), is_dataset_on_disk=True),
            dataset_name="toy", hook_points=[HOOK], output_dir=str(root / "acts"), total_tokens=16 * 64, context_size=16,
            model_batch_size=4, batch_size=4, device_type="cpu", format="safetensors",
        ))  # fmt: skip
        box[0] = str(root)
    dist.broadcast_object_list(box, src=0)
    root = Path(box[0])
    acts = root / "acts" if rank == 0 else root / "no-such-directory"
    items = [
        SweepingItem(
            sae=SAEConfig(hook_point_in=HOOK, hook_point_out=HOOK, d_model=16, expansion_factor=4, act_fn="topk", top_k=k, device="cpu",
                          dtype=torch.float32),
            sae_name=f"toy-k{k}", sae_series="sweep", initializer=InitializerConfig(),
            trainer=TrainerConfig(lr=1e-3, total_training_tokens=384, log_frequency=4, eval_frequency=10**6, n_checkpoints=0,
                                  lr_warm_up_steps=2, exp_result_path=str(root / f"out_k{k}"), amp_dtype=torch.float32, l1_coefficient=None),
        )
        for k in (2, 6)
    ]  # fmt: skip
    factory = ActivationFactoryConfig(
        sources=[ActivationFactoryActivationsSource(name="toy", path=str(acts), device="cpu", num_workers=0, prefetch=None)],
        target=ActivationFactoryTarget.ACTIVATIONS_1D, hook_points=[HOOK], batch_size=32, num_workers=0,
    )  # fmt: skip
    sweep_sae(SweepSAESettings(items=items, activation_factory=factory, device_type="cpu"))
    dist.barrier()
    mine = root / f"out_k{(2, 6)[rank]}"
    # (weights sit at the top level, or under checkpoints/step_N when the stream ended before the token budget)
    assert (mine / "config.json").exists() and list(mine.rglob("sae_weights.safetensors"))
    assert json.loads((mine / "config.json").read_text())["top_k"] == (2, 6)[rank]
