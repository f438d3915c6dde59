"""The example scripts build valid settings: every script that ends in a runner call is executed with the runner replaced
by a recorder, so that field names, enum values and cross-field validation of its settings are checked without a model, a
dataset or a GPU. Scripts that only define settings at import time are imported."""

import os
import runpy
import sys
from pathlib import Path

import pytest

import language_model_saes_b200 as L

EXAMPLES = Path(__file__).resolve().parents[1] / "examples"


@pytest.fixture
def recorded(monkeypatch):
    calls: dict[str, list] = {}
    for fn in ("generate_activations", "train_sae", "train_crosscoder", "train_clt", "train_lorsa", "train_molt", "analyze_sae",
               "analyze_crosscoder", "convert_topk_to_jumprelu"):  # fmt: skip
        if hasattr(L, fn):
            monkeypatch.setattr(L, fn, (lambda name: lambda settings: calls.setdefault(name, []).append(settings))(fn))
    return calls


def _run(script: Path, argv: list[str], monkeypatch) -> None:
    monkeypatch.setattr(sys, "argv", [str(script)] + argv)
    monkeypatch.syspath_prepend(str(script.parent))
    for name in ("common",):  # a helper module of one example folder must not leak into the next
        sys.modules.pop(name, None)
    runpy.run_path(str(script), run_name="__main__")


def test_crosscoder_over_checkpoints_scripts_build_their_settings(recorded, monkeypatch, tmp_path):
    folder = EXAMPLES / "crosscoder_over_checkpoints"
    root = ["--root", str(tmp_path)]
    _run(folder / "generate_activations.py", ["--steps", "step1,step2", "--target", "1d"] + root, monkeypatch)
    _run(folder / "generate_activations.py", ["--steps", "step1", "--target", "2d"] + root, monkeypatch)
    _run(folder / "train_crosscoder.py", ["--steps", "step1,step2,step3,step4", "--head-parallel", "2", "--sparsity-loss-type", "tanh"] + root, monkeypatch)
    _run(folder / "analyze_crosscoder.py", ["--steps", "step1,step2", "--name", "run"] + root, monkeypatch)
    gen = recorded["generate_activations"]
    assert len(gen) == 3 and gen[0].buffer_shuffle.perm_seed == gen[1].buffer_shuffle.perm_seed  # the same permutation per snapshot
    assert gen[2].buffer_shuffle is None and gen[2].target == L.ActivationFactoryTarget.ACTIVATIONS_2D
    (train,) = recorded["train_crosscoder"]
    assert train.sae.n_heads == 4 and [len(f.hook_points) for f in train.activation_factories] == [2, 2]
    # every head-parallel rank reads its own snapshots only
    assert set(train.activation_factories[1].sources[0].path) == {"step3/blocks.6.hook_resid_post", "step4/blocks.6.hook_resid_post"}
    assert all(str(tmp_path) in p for f in train.activation_factories for p in f.sources[0].path.values())
    (ana,) = recorded["analyze_crosscoder"]
    assert ana.sae.pretrained_name_or_path == os.path.join(str(tmp_path), "results", "run") and ana.mongo.mongo_uri.startswith("file://")


@pytest.mark.parametrize("script", ["generate_activations.py", "analyze_and_serve.py", "train_topk_sae_from_cache.py", "train_batchtopk_jumprelu.py"])
def test_settings_examples_validate(script, recorded, monkeypatch):
    path = EXAMPLES / script
    if not path.exists():
        pytest.skip("no such example")
    _run(path, [], monkeypatch)
    assert sum(len(v) for v in recorded.values()) >= 1, f"{script} called no runner"


@pytest.mark.parametrize("family", ["clt", "lorsa"])
def test_clt_and_lorsa_training_example_meets_the_fused_step_conditions(family, recorded, monkeypatch):
    _run(EXAMPLES / "train_clt_and_lorsa_topk.py", ["--family", family], monkeypatch)
    (settings,) = recorded[f"train_{family}"]
    import copy

    from language_model_saes_b200.models.sparse_dictionary import SparseDictionary
    from language_model_saes_b200.ops.fused_clt import FusedCLTStep
    from language_model_saes_b200.ops.fused_lorsa import FusedLorsaStep

    # a narrow copy of the model on the CPU: the conditions on the configuration are the same (the device one is set aside)
    small = {"clt": dict(expansion_factor=1, device="cpu"), "lorsa": dict(expansion_factor=1, n_qk_heads=12, device="cpu")}[family]
    model = SparseDictionary.from_config(settings.sae.model_copy(update=small))
    trainer_cfg = copy.copy(settings.trainer)
    import torch

    monkeypatch.setattr(torch.Tensor, "is_cuda", property(lambda self: True))  # only the question "is it on a GPU" is answered for it
    ok, why = (FusedCLTStep if family == "clt" else FusedLorsaStep).supports(model, trainer_cfg)
    monkeypatch.undo()
    assert ok, why


def test_family_config_example_builds_every_family_on_the_meta_device(capsys, monkeypatch):
    _run(EXAMPLES / "train_crosscoder_clt_lorsa.py", [], monkeypatch)
    out = capsys.readouterr().out
    for name in ("Crosscoder", "CrossLayerTranscoder", "LowRankSparseAttention", "MixtureOfLinearTransform"):
        assert name in out, out


def test_every_example_settings_object_can_be_written_to_a_settings_file_and_read_back(recorded, monkeypatch, tmp_path):
    """What the examples build in Python is what the command line reads from a file: dumped as JSON text (dtypes, enums and
    paths become strings) and validated again, a settings object keeps every field."""
    import json

    for script in ("generate_activations.py", "analyze_and_serve.py", "train_topk_sae_from_cache.py", "train_batchtopk_jumprelu.py"):
        if (EXAMPLES / script).exists():
            _run(EXAMPLES / script, [], monkeypatch)
    for family in ("clt", "lorsa"):
        _run(EXAMPLES / "train_clt_and_lorsa_topk.py", ["--family", family], monkeypatch)
    folder, root = EXAMPLES / "crosscoder_over_checkpoints", ["--root", str(tmp_path)]
    _run(folder / "generate_activations.py", ["--steps", "step1", "--target", "1d"] + root, monkeypatch)
    _run(folder / "train_crosscoder.py", ["--steps", "step1,step2", "--head-parallel", "2"] + root, monkeypatch)
    _run(folder / "analyze_crosscoder.py", ["--steps", "step1,step2", "--name", "run"] + root, monkeypatch)
    seen = 0
    for name, calls in recorded.items():
        for settings in calls:
            text = json.dumps(settings.model_dump(mode="json"))
            again = type(settings).model_validate(json.loads(text))
            assert again.model_dump(mode="json") == settings.model_dump(mode="json"), name
            seen += 1
    assert seen >= 8
