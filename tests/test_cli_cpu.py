"""Command line against the local file store: create / show / remove, and config-file loading."""

import json

import numpy as np
import pytest
from conftest import tiny_lm_config
from typer.testing import CliRunner

from language_model_saes_b200.cli import app, load_config
from language_model_saes_b200.database import MongoClient, MongoDBConfig
from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder

runner = CliRunner()


def test_load_config_formats(tmp_path):
    (tmp_path / "a.json").write_text(json.dumps({"x": 1}))
    (tmp_path / "a.yaml").write_text("x: 1\ny: [1, 2]\n")
    (tmp_path / "a.toml").write_text('x = 1\n[t]\nz = "s"\n')
    (tmp_path / "a.py").write_text("config = {'x': 1}\n")
    (tmp_path / "a.txt").write_text("x")
    assert load_config(tmp_path / "a.json") == {"x": 1}
    assert load_config(tmp_path / "a.yaml") == {"x": 1, "y": [1, 2]}
    assert load_config(tmp_path / "a.toml") == {"x": 1, "t": {"z": "s"}}
    assert load_config(tmp_path / "a.py") == {"x": 1}
    import typer

    with pytest.raises(typer.BadParameter):
        load_config(tmp_path / "a.txt")
    with pytest.raises(typer.BadParameter):
        load_config(tmp_path / "missing.json")


def test_create_show_remove_roundtrip(tiny_lm_workspace, tmp_path):
    uri, db = f"file://{tmp_path / 'db'}", "cli"
    common = ["--mongo-uri", uri, "--mongo-db", db]
    (tmp_path / "ds.json").write_text(json.dumps({"dataset_name_or_path": str(tiny_lm_workspace / "data"), "is_dataset_on_disk": True}))
    lm = tiny_lm_config(tiny_lm_workspace).model_dump()
    (tmp_path / "lm.json").write_text(json.dumps(lm))
    assert runner.invoke(app, ["create", "dataset", "toy", str(tmp_path / "ds.json"), *common]).exit_code == 0
    r = runner.invoke(app, ["create", "model", "tiny", str(tmp_path / "lm.json"), *common])
    assert r.exit_code == 0, r.output

    sae = SparseAutoEncoder(SAEConfig(hook_point_in="h", hook_point_out="h", d_model=16, expansion_factor=2, act_fn="relu"))
    sae.init_parameters(encoder_uniform_bound=0.1, decoder_uniform_bound=0.1)
    sae.save_pretrained(tmp_path / "sae")
    sae.cfg.save_hyperparameters(tmp_path / "sae")
    r = runner.invoke(app, ["create", "sae", "toy-sae", str(tmp_path / "sae"), "-s", "ser", *common])
    assert r.exit_code == 0, r.output

    client = MongoClient(MongoDBConfig(mongo_uri=uri, mongo_db=db))
    assert client.get_dataset_cfg("toy").is_dataset_on_disk and client.get_model_cfg("tiny").max_length == 32
    assert client.get_sae("toy-sae", "ser").cfg.d_sae == 32
    acts = np.zeros((2, 16), dtype=np.float32)
    acts[0, 3], acts[0, 4], acts[1, 7] = 2.0, 0.5, 1.0
    rows, cols = np.nonzero(acts)
    record = {
        "act_times": 3, "n_analyzed_tokens": 100, "max_feature_acts": 2.0,
        "samplings": [{"name": "top_activations", "feature_acts_indices": np.stack([rows, cols]).astype(np.float32),
                       "feature_acts_values": acts[rows, cols], "context_idx": np.array([5, 9]), "dataset_name": ["toy", "toy"],
                       "model_name": ["tiny", "tiny"], "shard_idx": np.array([0, 0]), "n_shards": np.array([1, 1])}],
    }  # fmt: skip
    client.add_feature_analysis("default", "toy-sae", "ser", [record], start_idx=0)
    client.update_feature("toy-sae", 0, {"interpretation": {"text": "a test feature"}}, "ser")

    r = runner.invoke(app, ["show", "feature", "toy-sae", "0", "-s", "ser", "-n", "2", "-r", "4", *common])
    assert r.exit_code == 0, r.output
    assert "Feature #0" in r.output and "a test feature" in r.output and "Activation Times" in r.output and "Sample 2" in r.output
    r = runner.invoke(app, ["show", "feature", "toy-sae", "999", "-s", "ser", *common])
    assert r.exit_code == 1

    assert runner.invoke(app, ["remove", "analysis", "toy-sae", "default", "-s", "ser", *common]).exit_code == 0
    assert client.get_feature("toy-sae", "ser", 0).analyses == []
    assert runner.invoke(app, ["remove", "sae", "toy-sae", "-s", "ser", *common]).exit_code == 0
    assert client.get_sae("toy-sae", "ser") is None


def test_public_names_and_alias_packages():
    import llamascopium
    import lm_saes

    import language_model_saes_b200 as L

    for name in L.__all__:
        assert getattr(llamascopium, name) is getattr(L, name) and getattr(lm_saes, name) is getattr(L, name)
    from llamascopium.models.sae import SparseAutoEncoder
    from lm_saes.circuits.attribution import attribute

    assert SparseAutoEncoder is L.SparseAutoEncoder and attribute is L.attribute
    assert L.TransformerLensLanguageModel is L.HookedLanguageModel
    for method in ("apply_saes", "detach_at", "attribute", "qk_trace", "run_with_cache_until", "run_with_ref_cache", "trace", "to_activations"):
        assert callable(getattr(L.HookedLanguageModel, method))


def test_job_commands_run_from_settings_files(tiny_lm_workspace, tmp_path):
    """``generate`` -> ``train`` -> ``analyze`` -> ``evaluate`` -> ``dla``, each from a settings file written by hand (strings
    for dtypes and enums, as a user writes them), in the three text formats."""
    import pickle

    import yaml

    hook = "blocks.1.hook_resid_post"
    lm = {"model_name": "gpt2", "model_from_pretrained_path": str(tiny_lm_workspace / "model"), "local_files_only": True, "backend": "hooked",
          "device": "cpu", "dtype": "float32", "max_length": 32, "bos_token_id": 0, "eos_token_id": 0, "pad_token_id": 1}  # fmt: skip
    acts, out, ana = tmp_path / "acts", tmp_path / "sae", tmp_path / "analysis"
    (tmp_path / "gen.yaml").write_text(yaml.safe_dump({
        "model": lm, "model_name": "tiny", "dataset": {"dataset_name_or_path": str(tiny_lm_workspace / "data"), "is_dataset_on_disk": True},
        "dataset_name": "toy", "hook_points": [hook], "output_dir": str(acts), "total_tokens": 1024, "context_size": 16,
        "model_batch_size": 4, "batch_size": 4, "device_type": "cpu", "format": "safetensors"}))  # fmt: skip
    r = runner.invoke(app, ["generate", str(tmp_path / "gen.yaml")])
    assert r.exit_code == 0, (r.output, r.exception)
    assert len(list((acts / hook).glob("*.safetensors"))) >= 4

    def factory(target, batch):
        return {"sources": [{"type": "activations", "name": "toy", "path": str(acts), "device": "cpu", "num_workers": 0, "prefetch": None}],
                "target": target, "hook_points": [hook], "batch_size": batch, "num_workers": 0}  # fmt: skip

    (tmp_path / "train.json").write_text(json.dumps({
        "sae": {"hook_point_in": hook, "hook_point_out": hook, "d_model": 16, "expansion_factor": 4, "act_fn": "topk", "top_k": 4,
                "device": "cpu", "dtype": "float32"},
        "sae_name": "toy-sae", "sae_series": "test", "initializer": {},
        "trainer": {"lr": 1e-3, "total_training_tokens": 512, "log_frequency": 4, "eval_frequency": 1000000, "n_checkpoints": 0,
                    "lr_warm_up_steps": 2, "exp_result_path": str(out), "amp_dtype": "float32", "l1_coefficient": None},
        "activation_factory": factory("activations-1d", 32), "device_type": "cpu"}))  # fmt: skip
    r = runner.invoke(app, ["train", str(tmp_path / "train.json"), "--kind", "sae"])
    assert r.exit_code == 0, (r.output, r.exception)
    assert (out / "sae_weights.safetensors").exists() and json.loads((out / "config.json").read_text())["expansion_factor"] == 4

    pre = {"pretrained_name_or_path": str(out), "device": "cpu", "dtype": "float32"}
    f2 = factory("activations-2d", 4)
    toml_src = "\n".join([
        'sae_name = "toy-sae"', 'sae_series = "test"', f'output_dir = "{ana}"', 'device_type = "cpu"', 'amp_dtype = "float32"',
        "[sae]", *(f'{k} = "{v}"' for k, v in pre.items()),
        "[analyzer]", "total_analyzing_tokens = 256", "ignore_token_ids = [1]",
        "[activation_factory]", f'target = "{f2["target"]}"', f'hook_points = ["{hook}"]', "batch_size = 4", "num_workers = 0",
        "[[activation_factory.sources]]", 'type = "activations"', 'name = "toy"', f'path = "{acts}"', 'device = "cpu"', "num_workers = 0",
    ])  # fmt: skip
    (tmp_path / "analyze.toml").write_text(toml_src)
    r = runner.invoke(app, ["analyze", str(tmp_path / "analyze.toml")])
    assert r.exit_code == 0, (r.output, r.exception)
    pkl = ana / "toy-sae" / "test" / "default_analysis_64_features.pkl"
    with open(pkl, "rb") as f:
        records = pickle.load(f)
    assert len(records) == 64 and sum(rec["act_times"] for rec in records) > 0

    (tmp_path / "eval.py").write_text("config = " + repr({
        "sae": pre, "sae_name": "toy-sae", "sae_series": "test", "activation_factory": factory("activations-1d", 32),
        "eval": {"total_eval_tokens": 128}, "device_type": "cpu"}) + "\n")  # fmt: skip
    r = runner.invoke(app, ["evaluate", str(tmp_path / "eval.py")])
    assert r.exit_code == 0, (r.output, r.exception)

    (tmp_path / "dla.json").write_text(json.dumps({
        "sae": pre, "sae_name": "toy-sae", "sae_series": "test", "model": lm, "model_name": "tiny",
        "direct_logit_attributor": {"top_k": 2}, "analysis_file": str(pkl), "device_type": "cpu"}))  # fmt: skip
    r = runner.invoke(app, ["dla", str(tmp_path / "dla.json")])
    assert r.exit_code == 0, (r.output, r.exception)
    with open(pkl, "rb") as f:
        assert len(pickle.load(f)[0]["logits"]["top_positive"]) == 2
    r = runner.invoke(app, ["train", str(tmp_path / "train.json"), "--kind", "nothing"])
    assert r.exit_code != 0


def test_a_run_that_outlives_its_stream_leaves_a_checkpoint_that_a_second_run_resumes(tiny_lm_workspace, tmp_path):
    """The cache holds fewer tokens than the run wants: ``train`` ends with a trainer checkpoint (weights, optimizer, schedule,
    counters) instead of final weights; a second ``train`` that names it (``sae.pretrained_name_or_path`` and
    ``trainer.from_pretrained_path``) picks up at that step, finishes and writes the final weights."""
    import torch

    hook = "blocks.1.hook_resid_post"
    lm = {"model_name": "gpt2", "model_from_pretrained_path": str(tiny_lm_workspace / "model"), "local_files_only": True, "backend": "hooked",
          "device": "cpu", "dtype": "float32", "max_length": 32, "bos_token_id": 0, "eos_token_id": 0, "pad_token_id": 1}  # fmt: skip
    acts, out = tmp_path / "acts", tmp_path / "sae"
    (tmp_path / "gen.json").write_text(json.dumps({
        "model": lm, "model_name": "tiny", "dataset": {"dataset_name_or_path": str(tiny_lm_workspace / "data"), "is_dataset_on_disk": True},
        "dataset_name": "toy", "hook_points": [hook], "output_dir": str(acts), "total_tokens": 512, "context_size": 16,
        "model_batch_size": 4, "batch_size": 4, "device_type": "cpu", "format": "safetensors"}))  # fmt: skip
    assert runner.invoke(app, ["generate", str(tmp_path / "gen.json")]).exit_code == 0
    settings = {
        "sae": {"hook_point_in": hook, "hook_point_out": hook, "d_model": 16, "expansion_factor": 4, "act_fn": "topk", "top_k": 4,
                "device": "cpu", "dtype": "float32"},
        "sae_name": "toy-sae", "sae_series": "test", "initializer": {},
        "trainer": {"lr": 1e-3, "total_training_tokens": 32 * 20, "log_frequency": 4, "eval_frequency": 1000000, "n_checkpoints": 0,
                    "lr_warm_up_steps": 2, "exp_result_path": str(out), "amp_dtype": "float32", "l1_coefficient": None},
        "activation_factory": {"sources": [{"type": "activations", "name": "toy", "path": str(acts), "device": "cpu", "num_workers": 0, "prefetch": None}],
                               "target": "activations-1d", "hook_points": [hook], "batch_size": 32, "num_workers": 0},
        "device_type": "cpu"}  # fmt: skip
    (tmp_path / "first.json").write_text(json.dumps(settings))
    r = runner.invoke(app, ["train", str(tmp_path / "first.json")])
    assert r.exit_code == 0, (r.output, r.exception)
    assert not (out / "sae_weights.safetensors").exists()
    (ckpt,) = list((out / "checkpoints").glob("step_*"))
    stopped_at = int(ckpt.name.split("_")[1])
    assert 0 < stopped_at < 20
    for name in ("sae_weights.safetensors", "config.json", "trainer.pt", "optimizer.pt", "scheduler.pt"):
        assert (ckpt / name).exists(), name
    state = torch.load(ckpt / "trainer.pt", weights_only=False)
    assert state["cur_step"] == stopped_at and state["total_training_steps"] == 20

    second = {**settings, "sae": {"pretrained_name_or_path": str(ckpt), "device": "cpu", "dtype": "float32"}, "initializer": None,
              "trainer": {**settings["trainer"], "from_pretrained_path": str(ckpt), "exp_result_path": str(tmp_path / "resumed")}}  # fmt: skip
    (tmp_path / "second.json").write_text(json.dumps(second))
    r = runner.invoke(app, ["train", str(tmp_path / "second.json")])
    assert r.exit_code == 0, (r.output, r.exception)
    done = tmp_path / "resumed"  # the final weights go where the second run's settings say
    assert (done / "sae_weights.safetensors").exists() and (done / "config.json").exists()
