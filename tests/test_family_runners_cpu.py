"""``train --kind crosscoder | clt | lorsa | molt`` from settings files, activations computed on the fly by the tiny language
model: each family's runner builds its dictionary (with the data-dependent initialisation), trains a few steps on the CPU,
saves weights and settings, and the saved dictionary loads again and reconstructs (runners/train.py of the reference
project: train_crosscoder, train_clt, train_lorsa, train_molt)."""

import json

import pytest
import torch
from typer.testing import CliRunner

from language_model_saes_b200.cli import app
from language_model_saes_b200.models.sparse_dictionary import SparseDictionary

runner = CliRunner()
UNTIED = {"init_encoder_with_decoder_transpose": False}  # only dictionaries with one encoder per decoder can start tied


def _settings(workspace, out, sae, hook_points, target, batch_size, *, name, trainer=None, initializer=None):
    lm = {"model_name": "gpt2", "model_from_pretrained_path": str(workspace / "model"), "local_files_only": True, "backend": "hooked",
          "device": "cpu", "dtype": "float32", "max_length": 32, "bos_token_id": 0, "eos_token_id": 0, "pad_token_id": 1}  # fmt: skip
    factory = {"sources": [{"type": "dataset", "name": "toy", "prepend_bos": True}], "target": target, "hook_points": hook_points,
               "batch_size": batch_size, "context_size": 16, "model_batch_size": 4, "num_workers": 0}  # fmt: skip
    return {
        "sae": {**sae, "device": "cpu", "dtype": "float32"}, "sae_name": name, "sae_series": "fam",
        "initializer": initializer if initializer is not None else {},
        "trainer": {"lr": 1e-3, "total_training_tokens": 384, "log_frequency": 2, "eval_frequency": 1000000, "n_checkpoints": 0, "lr_warm_up_steps": 2,
                    "exp_result_path": str(out), "amp_dtype": "float32", "l1_coefficient": None, **(trainer or {})},
        "model": lm, "model_name": "tiny", "datasets": {"toy": {"dataset_name_or_path": str(workspace / "data"), "is_dataset_on_disk": True}},
        "device_type": "cpu",
    }, factory  # fmt: skip


def _train(kind, settings, tmp_path):
    path = tmp_path / f"{kind}.json"
    path.write_text(json.dumps(settings))
    r = runner.invoke(app, ["train", str(path), "--kind", kind])
    assert r.exit_code == 0, (r.output, r.exception)


def _analyze(workspace, out, factory, name, tmp_path, **analyzer):
    """``analyze`` of a saved dictionary of any family into a file; returns the feature records."""
    import pickle

    s, _ = _settings(workspace, out, {}, [], "", 0, name=name)
    ana = tmp_path / "analysis"
    cfg = {"sae": {"pretrained_name_or_path": str(out), "device": "cpu", "dtype": "float32"}, "sae_name": name, "sae_series": "fam",
           "activation_factory": {**factory, "target": "activations-2d", "batch_size": 4}, "model": s["model"], "model_name": "tiny",
           "datasets": s["datasets"], "analyzer": {"total_analyzing_tokens": 256, **analyzer}, "output_dir": str(ana), "device_type": "cpu",
           "amp_dtype": "bfloat16"}  # fmt: skip
    path = tmp_path / "analyze.json"
    path.write_text(json.dumps(cfg))
    r = runner.invoke(app, ["analyze", str(path)])
    assert r.exit_code == 0, (r.output, r.exception)
    (pkl,) = list((ana / name / "fam").glob("*.pkl"))
    with open(pkl, "rb") as f:
        return pickle.load(f)


def _evaluate(workspace, out, factory, name, tmp_path, tokens):
    """``evaluate`` of a saved dictionary on activations computed on the fly."""
    s, _ = _settings(workspace, out, {}, [], "", 0, name=name)
    cfg = {"sae": {"pretrained_name_or_path": str(out), "device": "cpu", "dtype": "float32"}, "sae_name": name, "sae_series": "fam",
           "activation_factory": factory, "model": s["model"], "model_name": "tiny", "datasets": s["datasets"],
           "eval": {"total_eval_tokens": tokens}, "device_type": "cpu"}  # fmt: skip
    path = tmp_path / "evaluate.json"
    path.write_text(json.dumps(cfg))
    r = runner.invoke(app, ["evaluate", str(path)])
    assert r.exit_code == 0, (r.output, r.exception)


def _reload(out):
    assert (out / "config.json").exists() and (out / "sae_weights.safetensors").exists()
    m = SparseDictionary.from_pretrained(str(out), device="cpu", dtype=torch.float32)
    assert all(torch.isfinite(p).all() for p in m.parameters())
    return m


def test_cross_layer_transcoder(tiny_lm_workspace, tmp_path):
    out = tmp_path / "clt"
    ins, outs = [f"blocks.{l}.ln2.hook_normalized" for l in range(2)], [f"blocks.{l}.hook_mlp_out" for l in range(2)]
    s, f = _settings(tiny_lm_workspace, out, {"sae_type": "clt", "hook_points_in": ins, "hook_points_out": outs, "d_model": 16, "expansion_factor": 2,
                                              "act_fn": "topk", "top_k": 4}, ins + outs, "activations-1d", 64, name="toy-clt", initializer=UNTIED)  # fmt: skip
    _train("clt", {**s, "activation_factory": f}, tmp_path)
    m = _reload(out)
    assert type(m).__name__ == "CrossLayerTranscoder" and m.cfg.n_layers == 2
    x = torch.randn(5, 2, 16)  # [tokens, layers, d]; the reconstruction comes back layer-major
    assert m.forward(x).shape == (2, 5, 16)
    _evaluate(tiny_lm_workspace, out, f, "toy-clt", tmp_path, 128)
    records = _analyze(tiny_lm_workspace, out, f, "toy-clt", tmp_path, clt_layer=0)  # one layer's features per analysis
    assert len(records) == 32 and sum(r["act_times"] for r in records) > 0
    assert len(next(r for r in records if r["act_times"] > 0)["decoder_norms"]) == 2  # layer 0 writes to both layers


def test_low_rank_sparse_attention(tiny_lm_workspace, tmp_path):
    out = tmp_path / "lorsa"
    hin, hout = "blocks.1.ln1.hook_normalized", "blocks.1.hook_attn_out"
    s, f = _settings(tiny_lm_workspace, out, {"sae_type": "lorsa", "hook_point_in": hin, "hook_point_out": hout, "d_model": 16, "expansion_factor": 2,
                                              "n_qk_heads": 4, "d_qk_head": 8, "rotary_dim": 8, "n_ctx": 16, "act_fn": "topk", "top_k": 4,
                                              "positional_embedding_type": "rotary"},
                     [hin, hout], "activations-2d", 4, name="toy-lorsa", trainer={"total_training_tokens": 16 * 4 * 4}, initializer=UNTIED)  # fmt: skip
    _train("lorsa", {**s, "activation_factory": f}, tmp_path)
    m = _reload(out)
    assert type(m).__name__ == "LowRankSparseAttention"
    assert m.forward(torch.randn(2, 16, 16)).shape == (2, 16, 16)
    _evaluate(tiny_lm_workspace, out, f, "toy-lorsa", tmp_path, 128)
    records = _analyze(tiny_lm_workspace, out, f, "toy-lorsa", tmp_path)
    assert len(records) == 32 and sum(r["act_times"] for r in records) > 0
    top = next(r for r in records if r["act_times"] > 0)["samplings"][0]
    assert "z_pattern_indices" in top and "z_pattern_values" in top  # which source positions a head read from


def test_mixture_of_linear_transforms(tiny_lm_workspace, tmp_path):
    out = tmp_path / "molt"
    hin, hout = "blocks.1.ln2.hook_normalized", "blocks.1.hook_mlp_out"
    s, f = _settings(tiny_lm_workspace, out, {"sae_type": "molt", "hook_point_in": hin, "hook_point_out": hout, "d_model": 16, "expansion_factor": 2,
                                              "rank_counts": {"2": 16, "4": 16}, "act_fn": "relu"},
                     [hin, hout], "activations-1d", 64, name="toy-molt", trainer={"l1_coefficient": 1e-3}, initializer=UNTIED)  # fmt: skip
    _train("molt", {**s, "activation_factory": f}, tmp_path)
    m = _reload(out)
    assert type(m).__name__ == "MixtureOfLinearTransform"
    assert m.forward(torch.randn(5, 16)).shape == (5, 16)
    _evaluate(tiny_lm_workspace, out, f, "toy-molt", tmp_path, 128)


def test_crosscoder_over_two_layers_of_one_model(tiny_lm_workspace, tmp_path):
    out = tmp_path / "cc"
    hooks = ["blocks.0.hook_resid_post", "blocks.1.hook_resid_post"]
    s, f = _settings(tiny_lm_workspace, out, {"sae_type": "crosscoder", "hook_points": hooks, "d_model": 16, "expansion_factor": 2, "act_fn": "topk",
                                              "top_k": 4}, hooks, "activations-1d", 64, name="toy-cc")  # fmt: skip
    _train("crosscoder", {**s, "activation_factories": [f]}, tmp_path)
    m = _reload(out)
    assert type(m).__name__ == "Crosscoder" and m.cfg.n_heads == 2
    assert m.forward(torch.randn(5, 2, 16)).shape == (5, 2, 16)
    # the head count has to match the hook points the factories deliver
    bad = {**s, "activation_factories": [{**f, "hook_points": hooks[:1]}]}
    path = tmp_path / "bad.json"
    path.write_text(json.dumps(bad))
    r = runner.invoke(app, ["train", str(path), "--kind", "crosscoder"])
    assert r.exit_code != 0 and isinstance(r.exception, AssertionError)


def test_crosscoder_is_analysed_and_evaluated_from_cached_activations(tiny_lm_workspace, tmp_path):
    """``generate`` (sequence-shaped cache of both hook points) -> ``train --kind crosscoder`` from the cache -> ``analyze --kind
    crosscoder`` into a file -> ``evaluate --kind crosscoder``."""
    import pickle

    hooks = ["blocks.0.hook_resid_post", "blocks.1.hook_resid_post"]
    acts, out, ana = tmp_path / "acts", tmp_path / "cc", tmp_path / "analysis"
    s, _ = _settings(tiny_lm_workspace, out, {"sae_type": "crosscoder", "hook_points": hooks, "d_model": 16, "expansion_factor": 2, "act_fn": "topk",
                                              "top_k": 4}, hooks, "activations-1d", 64, name="toy-cc")  # fmt: skip
    gen = {"model": s["model"], "model_name": "tiny", "dataset": s["datasets"]["toy"], "dataset_name": "toy", "hook_points": hooks,
           "output_dir": str(acts), "total_tokens": 1024, "context_size": 16, "model_batch_size": 4, "batch_size": 4, "device_type": "cpu",
           "format": "safetensors"}  # fmt: skip
    (tmp_path / "gen.json").write_text(json.dumps(gen))
    r = runner.invoke(app, ["generate", str(tmp_path / "gen.json")])
    assert r.exit_code == 0, (r.output, r.exception)

    def cached(target, batch):
        return {"sources": [{"type": "activations", "name": "toy", "path": str(acts), "device": "cpu", "num_workers": 0, "prefetch": None}],
                "target": target, "hook_points": hooks, "batch_size": batch, "num_workers": 0}  # fmt: skip

    train = {k: v for k, v in s.items() if k not in ("model", "datasets")} | {"activation_factories": [cached("activations-1d", 64)]}
    _train("crosscoder", train, tmp_path)
    assert _reload(out).cfg.n_heads == 2

    pre = {"pretrained_name_or_path": str(out), "device": "cpu", "dtype": "float32"}
    (tmp_path / "ana.json").write_text(json.dumps({
        "sae": pre, "sae_name": "toy-cc", "sae_series": "fam", "activation_factories": [cached("activations-2d", 4)],
        "analyzer": {"total_analyzing_tokens": 256}, "output_dir": str(ana), "device_type": "cpu", "amp_dtype": "bfloat16"}))  # fmt: skip
    r = runner.invoke(app, ["analyze", str(tmp_path / "ana.json"), "--kind", "crosscoder"])
    assert r.exit_code == 0, (r.output, r.exception)
    (pkl,) = list((ana / "toy-cc" / "fam").glob("*.pkl"))
    with open(pkl, "rb") as f:
        records = pickle.load(f)
    assert len(records) == 32 and sum(rec["act_times"] for rec in records) > 0
    fired = next(rec for rec in records if rec["act_times"] > 0)
    assert len(fired["decoder_norms"]) == 2 and len(fired["decoder_similarity_matrices"]) == 2  # one entry per head

    (tmp_path / "eval.json").write_text(json.dumps({
        "sae": pre, "sae_name": "toy-cc", "sae_series": "fam", "activation_factories": [cached("activations-1d", 64)],
        "eval": {"total_eval_tokens": 128}, "device_type": "cpu"}))  # fmt: skip
    r = runner.invoke(app, ["evaluate", str(tmp_path / "eval.json"), "--kind", "crosscoder"])
    assert r.exit_code == 0, (r.output, r.exception)
