"""``ActivationWriter`` case by case (the round trip through the cached loader is in test_data_and_core_cpu.py): directory
layout, what a chunk file holds in each format, re-chunking of single samples, the token budget, sharded file names, and
the refusals (unknown format, a record without one of the hook points, samples with differing keys). The cases follow
tests/unit/test_activation_writer.py of the reference project."""

import json
from concurrent.futures import ThreadPoolExecutor

import pytest
import torch
from safetensors.torch import load_file

from language_model_saes_b200.activation.writer import ActivationWriter, ActivationWriterConfig

HOOKS = ["blocks.0.hook_resid_post", "blocks.1.hook_resid_post"]


def _sample(i: int, n_ctx: int = 4, d: int = 8) -> dict:
    g = torch.Generator().manual_seed(i)
    rec = {hp: torch.randn(n_ctx, d, generator=g) for hp in HOOKS}
    rec["tokens"] = torch.arange(n_ctx) + 10 * i
    rec["meta"] = {"context_idx": i}
    return rec


def _chunk(c: int, rows: int = 3, n_ctx: int = 4, d: int = 8) -> dict:
    g = torch.Generator().manual_seed(100 + c)
    rec = {hp: torch.randn(rows, n_ctx, d, generator=g) for hp in HOOKS}
    rec["tokens"] = torch.arange(rows * n_ctx).view(rows, n_ctx) + 1000 * c
    rec["meta"] = [{"context_idx": c * rows + r} for r in range(rows)]
    return rec


def test_directories_are_created_per_hook_point(tmp_path):
    w = ActivationWriter(ActivationWriterConfig(hook_points=HOOKS, cache_dir=str(tmp_path / "cache")))
    assert all((tmp_path / "cache" / hp).is_dir() for hp in HOOKS) and w.executor is None
    pooled = ActivationWriter(ActivationWriterConfig(hook_points=HOOKS, cache_dir=str(tmp_path / "cache"), num_workers=2))
    assert isinstance(pooled.executor, ThreadPoolExecutor)


def test_pt_chunks_hold_activation_tokens_and_meta(tmp_path):
    chunks = [_chunk(0), _chunk(1)]
    ActivationWriter(ActivationWriterConfig(hook_points=HOOKS, cache_dir=str(tmp_path), format="pt")).process(iter(chunks))
    for hp in HOOKS:
        files = sorted(p.name for p in (tmp_path / hp).iterdir())
        assert files == ["chunk-00000000.pt", "chunk-00000001.pt"]
        for c, want in enumerate(chunks):
            got = torch.load(tmp_path / hp / f"chunk-{c:08d}.pt", weights_only=False)
            assert set(got) == {"activation", "tokens", "meta"}
            assert torch.equal(got["activation"], want[hp]) and torch.equal(got["tokens"], want["tokens"]) and got["meta"] == want["meta"]


def test_safetensors_chunks_put_meta_in_a_sidecar(tmp_path):
    chunks = [_chunk(0)]
    ActivationWriter(ActivationWriterConfig(hook_points=HOOKS, cache_dir=str(tmp_path), format="safetensors")).process(iter(chunks))
    for hp in HOOKS:
        assert sorted(p.name for p in (tmp_path / hp).iterdir()) == ["chunk-00000000.meta.json", "chunk-00000000.safetensors"]
        got = load_file(str(tmp_path / hp / "chunk-00000000.safetensors"))
        assert set(got) == {"activation", "tokens"} and torch.equal(got["activation"], chunks[0][hp])
        assert json.loads((tmp_path / hp / "chunk-00000000.meta.json").read_text()) == chunks[0]["meta"]


def test_single_samples_are_stacked_into_chunks_of_the_configured_size(tmp_path):
    samples = [_sample(i) for i in range(5)]
    cfg = ActivationWriterConfig(hook_points=HOOKS, cache_dir=str(tmp_path), format="pt", n_samples_per_chunk=2)
    ActivationWriter(cfg).process(iter(samples))
    files = sorted(p.name for p in (tmp_path / HOOKS[0]).iterdir())
    assert files == ["chunk-00000000.pt", "chunk-00000001.pt", "chunk-00000002.pt"]  # 2 + 2 + 1 samples
    first = torch.load(tmp_path / HOOKS[0] / files[0], weights_only=False)
    assert first["activation"].shape == (2, 4, 8) and torch.equal(first["activation"][1], samples[1][HOOKS[0]])
    assert first["meta"] == [{"context_idx": 0}, {"context_idx": 1}]
    last = torch.load(tmp_path / HOOKS[0] / files[2], weights_only=False)
    assert last["activation"].shape == (1, 4, 8) and torch.equal(last["tokens"][0], samples[4]["tokens"])


def test_without_a_chunk_size_every_record_is_one_file(tmp_path):
    samples = [_sample(i) for i in range(3)]
    ActivationWriter(ActivationWriterConfig(hook_points=HOOKS, cache_dir=str(tmp_path), format="pt")).process(iter(samples))
    files = sorted(p.name for p in (tmp_path / HOOKS[1]).iterdir())
    assert len(files) == 3
    assert torch.load(tmp_path / HOOKS[1] / files[2], weights_only=False)["activation"].shape == (4, 8)  # stored as it came


def test_token_budget_stops_the_writer(tmp_path):
    cfg = ActivationWriterConfig(hook_points=HOOKS, cache_dir=str(tmp_path), format="pt", total_generating_tokens=20)
    ActivationWriter(cfg).process(_chunk(c) for c in range(10))  # 12 tokens per chunk: the second chunk crosses 20
    assert len(list((tmp_path / HOOKS[0]).iterdir())) == 2


def test_worker_pool_writes_the_same_files(tmp_path):
    chunks = [_chunk(c) for c in range(6)]
    for workers, sub in ((None, "serial"), (3, "pool")):
        cfg = ActivationWriterConfig(hook_points=HOOKS, cache_dir=str(tmp_path / sub), format="safetensors", num_workers=workers)
        ActivationWriter(cfg).process(iter(chunks))
    for hp in HOOKS:
        a, b = sorted((tmp_path / "serial" / hp).iterdir()), sorted((tmp_path / "pool" / hp).iterdir())
        assert [p.name for p in a] == [p.name for p in b] and len(a) == 12
        for pa, pb in zip(a, b):
            assert pa.read_bytes() == pb.read_bytes()


def test_refusals(tmp_path):
    with pytest.raises(Exception):  # the config itself rejects a format it does not know
        ActivationWriterConfig(hook_points=HOOKS, cache_dir=str(tmp_path), format="npz")
    cfg = ActivationWriterConfig(hook_points=HOOKS, cache_dir=str(tmp_path), format="pt")
    w = ActivationWriter(cfg)
    w.cfg = cfg.model_copy(update={"format": "npz"})  # ... and so does the writer, should one get past the config
    with pytest.raises(ValueError, match="Invalid format"):
        w.process(iter([_chunk(0)]))
    missing = _chunk(0)
    del missing[HOOKS[1]]
    with pytest.raises(AssertionError, match="hook points"):
        ActivationWriter(cfg).process(iter([missing]))
    uneven = [_sample(0), {k: v for k, v in _sample(1).items() if k != "tokens"}]
    with pytest.raises(AssertionError, match="same keys"):
        ActivationWriter(cfg.model_copy(update={"n_samples_per_chunk": 2})).process(iter(uneven))
