"""Activation pipeline pieces, writer / cached-loader round trips, pytrees, versioned serialisation, learning-rate
schedules, SparseAdam and checkpoint-resume equivalence on CPU (the unit-test ideas of the reference project:
tests/unit/test_activation_processors.py, test_activation_writer.py, test_pytree.py, test_serialize.py)."""

import dataclasses
from typing import Generic, TypeVar

import pytest
import torch

from language_model_saes_b200.activation.processors.activation import (
    ActivationBatchler,
    ActivationBuffer,
    ActivationGenerator,
    ActivationTransformer,
    BufferShuffleConfig,
    OverrideDtypeProcessor,
)
from language_model_saes_b200.activation.processors.cached_activation import CachedActivationLoader
from language_model_saes_b200.activation.processors.token import PadAndTruncateTokensProcessor
from language_model_saes_b200.activation.writer import ActivationWriter, ActivationWriterConfig
from language_model_saes_b200.core import serialize
from language_model_saes_b200.core.pytree import PyTree
from language_model_saes_b200.optim import SparseAdam, schedule_lambda


# ---- activation processors ---------------------------------------------------------------------------
class _FakeModel:
    """``to_activations`` returns arange tensors, as the mocked language model of the reference's tests does."""

    pad_token_id = 0

    def preprocess_raw_data(self, raw):
        return raw

    def to_activations(self, raw, hook_points, n_context=None):
        n = len(raw["text"])
        ctx = n_context or 4
        tokens = torch.arange(n * ctx).view(n, ctx) + 1
        out = {hp: torch.arange(n * ctx * 3, dtype=torch.float32).view(n, ctx, 3) + 100 * i for i, hp in enumerate(hook_points)}
        return {**out, "tokens": tokens, "mask": tokens % 4 != 1, "attention_mask": torch.ones_like(tokens, dtype=torch.bool)}


def test_pad_and_truncate():
    proc = PadAndTruncateTokensProcessor(seq_len=4)
    out = list(proc.process([{"tokens": torch.tensor([1, 2])}, {"tokens": torch.tensor([1, 2, 3, 4, 5, 6])}], pad_token_id=9))
    assert out[0]["tokens"].tolist() == [1, 2, 9, 9] and out[1]["tokens"].tolist() == [1, 2, 3, 4]


def test_generator_transformer_batchler_chain():
    gen = ActivationGenerator(hook_points=["h0", "h1"], batch_size=2, n_context=4)
    raw = [{"text": f"t{i}", "meta": {"i": i}} for i in range(5)]
    recs = list(gen.process(raw, model=_FakeModel(), model_name="fake"))
    assert [len(r["tokens"]) for r in recs] == [2, 2, 1]  # model batches of 2, the tail is kept
    assert recs[0]["h0"].shape == (2, 4, 3) and recs[0]["meta"][0]["model_name"] == "fake" and recs[0]["meta"][1]["i"] == 1
    flat = list(ActivationTransformer().process(recs))
    # masked tokens (ids congruent to 1 mod 4, i.e. the first of each context) are dropped; activations become 2-D
    assert flat[0]["h0"].shape == (6, 3) and flat[0]["tokens"].tolist() == [2, 3, 4, 6, 7, 8]
    assert torch.equal(flat[0]["h1"], flat[0]["h0"] + 100) and "meta" not in flat[0]
    ignored = list(ActivationTransformer().process(recs, ignore_token_ids=[2, 3]))
    assert ignored[0]["tokens"].tolist() == [1, 4, 5, 6, 7, 8]
    batches = list(ActivationBatchler(batch_size=4).process(flat))
    assert [len(b["tokens"]) for b in batches] == [4, 4, 4, 3]  # 15 kept tokens re-cut to 4 per batch
    assert torch.cat([b["tokens"] for b in batches]).tolist() == torch.cat([f["tokens"] for f in flat]).tolist()
    half = list(OverrideDtypeProcessor(torch.bfloat16).process(batches))
    assert half[0]["h0"].dtype == torch.bfloat16 and half[0]["tokens"].dtype == torch.int64


def test_buffer_is_a_fifo_and_shuffle_is_seeded():
    buf = ActivationBuffer()
    buf = buf.cat({"x": torch.arange(5)}).cat({"x": torch.arange(5, 8)})
    assert len(buf) == 8
    batch, rest = buf.yield_batch(6)
    assert batch["x"].tolist() == [0, 1, 2, 3, 4, 5] and rest.consume()["x"].tolist() == [6, 7] and len(buf) == 8  # out of place
    with pytest.raises(ValueError):
        ActivationBuffer().yield_batch(1)

    def run(seed):
        cfg = BufferShuffleConfig(perm_seed=seed, generator_device="cpu")
        data = [{"x": torch.arange(10 * i, 10 * i + 10)} for i in range(6)]
        return torch.cat([b["x"] for b in ActivationBatchler(batch_size=5, buffer_size=20, buffer_shuffle_config=cfg).process(data)])

    a, b, c = run(1), run(1), run(2)
    assert torch.equal(a, b) and not torch.equal(a, c)
    assert sorted(a.tolist()) == list(range(60)) and a.tolist() != list(range(60))  # a permutation, and actually mixed


@pytest.mark.parametrize("fmt", ["safetensors", "pt"])
@pytest.mark.parametrize("workers", [None, 2])
def test_writer_and_cached_loader_round_trip(tmp_path, fmt, workers):
    g = torch.Generator().manual_seed(0)
    chunks = [
        {"h0": torch.randn(3, 4, 8, generator=g), "h1": torch.randn(3, 4, 8, generator=g), "tokens": torch.arange(12).view(3, 4) + 100 * c,
         "mask": torch.ones(3, 4, dtype=torch.bool), "attention_mask": torch.ones(3, 4, dtype=torch.bool),
         "meta": [{"chunk": c, "row": r} for r in range(3)]}
        for c in range(4)
    ]  # fmt: skip
    cfg = ActivationWriterConfig(hook_points=["h0", "h1"], cache_dir=str(tmp_path), format=fmt, num_workers=workers)
    ActivationWriter(cfg).process(iter(chunks))
    files = sorted(p.name for p in (tmp_path / "h0").iterdir() if p.suffix == f".{fmt}")
    assert files == [f"chunk-{c:08d}.{fmt}" for c in range(4)]
    loader = CachedActivationLoader({"h0": tmp_path / "h0", "h1": tmp_path / "h1"}, device="cpu", num_workers=2 if workers else 0)
    back = list(loader.process())
    assert len(back) == 4
    for want, got in zip(chunks, back):
        for key in ("h0", "h1", "tokens", "mask", "attention_mask"):
            assert torch.equal(got[key], want[key]), key
        assert got["meta"] == want["meta"]
    # a hook point with a different number of chunks is refused; a missing directory too
    (tmp_path / "h1" / files[-1]).unlink()
    with pytest.raises(ValueError):
        list(CachedActivationLoader({"h0": tmp_path / "h0", "h1": tmp_path / "h1"}).process())
    with pytest.raises(FileNotFoundError):
        list(CachedActivationLoader({"h0": tmp_path / "nope"}).process())


def test_cached_loader_checks_tokens_agree_across_hook_points(tmp_path):
    from safetensors.torch import save_file

    for hp, shift in (("a", 0), ("b", 1)):
        (tmp_path / hp).mkdir()
        save_file({"activation": torch.zeros(2, 3, 4), "tokens": torch.arange(6).view(2, 3) + shift, "mask": torch.ones(2, 3, dtype=torch.bool),
                   "attention_mask": torch.ones(2, 3, dtype=torch.bool)}, str(tmp_path / hp / "chunk-0.safetensors"))  # fmt: skip
    with pytest.raises(AssertionError, match="tokens mismatch"):
        list(CachedActivationLoader({"a": tmp_path / "a", "b": tmp_path / "b"}).process())


# ---- pytree / serialisation ----------------------------------------------------------------------------
@dataclasses.dataclass
class _Leaf(PyTree):
    w: torch.Tensor
    tag: str = "leaf"


@dataclasses.dataclass
class _Tree(PyTree):
    leaf: _Leaf
    items: list[torch.Tensor]
    table: dict[str, torch.Tensor]
    n: int = 3


def test_pytree_maps_tensors_in_nested_containers():
    t = _Tree(_Leaf(torch.ones(2)), [torch.zeros(1), torch.ones(1)], {"a": torch.full((2,), 2.0)}, n=7)
    u = t.tree_map_tensor(lambda x: x + 1)
    assert type(u) is _Tree and type(u.leaf) is _Leaf and u.n == 7 and u.leaf.tag == "leaf"
    assert u.leaf.w.tolist() == [2, 2] and [x.item() for x in u.items] == [1, 2] and u.table["a"].tolist() == [3, 3]
    assert t.leaf.w.tolist() == [1, 1]  # out of place
    assert t.to("cpu").table["a"].device.type == "cpu"
    seen = []
    t.tree_map(lambda x: (seen.append(type(x).__name__), x)[1])
    assert "_Leaf" in seen and "Tensor" in seen  # tree_map hands nested pytrees to the function whole


V = TypeVar("V")


@dataclasses.dataclass
class _Box(Generic[V]):
    value: V
    history: tuple[V, ...] = ()


@dataclasses.dataclass
class _Record:
    name: str
    weights: torch.Tensor
    box: _Box[list[int]]
    extra: dict[str, float] = dataclasses.field(default_factory=dict)
    renamed: int = 0

    @serialize.migrate(before="2")
    @staticmethod
    def _from_v1(raw: dict) -> dict:
        raw = dict(raw)
        raw["renamed"] = raw.pop("old_name", 0)
        return raw


def test_serialize_round_trip_generics_and_migration():
    rec = _Record("r", torch.arange(3.0), _Box([1, 2], ([0], [1])), {"a": 0.5}, renamed=4)
    blob = serialize.dump(rec)
    assert blob["_version"] == serialize.FORMAT_VERSION and isinstance(blob["data"]["box"], dict)
    back = serialize.load(blob, _Record)
    assert back.name == "r" and torch.equal(back.weights, rec.weights) and back.renamed == 4
    assert isinstance(back.box, _Box) and back.box.value == [1, 2] and back.box.history == ([0], [1])
    again = serialize.loads(serialize.dumps(rec), _Record)
    assert again.extra == {"a": 0.5} and torch.equal(again.weights, rec.weights)
    # a blob written by format version 1 used another field name: the class's migration rewrites it while loading
    legacy = {"_version": "1", "data": {"name": "old", "weights": torch.zeros(1), "box": {"value": [9], "history": []}, "old_name": 11}}
    old = serialize.load(legacy, _Record)
    assert old.renamed == 11 and old.box.value == [9]
    current = {"_version": "2", "data": {"name": "new", "weights": torch.zeros(1), "box": {"value": [9], "history": []}, "renamed": 5}}
    assert serialize.load(current, _Record).renamed == 5  # not migrated


# ---- optimisation ----------------------------------------------------------------------------------------
def test_learning_rate_schedules_match_their_definitions():
    f = schedule_lambda("constantwithwarmup", warm_up_steps=4, training_steps=20, cool_down_steps=5, lr_end_ratio=0.1)
    assert [round(f(s), 4) for s in (0, 1, 3, 4, 10)] == [0.25, 0.5, 1.0, 1.0, 1.0]
    assert f(15) == pytest.approx(1.0) and f(16) == pytest.approx(0.1 + 0.9 / 5 * 4) and f(19) == pytest.approx(0.1 + 0.9 / 5)
    assert f(20) == pytest.approx(0.1 + 0.9 / 5)  # max(T - s, 1): the last value repeats
    lin = schedule_lambda("linearwarmupdecay", warm_up_steps=2, training_steps=10)
    assert [lin(0), lin(1), lin(2), lin(6)] == [0.5, 1.0, 1.0, 0.5]
    cos = schedule_lambda("cosineannealingwarmup", warm_up_steps=2, training_steps=10, lr_end=0.0)
    assert cos(2) == pytest.approx(1.0) and cos(6) == pytest.approx(0.5) and cos(10) == pytest.approx(0.0)
    ex = schedule_lambda("exponentialwarmup", warm_up_steps=2, training_steps=10, lr_end=1 / 16)
    assert ex(2) == pytest.approx(1.0) and ex(6) == pytest.approx(0.25) and ex(10) == pytest.approx(1 / 16)
    assert schedule_lambda(None)(123) == 1.0
    with pytest.raises(ValueError):
        schedule_lambda("nope", training_steps=1)


def test_sparse_adam_updates_only_where_the_gradient_is_nonzero():
    p = torch.nn.Parameter(torch.ones(4))
    q = torch.nn.Parameter(torch.ones(2))
    opt = SparseAdam([p, q], lr=0.1, betas=(0.9, 0.99))
    p.grad = torch.tensor([1.0, 0.0, -2.0, 0.0])
    q.grad = torch.zeros(2)
    opt.step()
    # first Adam step moves by lr * sign(g) where g != 0; untouched entries and all-zero parameters stay
    assert torch.allclose(p.data, torch.tensor([0.9, 1.0, 1.1, 1.0]), atol=1e-6) and torch.equal(q.data, torch.ones(2))
    m1 = opt.state[p]["exp_avg"].clone()
    p.grad = torch.tensor([0.0, 1.0, 0.0, 0.0])
    opt.step()
    m2 = opt.state[p]["exp_avg"]
    assert m2[0] == pytest.approx(0.9 * float(m1[0])) and m2[2] == pytest.approx(0.9 * float(m1[2]))  # moments decay everywhere
    assert p.data[0] == pytest.approx(0.9) and p.data[2] == pytest.approx(1.1)  # but parameters move only where g != 0
    assert p.data[1] < 1.0


# ---- checkpoint / resume ---------------------------------------------------------------------------------
def test_resume_from_checkpoint_continues_the_uninterrupted_run(tmp_path):
    from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
    from language_model_saes_b200.trainer import Trainer, TrainerConfig

    def stream(n, seed=0):
        g = torch.Generator().manual_seed(seed)
        basis = torch.randn(6, 16, generator=g)
        for _ in range(n):
            x = torch.relu(torch.randn(32, 6, generator=g)) @ basis
            yield {"in": x, "out": x, "tokens": torch.ones(32, dtype=torch.long)}

    def model():
        torch.manual_seed(0)
        cfg = SAEConfig(hook_point_in="in", hook_point_out="out", d_model=16, expansion_factor=4, act_fn="topk", top_k=4,
                        device="cpu", dtype=torch.float32, norm_activation="inference")  # fmt: skip
        m = SparseAutoEncoder(cfg)
        m.init_parameters(encoder_uniform_bound=0.3, decoder_uniform_bound=0.3, init_log_jumprelu_threshold_value=0.0)
        return m

    def trainer(exp, n_ckpt=0):
        return Trainer(TrainerConfig(lr=1e-2, total_training_tokens=32 * 12, lr_warm_up_steps=2, log_frequency=1000,
                                     n_checkpoints=n_ckpt, check_point_save_mode="linear", exp_result_path=str(exp),
                                     initial_k=4, k_warmup_steps=0, lr_scheduler_name="constantwithwarmup"))  # fmt: skip

    full = model()
    assert trainer(tmp_path / "full").fit(full, stream(12)) is None  # all 12 steps done

    first = model()
    t1 = trainer(tmp_path / "part")
    data = stream(12)
    assert t1.fit(first, (next(data) for _ in range(6))) is True and t1.cur_step == 6  # the stream ended half-way
    t1.save_checkpoint(first, tmp_path / "part")
    ckpt = tmp_path / "part" / "checkpoints" / "step_6"
    assert {"trainer.pt", "optimizer.pt", "scheduler.pt", "sae_weights.safetensors", "config.json"} <= {p.name for p in ckpt.iterdir()}
    from language_model_saes_b200.models.sparse_dictionary import SparseDictionary

    second = SparseDictionary.from_pretrained(str(ckpt), fold_activation_scale=False, device="cpu", dtype=torch.float32)
    t2 = Trainer.from_checkpoint(second, str(ckpt))
    assert t2.cur_step == 6 and t2.total_training_steps == 12
    assert t2.fit(second, data) is None and t2.cur_step == 12
    for (k, a), b in zip(full.state_dict().items(), second.state_dict().values()):
        assert torch.allclose(a, b, atol=1e-6), k
