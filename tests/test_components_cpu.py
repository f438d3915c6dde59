"""Behaviour specs of the components around the models: database client, hooked-transformer cache helpers and module
mounting, evaluator, initializer, local checkpoint loading (single process and sharded), and sharded state-dict loading
of every dictionary family. Same cases as the reference project's tests/unit/{test_database, test_tl_addons,
test_evaluator, test_initializer, test_from_local}.py and tests/distributed/{test_load_state_dict, test_utils}.py, on
this package's embedded store, own transformer and gloo ranks."""

import pytest
import torch
import torch.distributed as dist
import torch.nn as nn

from language_model_saes_b200.backend.hooked_transformer import HookedTransformer, HookedTransformerConfig
from language_model_saes_b200.database import MongoClient, MongoDBConfig, SAERecord
from language_model_saes_b200.evaluator import EvalConfig, Evaluator
from language_model_saes_b200.hooks import HookPoint
from language_model_saes_b200.initializer import Initializer, InitializerConfig
from language_model_saes_b200.models.clt import CLTConfig
from language_model_saes_b200.models.crosscoder import Crosscoder, CrosscoderConfig
from language_model_saes_b200.models.lorsa import LorsaConfig
from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
from language_model_saes_b200.models.sparse_dictionary import SparseDictionary
from language_model_saes_b200.parallel.mesh import build_mesh, execute_and_broadcast
from language_model_saes_b200.testing import distributed_test


# ---- database (embedded directory store behind the MongoClient interface) ---------------------------------------------
@pytest.fixture
def db(tmp_path):
    return MongoClient(MongoDBConfig(mongo_uri=f"file://{tmp_path / 'db'}", mongo_db="t"))


def _cfg(d_model=8, expansion=2):
    return SAEConfig(hook_point_in="h", hook_point_out="h", d_model=d_model, expansion_factor=expansion)


def test_database_saes_analyses_and_features(db):
    db.create_sae("sae1", "series1", "/p/1", _cfg())
    db.create_sae("sae2", "series1", "/p/2", _cfg())
    db.create_sae("sae3", "series2", "/p/3", _cfg(expansion=4))
    got = db.get_sae("sae3", "series2")
    assert isinstance(got, SAERecord) and (got.name, got.series, got.path) == ("sae3", "series2", "/p/3") and got.cfg.d_sae == 32
    assert set(db.list_saes()) == {"sae1", "sae2", "sae3"} and set(db.list_saes("series1")) == {"sae1", "sae2"}
    assert db.get_sae("nonexistent", "series1") is None and db.get_sae_path("sae1", "series1") == "/p/1"
    # creating a dictionary creates one feature record per latent
    f0 = db.get_feature("sae1", "series1", 0)
    assert f0 is not None and (f0.sae_name, f0.sae_series, f0.index) == ("sae1", "series1", 0)
    assert len(db.list_features("sae1", "series1", indices=range(4))) == 4 and db.get_feature("sae1", "series1", 16) is None
    db.create_analysis("probe", "sae1", "series1")
    assert db.list_analyses("sae1", "series1") == ["probe"] and db.list_saes("series1", has_analyses=True) == ["sae1"]
    rec = {"act_times": 3, "n_analyzed_tokens": 10, "max_feature_acts": 1.5, "samplings": []}
    db.add_feature_analysis("default", "sae1", "series1", [rec, {**rec, "act_times": 0, "max_feature_acts": 0.0}], start_idx=2)
    assert db.get_feature("sae1", "series1", 2).analyses[0].act_times == 3
    assert db.get_alive_feature_count("sae1", "series1") == 1 and db.get_max_feature_acts("sae1", "series1")[2] == 1.5
    db.update_feature("sae1", 2, {"interpretation": {"text": "a probe"}}, "series1")
    assert db.get_feature("sae1", "series1", 2).interpretation["text"] == "a probe"
    db.remove_sae("sae1", "series1")
    assert db.get_sae("sae1", "series1") is None and db.list_saes("series1") == ["sae2"] and db.get_feature("sae1", "series1", 0) is None


def test_database_bookmarks_sets_and_circuits(db):
    from language_model_saes_b200.database import CircuitConfig, CircuitStatus, CircuitTextInput

    db.create_sae("a", "s", "/a", _cfg())
    assert db.add_bookmark("a", "s", 1, tags=["x"], notes="n") and not db.add_bookmark("a", "s", 1)  # a second time: already there
    assert db.is_bookmarked("a", "s", 1) and db.get_bookmark("a", "s", 1).tags == ["x"] and db.get_bookmark_count("a", "s") == 1
    assert db.update_bookmark("a", "s", 1, notes="m") and db.list_bookmarks("a", "s")[0].notes == "m"
    assert db.remove_bookmark("a", "s", 1) and not db.is_bookmarked("a", "s", 1)
    db.add_sae_set("all", "s", ["a"])
    assert db.get_sae_set("all").sae_names == ["a"] and [x.name for x in db.list_sae_sets()] == ["all"]
    cid = db.create_circuit("all", "s", "a prompt", CircuitTextInput(text="a prompt"), CircuitConfig(), name="c", group=None)
    assert db.get_circuit(cid).status == CircuitStatus.PENDING and db.get_circuit_status(cid)["progress"] in (None, 0, 0.0)
    db.update_circuit_progress(cid, 0.5, "attributing")
    db.update_circuit_status(cid, CircuitStatus.FAILED, error_message="boom")
    st = db.get_circuit_status(cid)
    assert st["progress"] == 0.5 and st["progress_phase"] == "attributing" and st["error_message"] == "boom"
    assert db.update_circuits_group([cid], "g") == 1 and db.list_circuits("s", group="g")[0].id == cid
    assert db.delete_circuit(cid) and db.get_circuit(cid) is None


# ---- hooked transformer: partial forward with a cache, graph-attached cache, mounting extra hooked modules ------------
def _tiny_transformer():
    torch.manual_seed(0)
    return HookedTransformer(HookedTransformerConfig(n_layers=3, d_model=16, n_heads=2, d_vocab=50, n_ctx=32))


class _Probe(nn.Module):
    """A stand-in for a dictionary: one hook point that sees whatever is passed through."""

    def __init__(self):
        super().__init__()
        self.hook_seen = HookPoint()

    def forward(self, x):
        return self.hook_seen(x)


def test_run_with_cache_until_matches_run_with_cache_and_skips_later_layers():
    m, toks = _tiny_transformer(), torch.randint(0, 50, (2, 8))
    names = ["blocks.0.hook_resid_pre", "blocks.0.attn.hook_q", "blocks.1.hook_mlp_out"]  # not in module-definition order
    _, full = m.run_with_cache(toks, names_filter=names)
    ran = []
    m.add_hook("blocks.2.hook_resid_pre", lambda t, hook: ran.append(hook.name))
    out, part = m.run_with_cache_until(toks, names_filter=names)
    m.reset_hooks()
    assert out is None and ran == []  # stopped before the last block ran
    assert set(part) == set(names) and all(torch.equal(part[n], full[n]) for n in names)
    _, early = m.run_with_cache_until(toks, names_filter=names[:2])  # the later-defined hook of the two runs first
    assert set(early) == set(names[:2])
    logits, explicit = m.run_with_cache_until(toks, names_filter=names[:1], until="blocks.1.hook_resid_post")
    assert logits is None and set(explicit) == {names[0]}


def test_run_with_ref_cache_keeps_the_graph():
    m, toks = _tiny_transformer(), torch.randint(0, 50, (2, 8))
    names = ["blocks.0.hook_resid_post", "blocks.1.hook_resid_post"]
    _, detached = m.run_with_cache(toks, names_filter=names)
    logits, ref = m.run_with_ref_cache(toks, names_filter=names, retain_grad=True)
    assert all(torch.equal(ref[n], detached[n]) for n in names)
    assert all(ref[n].requires_grad and ref[n].grad_fn is not None for n in names) and not detached[names[0]].requires_grad
    logits.sum().backward()
    assert ref[names[1]].grad is not None and float(ref[names[1]].grad.abs().sum()) > 0


def test_mount_hooked_modules_attaches_and_always_detaches():
    m, toks = _tiny_transformer(), torch.randint(0, 50, (2, 8))
    before = set(m.hook_dict)
    want = m(toks)
    a, b = _Probe(), _Probe()
    with m.mount_hooked_modules([("blocks.0.hook_mlp_out", "sae", a), ("blocks.1.hook_attn_out", "lorsa", b)]):
        assert m.mod_dict["blocks.0.hook_mlp_out.sae"] is a and "blocks.1.hook_attn_out.lorsa.hook_seen" in m.hook_dict
        # a hook on the mounted child fires when the parent hook's user calls the child during the forward pass
        seen = []
        m.add_hook("blocks.0.hook_mlp_out", lambda t, hook: a(t))
        m.add_hook("blocks.0.hook_mlp_out.sae.hook_seen", lambda t, hook: seen.append(t.shape))
        assert torch.equal(m(toks), want) and seen == [(2, 8, 16)]
        m.reset_hooks()
    assert set(m.hook_dict) == before and not hasattr(m.blocks[0].hook_mlp_out, "sae")
    with pytest.raises(RuntimeError, match="inside"):
        with m.mount_hooked_modules([("blocks.0.hook_mlp_out", "sae", a)]):
            raise RuntimeError("inside")
    assert set(m.hook_dict) == before  # removed although the block raised
    assert torch.equal(m(toks), want)


# ---- evaluator and initializer ------------------------------------------------------------------------------------
def _stream(n, batch=64, d=8, seed=0):
    g = torch.Generator().manual_seed(seed)
    basis = torch.randn(4, d, generator=g)
    for _ in range(n):
        x = torch.randn(batch, 4, generator=g) @ basis
        yield {"h": x, "tokens": torch.ones(batch, dtype=torch.long), "mask": torch.ones(batch, dtype=torch.bool)}


def test_evaluator_reports_the_standard_metrics_and_honours_the_token_budget():
    torch.manual_seed(0)
    sae = SparseAutoEncoder(SAEConfig(hook_point_in="h", hook_point_out="h", d_model=8, expansion_factor=4, act_fn="topk", top_k=4))
    sae.init_parameters(encoder_uniform_bound=0.5, decoder_uniform_bound=0.5)
    sae.set_dataset_average_activation_norm({"h": 8**0.5})
    seen = []

    def counted():
        for b in _stream(10):
            seen.append(b["tokens"].numel())
            yield b

    logged = []

    class Log:
        def log(self, d, **kw):
            logged.append(d)

    out = Evaluator(EvalConfig(total_eval_tokens=150)).evaluate(sae, counted(), wandb_logger=Log())
    assert sum(seen) == 192  # three batches of 64: the stream is left as soon as the budget is reached
    for key in ("metrics/l0", "metrics/explained_variance", "metrics/l2_norm_error"):
        assert key in out and isinstance(out[key], float)
    assert out["metrics/l0"] == pytest.approx(4.0) and out["metrics/explained_variance"] <= 1.0
    assert logged == [out]


def test_initializer_ties_the_encoder_and_searches_the_norm():
    cfg = SAEConfig(hook_point_in="h", hook_point_out="h", d_model=8, expansion_factor=4, act_fn="relu", norm_activation="dataset-wise")
    init = Initializer(InitializerConfig(grid_search_init_norm=True, init_encoder_with_decoder_transpose=True,
                                         init_encoder_with_decoder_transpose_factor=1.0))  # fmt: skip
    torch.manual_seed(0)
    sae = init.initialize_sae_from_config(cfg, activation_stream=_stream(4), activation_norm={"h": 8**0.5})
    assert isinstance(sae, SparseAutoEncoder) and sae.dataset_average_activation_norm == {"h": 8**0.5}
    # after the search every decoder row has ONE common norm and the encoder is the decoder's transpose
    norms = sae.W_D.detach().norm(dim=1)
    assert torch.allclose(norms, norms[0].expand_as(norms), rtol=1e-4) and torch.allclose(sae.W_E.detach(), sae.W_D.detach().t())
    # the norm it picked is no worse than its neighbours on the batch it searched with
    batch = sae.normalize_activations(next(_stream(1)))

    def mse(scale):
        probe = SparseAutoEncoder(cfg)
        probe.load_state_dict(sae.state_dict())
        probe.set_dataset_average_activation_norm({"h": 8**0.5})
        with torch.no_grad():
            probe.W_D.mul_(scale)
            probe.W_E.copy_(probe.W_D.t())
        return float(probe.compute_loss(batch)["l_rec"].float().mean())

    assert mse(1.0) <= mse(3.0) and mse(1.0) <= mse(0.3)
    # without the search the uniform bounds of the config are used as they are
    plain = Initializer(InitializerConfig(encoder_uniform_bound=0.25, decoder_uniform_bound=0.5, init_encoder_with_decoder_transpose=False))
    sae2 = plain.initialize_sae_from_config(cfg.model_copy(update={"norm_activation": "token-wise"}), activation_stream=_stream(1))
    assert float(sae2.W_D.abs().max()) <= 0.5 and float(sae2.W_E.abs().max()) <= 0.25 and float(sae2.b_E.abs().max()) == 0.0


# ---- local checkpoints and sharded loading ---------------------------------------------------------------------------
def _family_configs():
    return {
        "sae": SAEConfig(hook_point_in="h", hook_point_out="h", d_model=8, expansion_factor=4, act_fn="topk", top_k=4),
        "crosscoder": CrosscoderConfig(hook_points=["a", "b"], d_model=8, expansion_factor=4, act_fn="topk", top_k=4),
        "clt": CLTConfig(hook_points_in=["i0", "i1"], hook_points_out=["o0", "o1"], d_model=8, expansion_factor=4, act_fn="topk", top_k=4),
        "lorsa": LorsaConfig(hook_point_in="x", hook_point_out="y", d_model=8, expansion_factor=4, n_qk_heads=4, d_qk_head=4,
                             rotary_dim=4, n_ctx=16, act_fn="topk", top_k=4),  # fmt: skip
    }


def _saved(cfg, path, seed=0):
    torch.manual_seed(seed)
    m = SparseDictionary.from_config(cfg)
    m.init_parameters(encoder_uniform_bound=0.5, decoder_uniform_bound=0.5)
    m.set_dataset_average_activation_norm({h: 2.0 + i for i, h in enumerate(cfg.associated_hook_points)})
    m.save_pretrained(path)
    m.cfg.save_hyperparameters(path)
    return m


@pytest.mark.parametrize("family", ["sae", "crosscoder", "clt", "lorsa"])
def test_from_local_restores_config_and_weights(tmp_path, family):
    cfg = _family_configs()[family]
    src = _saved(cfg, tmp_path / family)
    got = SparseDictionary.from_pretrained(str(tmp_path / family))
    assert type(got) is type(src) and got.cfg.d_sae == src.cfg.d_sae
    want = src.full_state_dict()
    have = got.full_state_dict()
    assert set(have) == set(want) and all(torch.equal(have[k], want[k]) for k in want)


@distributed_test(nproc_per_node=2, backend="gloo")
def test_sharded_loading_of_every_family_matches_the_full_state(tmp_path_factory=None):
    """Every rank loads its shard (from the full state dict and from a local checkpoint); gathering gives the full
    tensors back, for SAE, crosscoder, cross-layer transcoder and Lorsa."""
    import tempfile

    mesh = build_mesh("cpu", (1, 2), ("data", "model"))
    root = execute_and_broadcast(lambda: tempfile.mkdtemp(prefix="lmsae_fromlocal_"), mesh)
    for family, cfg in _family_configs().items():
        torch.manual_seed(0)
        full = SparseDictionary.from_config(cfg)
        full.init_parameters(encoder_uniform_bound=0.5, decoder_uniform_bound=0.5)
        full.set_dataset_average_activation_norm({h: 2.0 + i for i, h in enumerate(cfg.associated_hook_points)})
        want = full.full_state_dict()
        if dist.get_rank() == 0:
            full.save_pretrained(f"{root}/{family}")
            full.cfg.save_hyperparameters(f"{root}/{family}")
        dist.barrier()
        sharded = SparseDictionary.from_config(cfg, device_mesh=mesh)
        sharded.load_full_state_dict(want)
        local = SparseDictionary.from_pretrained(f"{root}/{family}", device_mesh=mesh)
        for m in (sharded, local):
            have = m.full_state_dict()
            assert set(have) == set(want), family
            for k in want:
                assert torch.equal(have[k], want[k]), (family, k)
            # something really is sharded: the local parameter count is below the full one
            assert sum(p.numel() for p in m.parameters()) < sum(p.numel() for p in full.parameters()), family


@distributed_test(nproc_per_node=2, backend="gloo")
def test_execute_and_broadcast_runs_once_and_shares_the_result():
    mesh = build_mesh("cpu", (2,), ("data",))
    calls = []

    def fn():
        calls.append(dist.get_rank())
        return {"rank": dist.get_rank(), "value": [1, 2, 3]}

    out = execute_and_broadcast(fn, mesh)
    assert out == {"rank": 0, "value": [1, 2, 3]}  # rank 0's result everywhere
    assert calls == ([0] if dist.get_rank() == 0 else [])
    assert execute_and_broadcast(lambda: 7, None) == 7  # no mesh: just a call


def test_closed_form_lr_factor_equals_the_torch_scheduler_for_every_schedule():
    """The fused path never steps the torch scheduler; it evaluates ``schedule_lambda`` instead. Both must give the same
    learning rate at every step, for every scheduler name the trainer configuration accepts."""
    import torch

    from language_model_saes_b200.optim import get_scheduler, schedule_lambda

    base, total = 3e-4, 40
    kw = dict(warm_up_steps=5, cool_down_steps=8, training_steps=total, lr_end_ratio=1 / 32)
    for name in ("constant", "constantwithwarmup", "linearwarmupdecay", "cosineannealing", "cosineannealingwarmup", "exponentialwarmup"):
        p = torch.nn.Parameter(torch.zeros(2))
        opt = torch.optim.Adam([p], lr=base)
        sched = get_scheduler(name, opt, **kw)
        factor = schedule_lambda(name, base_lr=base, **kw)
        for s in range(total):
            assert abs(sched.get_last_lr()[0] - base * factor(s)) <= 1e-9 + 1e-6 * base, (name, s)
            opt.step()
            sched.step()


def test_trainer_remembers_whether_a_reused_device_mask_is_all_true(tmp_path):
    """The fused paths that refuse masked tokens ask a device mask once per tensor object, not once per step; a changed or
    different tensor is asked again (here on the CPU, with the device branch reached through a stand-in device type)."""
    from language_model_saes_b200.trainer import Trainer, TrainerConfig

    tr = Trainer(TrainerConfig(total_training_tokens=10, exp_result_path=str(tmp_path), n_checkpoints=0))
    assert tr._all_tokens_valid({}) and tr._all_tokens_valid({"mask": torch.ones(4, dtype=torch.bool)})
    assert not tr._all_tokens_valid({"mask": torch.tensor([True, False])})
    assert tr._all_tokens_valid({"mask": torch.tensor([True, False]), "_mask_all": True})  # the summary made on arrival wins

    class OnDevice(torch.Tensor):  # a CPU tensor that says it lives elsewhere, and counts how often it is read
        reads = 0

        @property
        def device(self):
            return torch.device("meta")

        def all(self, *a, **k):
            OnDevice.reads += 1
            return torch.Tensor.all(self.as_subclass(torch.Tensor), *a, **k)

    m = torch.ones(6, dtype=torch.bool).as_subclass(OnDevice)
    assert tr._all_tokens_valid({"mask": m}) and tr._all_tokens_valid({"mask": m}) and OnDevice.reads == 1
    m[2] = False  # an in-place change is seen through the tensor's version counter
    assert not tr._all_tokens_valid({"mask": m}) and OnDevice.reads == 2
    other = torch.ones(6, dtype=torch.bool).as_subclass(OnDevice)
    assert tr._all_tokens_valid({"mask": other}) and OnDevice.reads == 3
