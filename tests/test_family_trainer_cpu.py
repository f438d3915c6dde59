"""``Trainer.fit`` on the fused paths of the Lorsa and cross-layer transcoder families, on the CPU: the trainer's own
parts of those paths (selection, schedules, masks as row weights, logging of the generic metric set, checkpoints and
resuming) run here with the engines' torch statements. Only the condition "the model is on a GPU" is set aside, by
asking each engine for its model-only conditions."""

import copy

import pytest
import torch

from language_model_saes_b200.models.clt import CLTConfig, CrossLayerTranscoder
from language_model_saes_b200.models.lorsa import LorsaConfig, LowRankSparseAttention
from language_model_saes_b200.models.sparse_dictionary import SparseDictionary
from language_model_saes_b200.ops.fused_clt import FusedCLTStep
from language_model_saes_b200.ops.fused_lorsa import FusedLorsaStep
from language_model_saes_b200.trainer import Trainer, TrainerConfig


@pytest.fixture
def fused_on_cpu(monkeypatch):
    for cls in (FusedCLTStep, FusedLorsaStep):
        orig = cls.supports
        monkeypatch.setattr(cls, "supports", staticmethod(lambda model, trainer_cfg=None, _orig=orig: _orig(model, None)))


def lorsa(seed=0):
    torch.manual_seed(seed)
    cfg = LorsaConfig(hook_point_in="blocks.1.ln1.hook_normalized", hook_point_out="blocks.1.hook_attn_out", d_model=64, expansion_factor=1,
                      n_qk_heads=2, d_qk_head=16, rotary_dim=16, n_ctx=16, act_fn="topk", top_k=6, device="cpu", dtype=torch.float32,
                      norm_activation="inference")  # fmt: skip
    m = LowRankSparseAttention(cfg)
    m.init_parameters()
    return m


def lorsa_stream(n, b=2, s=16, d=64, seed=1, masked=False):
    g = torch.Generator().manual_seed(seed)
    mix = torch.randn(d, d, generator=g) / d**0.5
    for _ in range(n):
        x = torch.randn(b, s, d, generator=g)
        y = torch.tanh(x @ mix).cumsum(1) / 4
        rec = {"blocks.1.ln1.hook_normalized": x, "blocks.1.hook_attn_out": y, "tokens": torch.ones(b, s, dtype=torch.long)}
        if masked:
            rec["mask"] = torch.rand(b, s, generator=g) > 0.2
        yield rec


def trainer(path, tokens, **kw):
    base = dict(lr=1e-3, total_training_tokens=tokens, lr_warm_up_steps=2, log_frequency=1000, n_checkpoints=0, exp_result_path=str(path),
                lr_scheduler_name="constantwithwarmup", amp_dtype=torch.bfloat16)  # fmt: skip
    base.update(kw)
    return Trainer(TrainerConfig(**base))


def test_lorsa_fit_takes_the_fused_step_logs_and_weighs_masked_tokens(fused_on_cpu, tmp_path):
    m = lorsa()
    tr = trainer(tmp_path, 32 * 8, log_frequency=4, skip_metrics_calculation=False)
    emitted = []
    tr._emit = lambda sae, out: emitted.append(out)
    assert tr.fit(m, lorsa_stream(9, masked=True)) is None
    assert type(tr.fused).__name__ == "FusedLorsaStep" and tr.cur_step == 8
    assert len(emitted) == 2 and all({"metrics/explained_variance", "metrics/l0", "losses/mse_loss", "details/current_learning_rate"} <= set(e) for e in emitted)
    assert emitted[0]["details/current_learning_rate"] == pytest.approx(1e-3)  # past the two warm-up steps
    # the same run on the generic path (autograd, torch Adam) gives the same weights: masks, schedule and loss agree
    m2 = lorsa()
    tr2 = trainer(tmp_path / "generic", 32 * 8, use_fused_kernels=False, amp_dtype=torch.float32)
    assert tr2.fit(m2, lorsa_stream(9, masked=True)) is None and tr2.fused is None
    start = lorsa()
    for (name, p), (_, q), (_, p0) in zip(m.named_parameters(), m2.named_parameters(), start.named_parameters()):
        if name == "b_K":
            continue  # a bias on every key: its true gradient is (close to) zero, Adam steps along rounding noise
        moved = float((q - p0).abs().mean())
        assert float((p - q).abs().mean()) < 0.1 * moved + 1e-7, name


def test_lorsa_fused_run_resumes_from_a_trainer_checkpoint(fused_on_cpu, tmp_path):
    full = lorsa()
    assert trainer(tmp_path / "full", 32 * 10).fit(full, lorsa_stream(11)) is None
    first = lorsa()
    t1 = trainer(tmp_path / "part", 32 * 10)
    data = lorsa_stream(11)
    assert t1.fit(first, (next(data) for _ in range(5))) is True and t1.cur_step == 5
    t1.save_checkpoint(first, tmp_path / "part")
    ckpt = tmp_path / "part" / "checkpoints" / "step_5"
    second = SparseDictionary.from_pretrained(str(ckpt), fold_activation_scale=False, device="cpu", dtype=torch.float32)
    t2 = Trainer.from_checkpoint(second, str(ckpt))
    assert t2.fit(second, data) is None and t2.cur_step == 10 and type(t2.fused).__name__ == "FusedLorsaStep"
    assert t2.fused.t == 10  # the engine's Adam step counter came back with the moments
    for (k, a), b in zip(full.state_dict().items(), second.state_dict().values()):
        assert torch.allclose(a, b, atol=1e-6), k


def clt(seed=0):
    torch.manual_seed(seed)
    cfg = CLTConfig(hook_points_in=["i0", "i1", "i2"], hook_points_out=["o0", "o1", "o2"], d_model=32, expansion_factor=4, act_fn="topk", top_k=4,
                    device="cpu", dtype=torch.float32, norm_activation="inference")  # fmt: skip
    m = CrossLayerTranscoder(cfg)
    m.init_parameters(encoder_uniform_bound=0.3, decoder_uniform_bound=0.2)
    return m


def clt_stream(n, B=48, d=32, seed=2, masked=False):
    g = torch.Generator().manual_seed(seed)
    for _ in range(n):
        rec = {f"i{l}": torch.randn(B, d, generator=g) for l in range(3)}
        rec |= {f"o{l}": torch.randn(B, d, generator=g) * 0.5 for l in range(3)}
        rec["tokens"] = torch.ones(B, dtype=torch.long)
        if masked:
            rec["mask"] = torch.rand(B, generator=g) > 0.3
        yield rec


def test_clt_fit_takes_the_fused_step_ignores_masks_and_resumes(fused_on_cpu, tmp_path):
    full, masked = clt(), clt()
    assert trainer(tmp_path / "a", 48 * 8).fit(full, clt_stream(9)) is None
    tr = trainer(tmp_path / "b", 48 * 8, log_frequency=4, skip_metrics_calculation=False)
    emitted = []
    tr._emit = lambda sae, out: emitted.append(out)
    assert tr.fit(masked, clt_stream(9, masked=True)) is None and type(tr.fused).__name__ == "FusedCLTStep"
    assert len(emitted) == 2 and "metrics/explained_variance" in emitted[0]
    # this model's loss is the mean over all tokens and layers, mask or not. (The masked stream draws one more tensor per
    # batch, so the two runs see different data: compare a masked and an unmasked run on the SAME batches instead.)
    same, same_masked = clt(), clt()
    batches = list(clt_stream(9))
    with_mask = [dict(b, mask=torch.arange(48) % 3 != 0) for b in batches]
    assert trainer(tmp_path / "c", 48 * 8).fit(same, iter(copy.deepcopy(batches))) is None
    assert trainer(tmp_path / "d", 48 * 8).fit(same_masked, iter(with_mask)) is None
    for (k, a), b in zip(same.state_dict().items(), same_masked.state_dict().values()):
        assert torch.equal(a, b), k
    # resume
    first = clt()
    t1 = trainer(tmp_path / "part", 48 * 8)
    data = clt_stream(9)
    assert t1.fit(first, (next(data) for _ in range(4))) is True
    t1.save_checkpoint(first, tmp_path / "part")
    ckpt = tmp_path / "part" / "checkpoints" / "step_4"
    second = SparseDictionary.from_pretrained(str(ckpt), fold_activation_scale=False, device="cpu", dtype=torch.float32)
    t2 = Trainer.from_checkpoint(second, str(ckpt))
    assert t2.fit(second, data) is None and t2.cur_step == 8 and type(t2.fused).__name__ == "FusedCLTStep"
    for (k, a), b in zip(full.state_dict().items(), second.state_dict().values()):
        assert torch.allclose(a, b, atol=1e-6), k


def test_explained_variance_of_a_layer_major_label_uses_per_layer_means():
    """A cross-layer transcoder keeps labels and reconstructions as ``[layers, tokens, d]``: the variance is taken around
    each layer's own mean over the (valid) tokens."""
    from language_model_saes_b200.metrics import ExplainedVarianceMetric

    m = clt()
    g = torch.Generator().manual_seed(0)
    label = torch.randn(3, 48, 32, generator=g) + torch.arange(3.0).view(3, 1, 1)  # layers with different means
    rec = label + 0.3 * torch.randn(3, 48, 32, generator=g)
    mask = torch.rand(48, generator=g) > 0.3
    for msk in (None, mask):
        metric = ExplainedVarianceMetric(m)
        out = metric.update({"label": label, "reconstructed": rec, "mask": msk})
        keep = torch.ones(48, dtype=torch.bool) if msk is None else msk
        lab, r = label[:, keep], rec[:, keep]
        err = (r - lab).pow(2).sum(-1).mean(1)
        var = (lab - lab.mean(1, keepdim=True)).pow(2).sum(-1).mean(1)
        assert torch.allclose(out["explained_variance"], 1 - err / var, atol=1e-5)
        assert 0.85 < float(out["explained_variance"].mean()) < 0.95


@pytest.fixture
def crosscoder_on_cpu(monkeypatch):
    from language_model_saes_b200.ops.fused_crosscoder import FusedCrosscoderStep

    orig = FusedCrosscoderStep.supports
    monkeypatch.setattr(FusedCrosscoderStep, "supports", staticmethod(lambda model, trainer_cfg=None, _orig=orig: _orig(model, None)))


def jumprelu_sae(seed=0):
    from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder

    torch.manual_seed(seed)
    cfg = SAEConfig(hook_point_in="h", hook_point_out="h", d_model=64, expansion_factor=4, act_fn="jumprelu", device="cpu", dtype=torch.float32,
                    norm_activation="inference")  # fmt: skip
    m = SparseAutoEncoder(cfg)
    m.init_parameters(encoder_uniform_bound=0.2, decoder_uniform_bound=0.2, init_log_jumprelu_threshold_value=-1.0)
    m.set_decoder_to_fixed_norm(1.0, True)
    m.init_encoder_with_decoder_transpose()
    return m


def sae_stream(n, B=64, d=64, seed=3):
    g = torch.Generator().manual_seed(seed)
    basis = torch.randn(10, d, generator=g)
    for _ in range(n):
        x = torch.randn(B, 10, generator=g) @ basis + 0.05 * torch.randn(B, d, generator=g)
        yield {"h": x * (d**0.5 / x.norm(dim=-1).mean()), "tokens": torch.ones(B, dtype=torch.long)}


@pytest.mark.parametrize("penalty", ["tanh", "tanh-quad"])
def test_jumprelu_sae_fit_on_the_fused_step_follows_the_generic_run_and_resumes(crosscoder_on_cpu, tmp_path, penalty):
    kw = dict(sparsity_loss_type=penalty, l1_coefficient=0.02, jumprelu_lr_factor=0.5)
    fused = jumprelu_sae()
    tr = trainer(tmp_path / "fused", 64 * 10, log_frequency=5, skip_metrics_calculation=False, **kw)
    emitted = []
    tr._emit = lambda sae, out: emitted.append(out)
    assert tr.fit(fused, sae_stream(11)) is None
    assert type(tr.fused).__name__ == "FusedCrosscoderStep" and tr.fused.single
    assert len(emitted) == 2 and {"losses/sparsity_loss", "metrics/explained_variance", "metrics/l0"} <= set(emitted[0])
    generic = jumprelu_sae()
    tg = trainer(tmp_path / "generic", 64 * 10, use_fused_kernels=False, amp_dtype=torch.float32, **kw)
    assert tg.fit(generic, sae_stream(11)) is None and tg.fused is None
    start = jumprelu_sae()
    for (name, p), (_, q), (_, p0) in zip(fused.named_parameters(), generic.named_parameters(), start.named_parameters()):
        moved = float((q - p0).abs().mean())
        assert float((p - q).abs().mean()) < 0.1 * moved + 1e-7, name
    # resume half-way: same end state as the uninterrupted fused run
    first = jumprelu_sae()
    t1 = trainer(tmp_path / "part", 64 * 10, **kw)
    data = sae_stream(11)
    assert t1.fit(first, (next(data) for _ in range(5))) is True
    t1.save_checkpoint(first, tmp_path / "part")
    ckpt = tmp_path / "part" / "checkpoints" / "step_5"
    second = SparseDictionary.from_pretrained(str(ckpt), fold_activation_scale=False, device="cpu", dtype=torch.float32)
    t2 = Trainer.from_checkpoint(second, str(ckpt))
    assert t2.fit(second, data) is None and t2.cur_step == 10 and type(t2.fused).__name__ == "FusedCrosscoderStep"
    for (k, a), b in zip(fused.state_dict().items(), second.state_dict().values()):
        assert torch.allclose(a, b, atol=1e-6), k


def jumprelu_transcoder(seed=0):
    from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder

    torch.manual_seed(seed)
    cfg = SAEConfig(hook_point_in="pre", hook_point_out="post", d_model=64, expansion_factor=4, act_fn="jumprelu", device="cpu",
                    dtype=torch.float32, norm_activation="inference")  # fmt: skip
    m = SparseAutoEncoder(cfg)
    m.init_parameters(encoder_uniform_bound=0.2, decoder_uniform_bound=0.2, init_log_jumprelu_threshold_value=-1.0)
    m.set_decoder_to_fixed_norm(1.0, True)
    m.init_encoder_with_decoder_transpose()
    return m


def transcoder_stream(n, B=64, d=64, seed=5):
    g = torch.Generator().manual_seed(seed)
    basis, mix = torch.randn(10, d, generator=g), torch.randn(d, d, generator=g) / d**0.5
    for _ in range(n):
        x = torch.randn(B, 10, generator=g) @ basis + 0.05 * torch.randn(B, d, generator=g)
        x = x * (d**0.5 / x.norm(dim=-1).mean())
        yield {"pre": x, "post": torch.tanh(x @ mix) * 3, "tokens": torch.ones(B, dtype=torch.long)}


def test_jumprelu_transcoder_trains_on_the_fused_step_towards_its_own_target(crosscoder_on_cpu, tmp_path):
    """A JumpReLU dictionary that reads one hook point and reconstructs another: the fused step takes the other hook point's
    activations as targets and follows the generic run."""
    kw = dict(sparsity_loss_type="tanh", l1_coefficient=0.02, jumprelu_lr_factor=0.5)
    fused = jumprelu_transcoder()
    tr = trainer(tmp_path / "fused", 64 * 8, **kw)
    assert tr.fit(fused, transcoder_stream(9)) is None
    assert type(tr.fused).__name__ == "FusedCrosscoderStep" and tr.fused.single
    generic = jumprelu_transcoder()
    tg = trainer(tmp_path / "generic", 64 * 8, use_fused_kernels=False, amp_dtype=torch.float32, **kw)
    assert tg.fit(generic, transcoder_stream(9)) is None and tg.fused is None
    start = jumprelu_transcoder()
    for (name, p), (_, q), (_, p0) in zip(fused.named_parameters(), generic.named_parameters(), start.named_parameters()):
        moved = float((q - p0).abs().mean())
        assert float((p - q).abs().mean()) < 0.1 * moved + 1e-7, name
    # and it is the target that is being learned: the error against "post" fell from where the untrained model stands
    batch = next(transcoder_stream(1, seed=9))
    with torch.no_grad():
        err = [float((m.decode(m.encode(batch["pre"])) - batch["post"]).pow(2).mean()) for m in (start, fused)]
    assert err[1] < err[0]
