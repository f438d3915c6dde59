"""Schedules of the trainer that the other tests leave at their defaults: the k schedule (cold boot, linear and exponential
decay towards ``top_k``), the warm-up of the sparsity coefficient, gradient accumulation, and the sparse Adam optimizer
(trainer.py:457-491 of the reference project for the schedules)."""

import math

import pytest
import torch

from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
from language_model_saes_b200.trainer import Trainer, TrainerConfig

D, F = 16, 64


def _sae(act_fn="topk", **kw):
    torch.manual_seed(0)
    sae = SparseAutoEncoder(SAEConfig(hook_point_in="h", hook_point_out="h", d_model=D, expansion_factor=F // D, act_fn=act_fn, top_k=4,
                                      norm_activation="inference", device="cpu", dtype=torch.float32, **kw))  # fmt: skip
    sae.init_parameters(encoder_uniform_bound=0.3, decoder_uniform_bound=0.3)
    return sae


def _stream(n, rows=32, seed=1):
    g = torch.Generator().manual_seed(seed)
    for _ in range(n):
        yield {"h": torch.randn(rows, D, generator=g), "tokens": torch.ones(rows, dtype=torch.long)}


def _cfg(tmp_path, **kw):
    base = dict(lr=1e-2, total_training_tokens=32 * 20, log_frequency=1000, eval_frequency=10**6, n_checkpoints=0, lr_warm_up_steps=0,
                lr_scheduler_name="constant", exp_result_path=str(tmp_path), amp_dtype=torch.float32, l1_coefficient=None, use_fused_kernels=False)  # fmt: skip
    return TrainerConfig(**(base | kw))


@pytest.mark.parametrize("kind", ["linear", "exponential"])
def test_k_schedule_boots_cold_then_decays_to_top_k(tmp_path, kind):
    sae = _sae()
    t = Trainer(_cfg(tmp_path, initial_k=20, k_warmup_steps=10, k_cold_booting_steps=3, k_schedule_type=kind, k_exponential_factor=2.0))
    t._initialize_trainer(sae, next(_stream(1)))
    assert (t.total_training_steps, t.k_warmup_steps, t.k_cold_booting_steps) == (20, 10, 3)
    seen = []
    for step in range(20):
        t.cur_step = step
        seen.append(t._current_k(sae))
    assert seen[:3] == [20, 20, 20] and seen[3] == 20  # the decay starts where the cold boot ends
    assert seen[13:] == [4] * 7
    assert all(a >= b for a, b in zip(seen, seen[1:]))
    for step in range(3, 13):
        p = (step - 3) / 10
        if kind == "exponential":
            p = (1 - math.exp(-2.0 * p)) / (1 - math.exp(-2.0))
        assert seen[step] == max(4, math.ceil(20 + (4 - 20) * p))
    if kind == "exponential":  # faster at first than the straight line
        lin = [max(4, math.ceil(20 - 16 * (s - 3) / 10)) for s in range(3, 13)]
        assert all(e <= l for e, l in zip(seen[3:13], lin)) and seen[6] < lin[3]
    # fractions are shares of the run; no initial k means a constant k
    t2 = Trainer(_cfg(tmp_path, initial_k=8, k_warmup_steps=0.5, k_cold_booting_steps=0.1))
    t2._initialize_trainer(sae, next(_stream(1)))
    assert (t2.k_warmup_steps, t2.k_cold_booting_steps) == (10, 2)
    t3 = Trainer(_cfg(tmp_path))
    t3._initialize_trainer(sae, next(_stream(1)))
    assert t3._current_k(sae) is None
    t4 = Trainer(_cfg(tmp_path, initial_k=2, k_warmup_steps=5))
    t4._initialize_trainer(sae, next(_stream(1)))
    with pytest.raises(AssertionError, match="initial_k"):
        t4._current_k(sae)


def test_k_schedule_drives_the_number_of_active_features_during_fit(tmp_path):
    sae = _sae()
    seen = []
    real = sae.set_current_k
    sae.set_current_k = lambda k: (seen.append(k), real(k))[1]
    Trainer(_cfg(tmp_path, initial_k=12, k_warmup_steps=4, total_training_tokens=32 * 8)).fit(sae, _stream(10))
    assert seen[:5] == [12, 10, 8, 6, 4] and set(seen[5:]) == {4}
    assert sae.current_k == 4


def test_sparsity_coefficient_warms_up_linearly(tmp_path):
    sae = _sae("relu")
    t = Trainer(_cfg(tmp_path, l1_coefficient=0.5, l1_coefficient_warmup_steps=0.25, sparsity_loss_type="power"))
    t._initialize_trainer(sae, next(_stream(1)))
    assert t.l1_coefficient_warmup_steps == 5
    got = []
    for step in range(8):
        t.cur_step = step
        got.append(t._l1_coefficient())
    assert got == pytest.approx([0.0, 0.1, 0.2, 0.3, 0.4, 0.5, 0.5, 0.5])
    t0 = Trainer(_cfg(tmp_path, l1_coefficient=0.5, l1_coefficient_warmup_steps=0))
    t0._initialize_trainer(sae, next(_stream(1)))
    assert t0._l1_coefficient() == 0.5
    tn = Trainer(_cfg(tmp_path, l1_coefficient=None))
    tn._initialize_trainer(sae, next(_stream(1)))
    assert tn._l1_coefficient() == 1.0  # models without a sparsity penalty see a neutral factor


def test_two_accumulated_half_batches_step_like_one_whole_batch(tmp_path):
    """With a mean loss, the average of the gradients of two half batches is the gradient of the whole batch; the optimizer
    steps once per two iterations."""
    whole, halves = _sae("relu"), _sae("relu")
    g = torch.Generator().manual_seed(3)
    batches = [torch.randn(32, D, generator=g) for _ in range(3)]
    common = dict(l1_coefficient=1e-3, sparsity_loss_type="power", skip_metrics_calculation=True)
    Trainer(_cfg(tmp_path, total_training_tokens=32 * 3, **common)).fit(
        whole, iter({"h": b, "tokens": torch.ones(32, dtype=torch.long)} for b in batches))
    Trainer(_cfg(tmp_path, total_training_tokens=16 * 6, gradient_accumulation_steps=2, **common)).fit(
        halves, iter({"h": h, "tokens": torch.ones(16, dtype=torch.long)} for b in batches for h in (b[:16], b[16:])))
    for (n, a), (_, b) in zip(whole.named_parameters(), halves.named_parameters()):
        assert torch.allclose(a, b, atol=2e-5), n


def test_sparse_adam_moves_only_what_received_a_gradient(tmp_path):
    sae = _sae()
    before = {n: p.detach().clone() for n, p in sae.named_parameters()}
    t = Trainer(_cfg(tmp_path, optimizer_class="sparseadam", total_training_tokens=8))  # one step of 8 rows: at most 32 features fire
    t.fit(sae, _stream(2, rows=8))
    assert type(t.optimizer).__name__ == "SparseAdam"
    moved = (sae.W_D.detach() - before["W_D"]).abs().sum(-1) > 0
    assert 0 < int(moved.sum()) <= 32  # decoder rows of features that did not fire keep their values
    assert all(torch.isfinite(p).all() for p in sae.parameters())


@pytest.mark.parametrize("mode,want", [("linear", [5, 10, 15]), ("log", [3, 5, 10])])
def test_model_snapshots_are_taken_at_linear_or_log_spaced_steps(tmp_path, mode, want):
    from safetensors.torch import load_file

    sae = _sae("relu")
    t = Trainer(_cfg(tmp_path, n_checkpoints=4, check_point_save_mode=mode, skip_metrics_calculation=True))
    t.fit(sae, _stream(22))
    files = sorted(int(p.stem) for p in (tmp_path / "checkpoints").glob("*.safetensors"))
    assert files == want and t.checkpoint_thresholds == []
    last = load_file(tmp_path / "checkpoints" / f"{want[-1]}.safetensors")
    assert set(last) >= {"W_E", "W_D", "b_E", "b_D"} and not torch.equal(last["W_D"], sae.W_D.detach())  # training went on after it
    # fewer steps than snapshots: every step at most once
    short = Trainer(_cfg(tmp_path / "short", n_checkpoints=8, check_point_save_mode=mode, total_training_tokens=32 * 3))
    short._initialize_trainer(sae, next(_stream(1)))
    assert short.checkpoint_thresholds == sorted(set(short.checkpoint_thresholds)) and all(0 < s <= 3 for s in short.checkpoint_thresholds)
