"""Every dictionary family trains through ``Trainer.fit`` (autograd path, bf16 autocast) on the GPU and on the CPU: a few steps on
synthetic activations, the loss must be finite and go down. The SAE cases also cover the fused-kernel path with the
Aux-K loss and a JumpReLU SAE (fused straight-through kernels)."""

import tempfile

import pytest
import torch

from language_model_saes_b200.models.clt import CLTConfig
from language_model_saes_b200.models.crosscoder import CrosscoderConfig
from language_model_saes_b200.models.lorsa import LorsaConfig
from language_model_saes_b200.models.molt import MOLTConfig
from language_model_saes_b200.models.sae import SAEConfig
from language_model_saes_b200.models.sparse_dictionary import SparseDictionary
from language_model_saes_b200.trainer import Trainer, TrainerConfig


D = 64
DEVICES = [pytest.param("cuda", marks=pytest.mark.gpu), "cpu"]


def _stream(keys, n, batch, dev, seq=None, seed=0):
    g = torch.Generator(device=dev).manual_seed(seed)
    basis = torch.randn(12, D, device=dev, generator=g)
    for _ in range(n):
        shape = (batch, 12) if seq is None else (batch, seq, 12)
        base = torch.randn(*shape, device=dev, generator=g) @ basis
        rec = {k: base + 0.05 * (i + 1) * torch.randn_like(base) for i, k in enumerate(keys)}
        rec = {k: v * (D**0.5 / v.norm(dim=-1).mean()) for k, v in rec.items()}
        rec["tokens"] = torch.ones(shape[:-1], dtype=torch.long, device=dev)
        yield rec


def _fit(cfg, keys, seq=None, steps=30, batch=256, **trainer_kw):
    torch.manual_seed(0)
    sae = SparseDictionary.from_config(cfg)
    sae.init_parameters(encoder_uniform_bound=0.1, decoder_uniform_bound=0.1, init_log_jumprelu_threshold_value=-2.0)
    if hasattr(sae, "set_dataset_average_activation_norm"):
        sae.set_dataset_average_activation_norm({k: D**0.5 for k in keys})
    tokens_per_step = batch * (seq or 1)
    losses = []
    with tempfile.TemporaryDirectory() as tmp:
        tcfg = TrainerConfig(total_training_tokens=steps * tokens_per_step, lr=2e-3, lr_warm_up_steps=2, log_frequency=10**6,
                             n_checkpoints=0, exp_result_path=tmp, skip_metrics_calculation=True, **trainer_kw)  # fmt: skip
        trainer = Trainer(tcfg)
        orig = trainer._generic_iteration

        def spy(*a, **kw):
            out = orig(*a, **kw)
            losses.append(float(out))
            return out

        trainer._generic_iteration = spy
        if trainer_kw.get("use_fused_kernels", True):
            orig_f = trainer._fused_iteration

            def spy_f(*a, **kw):
                out = orig_f(*a, **kw)
                losses.append(float(out))
                return out

            trainer._fused_iteration = spy_f
        trainer.fit(sae, _stream(keys, steps + 1, batch, cfg.device, seq))
    assert len(losses) == steps and all(torch.isfinite(torch.tensor(losses))), losses
    assert sum(losses[-5:]) < sum(losses[:5]), losses
    return sae, trainer


@pytest.mark.gpu
def test_sae_fused_with_auxk(dev="cuda"):
    cfg = SAEConfig(hook_point_in="h", hook_point_out="h", d_model=D, expansion_factor=32, act_fn="topk", top_k=8, device=dev, dtype=torch.float32)
    sae, trainer = _fit(cfg, ["h"], l1_coefficient=None, auxk_coefficient=1 / 32, k_aux=32, dead_threshold=2000)
    assert trainer.fused is not None and trainer.fused.last_aux_loss is not None
    assert trainer.tokens_since_last_activation is not None and int(trainer.tokens_since_last_activation.max()) > 0


@pytest.mark.gpu
@pytest.mark.parametrize("auxk", [None, 1 / 32])
def test_sae_fused_with_gradient_clipping(auxk, dev="cuda"):
    cfg = SAEConfig(hook_point_in="h", hook_point_out="h", d_model=D, expansion_factor=32, act_fn="topk", top_k=8, device=dev, dtype=torch.float32)
    sae, trainer = _fit(cfg, ["h"], l1_coefficient=None, clip_grad_norm=1e-5, auxk_coefficient=auxk, k_aux=32, dead_threshold=2000)
    assert trainer.fused is not None and float(trainer.fused.last_grad_norm) > 0


@pytest.mark.parametrize("dev", DEVICES)
def test_sae_jumprelu_autograd(dev):
    cfg = SAEConfig(hook_point_in="h", hook_point_out="h", d_model=D, expansion_factor=8, act_fn="jumprelu", device=dev, dtype=torch.float32)
    sae, _ = _fit(cfg, ["h"], l1_coefficient=1e-3, sparsity_loss_type="tanh", lp_coefficient=1e-3)
    assert float((sae.activation_function.log_jumprelu_threshold + 2.0).abs().max()) > 1e-3  # the thresholds were trained


@pytest.mark.parametrize("dev", DEVICES)
def test_batchtopk_transcoder(dev):
    cfg = SAEConfig(hook_point_in="a", hook_point_out="b", d_model=D, expansion_factor=8, act_fn="batchtopk", top_k=8, device=dev, dtype=torch.float32)
    _fit(cfg, ["a", "b"], l1_coefficient=None)


@pytest.mark.parametrize("dev", DEVICES)
def test_crosscoder(dev):
    cfg = CrosscoderConfig(hook_points=["s0", "s1", "s2"], d_model=D, expansion_factor=8, act_fn="topk", top_k=8, device=dev, dtype=torch.float32)
    _fit(cfg, ["s0", "s1", "s2"], l1_coefficient=None)


@pytest.mark.parametrize("dev", DEVICES)
def test_clt(dev):
    ins, outs = [f"blocks.{i}.ln2.hook_normalized" for i in range(3)], [f"blocks.{i}.hook_mlp_out" for i in range(3)]
    cfg = CLTConfig(hook_points_in=ins, hook_points_out=outs, d_model=D, expansion_factor=4, act_fn="topk", top_k=8, device=dev, dtype=torch.float32)
    _fit(cfg, ins + outs, l1_coefficient=None)


@pytest.mark.parametrize("dev", DEVICES)
def test_lorsa(dev):
    cfg = LorsaConfig(hook_point_in="x", hook_point_out="y", d_model=D, expansion_factor=4, n_qk_heads=8, d_qk_head=16, rotary_dim=16, n_ctx=32,
                      act_fn="topk", top_k=8, device=dev, dtype=torch.float32)  # fmt: skip
    _fit(cfg, ["x", "y"], seq=16, batch=32, l1_coefficient=None)


@pytest.mark.parametrize("dev", DEVICES)
def test_molt(dev):
    cfg = MOLTConfig(hook_point_in="a", hook_point_out="b", d_model=D, expansion_factor=2, rank_counts={2: 64, 4: 64}, act_fn="relu",
                     device=dev, dtype=torch.float32)  # fmt: skip
    _fit(cfg, ["a", "b"], l1_coefficient=1e-4, sparsity_loss_type="tanh")
