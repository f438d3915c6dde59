"""Numerical parity with the reference project itself: identical parameters and batches go through the reference's own
``compute_loss`` (installed copy under ``baseline/_ref``, run in a child process so that its package name cannot collide
with this repository's alias packages) and through this package's; losses, codes, reconstructions and parameter
gradients must agree. Cases follow tests/unit/test_sae.py:58-239 and tests/unit/test_crosscoder.py:120-476 of the
reference project (loss pieces per activation function and family) on tiny fp32 CPU shapes. Skipped when the reference
is not installed."""

import os
import subprocess
import sys
import tempfile
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
REF = ROOT / "baseline" / "_ref"
pytestmark = pytest.mark.skipif(not (REF / "llamascopium").is_dir(), reason="the reference project is not installed under baseline/_ref")

D = 32


def _run_reference(jobs: dict, gpu: bool = False) -> dict:
    with tempfile.TemporaryDirectory() as tmp:
        inp, out = os.path.join(tmp, "in.pt"), os.path.join(tmp, "out.pt")
        torch.save(jobs, inp)
        env = dict(os.environ, PYTHONPATH=os.pathsep.join([str(ROOT / "baseline" / "_stubs"), str(REF)]))
        if not gpu:
            env["CUDA_VISIBLE_DEVICES"] = ""
        r = subprocess.run([sys.executable, str(Path(__file__).with_name("reference_side.py")), inp, out], env=env, cwd=tmp,
                           capture_output=True, text=True, timeout=1200)  # fmt: skip
        assert r.returncode == 0, r.stderr[-3000:]
        return torch.load(out, weights_only=False)


def _ours(config_class: str, config: dict, state: dict, batch: dict, loss_kwargs: dict, norm: dict | None):
    import language_model_saes_b200 as lm
    from language_model_saes_b200.models.sparse_dictionary import SparseDictionary

    kw = dict(config)
    kw["dtype"] = getattr(torch, kw["dtype"])
    model = SparseDictionary.from_config(getattr(lm, config_class)(**kw))
    model.load_state_dict(state, strict=False)
    if norm:
        model.set_dataset_average_activation_norm(norm)
    b = model.normalize_activations(dict(batch))
    extra = dict(loss_kwargs)
    if extra.get("auxk_coefficient", 0.0) > 0.0:
        extra["update_dead_statistics"] = lambda fa, mask, specs: ~(fa.reshape(-1, fa.shape[-1]).sum(0) > 0)
    res = model.compute_loss(b, return_aux_data=True, **extra)
    res["loss"].backward()
    return model, res


def _fresh_state(config_class: str, config: dict, seed: int = 0) -> dict:
    import language_model_saes_b200 as lm
    from language_model_saes_b200.models.sparse_dictionary import SparseDictionary

    torch.manual_seed(seed)
    kw = dict(config)
    kw["dtype"] = getattr(torch, kw["dtype"])
    model = SparseDictionary.from_config(getattr(lm, config_class)(**kw))
    model.init_parameters(encoder_uniform_bound=0.3, decoder_uniform_bound=0.3, init_log_jumprelu_threshold_value=-1.0)
    with torch.no_grad():
        for n, p in model.named_parameters():  # biases start at zero: give every parameter a gradient worth comparing
            if p.ndim <= 2 and "b_" in n:
                p.add_(0.05 * torch.randn_like(p))
    return {k: v.detach().clone().contiguous() for k, v in model.state_dict().items()}


def _batch(keys, shape, seed=1):
    g = torch.Generator().manual_seed(seed)
    out = {k: torch.randn(*shape, D, generator=g) * (1 + 0.1 * i) for i, k in enumerate(keys)}
    out["tokens"] = torch.ones(*shape, dtype=torch.long)
    return out


CASES: dict[str, dict] = {}


def _case(name, config_class, config, keys, shape, loss_kwargs=None, atol=2e-5, mask=None):
    state = _fresh_state(config_class, config)
    batch = _batch(keys, shape)
    if mask is not None:
        batch["mask"] = mask
    CASES[name] = {"config_class": config_class, "config": config, "state": state, "batch": batch, "loss_kwargs": loss_kwargs or {},
                   "norm": {k: float(D**0.5) for k in keys}, "atol": atol}  # fmt: skip


SAE = dict(hook_point_in="a", hook_point_out="a", d_model=D, expansion_factor=4, device="cpu", dtype="float32")
_case("sae-topk", "SAEConfig", {**SAE, "act_fn": "topk", "top_k": 6}, ["a"], (48,))
_case("sae-topk-no-norm-gate", "SAEConfig", {**SAE, "act_fn": "topk", "top_k": 6, "sparsity_include_decoder_norm": False}, ["a"], (48,))
_case("sae-topk-auxk", "SAEConfig", {**SAE, "act_fn": "topk", "top_k": 6}, ["a"], (48,), dict(auxk_coefficient=1 / 32, k_aux=16))
_case("sae-batchtopk", "SAEConfig", {**SAE, "act_fn": "batchtopk", "top_k": 6}, ["a"], (48,))
_case("sae-relu-power", "SAEConfig", {**SAE, "act_fn": "relu"}, ["a"], (48,), dict(sparsity_loss_type="power", l1_coefficient=3e-3))
_case("sae-relu-tanh", "SAEConfig", {**SAE, "act_fn": "relu"}, ["a"], (48,), dict(sparsity_loss_type="tanh", l1_coefficient=3e-3))
_case("sae-jumprelu-tanh-lp", "SAEConfig", {**SAE, "act_fn": "jumprelu"}, ["a"], (48,),
      dict(sparsity_loss_type="tanh", l1_coefficient=3e-3, lp_coefficient=1e-2))  # fmt: skip
_case("transcoder-masked", "SAEConfig", {**SAE, "hook_point_out": "b", "act_fn": "topk", "top_k": 6}, ["a", "b"], (48,),
      mask=torch.rand(48, generator=torch.Generator().manual_seed(5)) > 0.3)  # fmt: skip
_CC = dict(hook_points=["s0", "s1", "s2"], d_model=D, expansion_factor=4, device="cpu", dtype="float32")
_case("crosscoder-topk", "CrosscoderConfig", {**_CC, "act_fn": "topk", "top_k": 6}, ["s0", "s1", "s2"], (40,))
_case("crosscoder-jumprelu", "CrosscoderConfig", {**_CC, "act_fn": "jumprelu"}, ["s0", "s1", "s2"], (40,),
      dict(sparsity_loss_type="tanh", l1_coefficient=3e-3))  # fmt: skip
_INS, _OUTS = [f"blocks.{i}.ln2.hook_normalized" for i in range(3)], [f"blocks.{i}.hook_mlp_out" for i in range(3)]
_case("clt-topk", "CLTConfig", dict(hook_points_in=_INS, hook_points_out=_OUTS, d_model=D, expansion_factor=2, act_fn="topk", top_k=6,
                                    device="cpu", dtype="float32"), _INS + _OUTS, (40,))  # fmt: skip
_case("lorsa-topk", "LorsaConfig", dict(hook_point_in="x", hook_point_out="y", d_model=D, expansion_factor=4, n_qk_heads=8, d_qk_head=8,
                                        rotary_dim=8, n_ctx=16, act_fn="topk", top_k=6, device="cpu", dtype="float32"),
      ["x", "y"], (4, 12), atol=5e-5)  # fmt: skip
_case("molt-relu-tanh", "MOLTConfig", dict(hook_point_in="a", hook_point_out="b", d_model=D, expansion_factor=2, rank_counts={2: 32, 4: 32},
                                           act_fn="relu", device="cpu", dtype="float32"),
      ["a", "b"], (40,), dict(sparsity_loss_type="tanh", l1_coefficient=1e-3))  # fmt: skip


@pytest.fixture(scope="module")
def reference_results():
    """Every case through the reference in ONE child process (its import alone takes tens of seconds)."""
    return _run_reference({n: {k: v for k, v in c.items() if k != "atol"} for n, c in CASES.items()})


@pytest.mark.parametrize("name", list(CASES))
def test_losses_codes_and_gradients_match_the_reference(name, reference_results):
    case, ref = CASES[name], reference_results[name]
    assert "error" not in ref, ref.get("error")
    atol = case["atol"]
    model, res = _ours(case["config_class"], case["config"], case["state"], case["batch"], case["loss_kwargs"], case["norm"])
    assert torch.allclose(res["loss"].detach(), ref["loss"], atol=atol, rtol=1e-4), (res["loss"], ref["loss"])
    for key in ("l_rec", "l_s", "l_p", "l_aux"):
        if key in ref:
            assert res.get(key) is not None, key
            assert torch.allclose(res[key].detach().float(), ref[key].float(), atol=atol, rtol=1e-4), key
    fa, fb = res["feature_acts"].detach(), ref["feature_acts"]
    fa = fa.to_dense() if fa.layout != torch.strided else fa
    fb = fb.to_dense() if fb.layout != torch.strided else fb
    assert torch.equal(fa != 0, fb != 0), "the supports of the codes differ"
    assert torch.allclose(fa, fb, atol=atol, rtol=1e-4)
    assert torch.allclose(res["reconstructed"].detach(), ref["reconstructed"], atol=10 * atol, rtol=1e-4)
    ours = {n: p.grad for n, p in model.named_parameters() if p.grad is not None}
    assert set(ours) == set(ref["grads"]), (sorted(ours), sorted(ref["grads"]))
    for n, g in ref["grads"].items():
        assert torch.allclose(ours[n], g, atol=atol, rtol=1e-3), (n, float((ours[n] - g).abs().max()))


@pytest.mark.gpu
def test_five_fused_steps_follow_five_steps_of_the_reference_trainer():
    """The same TopK SAE, batches and hyper-parameters through the reference's ``Trainer.fit`` (its autograd path under bf16
    autocast, torch Adam) and through this package's ``Trainer.fit`` on the fused kernel path: after five steps every
    parameter has moved the same way (the difference is a small fraction of the movement itself)."""
    from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder
    from language_model_saes_b200.trainer import Trainer, TrainerConfig

    d, F, k, B, steps = 64, 2048, 8, 512, 5
    config = dict(hook_point_in="h", hook_point_out="h", d_model=d, expansion_factor=F / d, act_fn="topk", top_k=k, device="cuda", dtype="float32")
    torch.manual_seed(0)
    sae = SparseAutoEncoder(SAEConfig(**{**config, "dtype": torch.float32}))
    sae.init_parameters(encoder_uniform_bound=0.1, decoder_uniform_bound=0.1)
    sae.set_decoder_to_fixed_norm(1.0, True)
    sae.init_encoder_with_decoder_transpose()
    norm = {"h": float(d**0.5)}
    sae.set_dataset_average_activation_norm(norm)
    start = {k_: v.detach().cpu().clone().contiguous() for k_, v in sae.state_dict().items()}
    g = torch.Generator().manual_seed(3)
    basis = torch.randn(10, d, generator=g)
    batches = []
    for _ in range(steps):
        x = torch.randn(B, 10, generator=g) @ basis + 0.1 * torch.randn(B, d, generator=g)
        x = (x * (d**0.5 / x.norm(dim=-1).mean())).to(torch.bfloat16).float()  # bf16-exact values: both sides see the same numbers
        batches.append({"h": x, "tokens": torch.zeros(B, dtype=torch.long), "mask": torch.ones(B, dtype=torch.bool)})
    trainer_kw = dict(total_training_tokens=steps * B, lr=1e-3, lr_scheduler_name="constant", log_frequency=10**6, n_checkpoints=0,
                      skip_metrics_calculation=True, k_warmup_steps=0, l1_coefficient=None)  # fmt: skip
    ref = _run_reference({"train": {"kind": "train", "config_class": "SAEConfig", "config": config, "state": start, "norm": norm,
                                    "batches": batches, "trainer": trainer_kw}}, gpu=True)["train"]  # fmt: skip
    assert "error" not in ref, ref.get("error")
    with tempfile.TemporaryDirectory() as tmp:
        tr = Trainer(TrainerConfig(exp_result_path=tmp, lr_warm_up_steps=0, lr_cool_down_steps=0, **trainer_kw))
        tr.fit(sae, iter([{k_: v.cuda() for k_, v in b.items()} for b in batches]))
        assert tr.fused is not None
    for name, after_ref in ref["state"].items():
        if name not in start or not after_ref.is_floating_point():
            continue
        ours = sae.state_dict()[name].detach().cpu().float()
        moved = (after_ref.float() - start[name].float()).abs().mean()
        if float(moved) == 0.0:
            continue
        assert float((ours - after_ref.float()).abs().mean()) < 0.3 * float(moved), name
