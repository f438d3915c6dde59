"""Context managers that rewire a hooked transformer for attribution (circuits/hooks.py:21-281 of the reference
project):

* ``apply_saes``: splice dictionaries into the forward pass: encode at ``hook_point_in``, replace the activation at
  ``hook_point_out`` by ``decode(features) + error`` where the error term passes through its own hook point, so that
  features and errors are separate graph nodes. The dictionary is mounted at ``<hook_point_out>.sae`` and the error
  hook at ``<hook_point_out>.error``.
* ``detach_at``: cut the autograd graph at hook points, exposing ``<hook>.pre`` (upstream side) and ``<hook>.post``
  (a fresh leaf on the downstream side).
* ``replace_model_biases_with_leaves`` / ``replace_sae_biases_with_leaves``: zero bias parameters and add them back
  as per-position leaf tensors behind a hook point, which makes every bias an attributable source node.
"""

from __future__ import annotations

from contextlib import contextmanager
from typing import Callable, NamedTuple

import torch
import torch.nn as nn

from ..backend.hooked_transformer import HookedTransformer
from ..hooks import HookPoint
from ..models.lorsa import LowRankSparseAttention
from ..models.molt import MixtureOfLinearTransform
from ..models.sae import SparseAutoEncoder
from ..models.sparse_dictionary import SparseDictionary
from ..utils.timer import timer

_SPLICEABLE = (SparseAutoEncoder, LowRankSparseAttention, MixtureOfLinearTransform)


def _splice_hooks(sae) -> tuple[list[tuple[str, Callable]], HookPoint]:
    state: dict[str, torch.Tensor | None] = {"acts": None}
    error_hook = HookPoint()
    kwargs = {"hook_attn_scores": True} if isinstance(sae, LowRankSparseAttention) else {}

    @timer.time(f"hook_in_{sae.cfg.sae_type}")
    def hook_in(tensor: torch.Tensor, hook: HookPoint):
        # the input hook can fire several times per pass (a shared layer norm feeding Q, K and V): encode once
        if state["acts"] is None:
            state["acts"] = sae.encode(tensor, **kwargs)
            if isinstance(sae, MixtureOfLinearTransform):
                state["x"] = tensor
        return tensor

    @timer.time(f"hook_out_{sae.cfg.sae_type}")
    def hook_out(tensor: torch.Tensor, hook: HookPoint):
        assert state["acts"] is not None, "hook_in must be called before hook_out."
        extra = {"x": state.pop("x")} if isinstance(sae, MixtureOfLinearTransform) else {}
        reconstructed = sae.decode(state["acts"], **extra)
        state["acts"] = None
        return reconstructed + error_hook(tensor - reconstructed)

    return [(sae.cfg.hook_point_in, hook_in), (sae.cfg.hook_point_out, hook_out)], error_hook


@contextmanager
def apply_saes(model: HookedTransformer, saes: list[SparseDictionary]):
    assert all(isinstance(s, _SPLICEABLE) for s in saes), (
        "Currently only support sparse dictionaries that guarantee the hook points in happen before the hook points out."
    )
    fwd_hooks: list[tuple[str, Callable]] = []
    mounts: list[tuple[str, str, nn.Module]] = []
    for sae in saes:
        hooks, error_hook = _splice_hooks(sae)
        fwd_hooks.extend(hooks)
        mounts.append((sae.cfg.hook_point_out, "sae", sae))
        mounts.append((sae.cfg.hook_point_out, "error", error_hook))
    with model.mount_hooked_modules(mounts):
        with model.hooks(fwd_hooks=fwd_hooks):
            yield model


@contextmanager
def detach_at(model: HookedTransformer, hook_points: list[str]):
    mounts, fwd_hooks = [], []
    for name in hook_points:
        pre, post = HookPoint(), HookPoint()

        def cut(tensor: torch.Tensor, hook: HookPoint, pre=pre, post=post):
            return post(pre(tensor).detach().requires_grad_())

        mounts += [(name, "pre", pre), (name, "post", post)]
        fwd_hooks.append((name, cut))
    with model.mount_hooked_modules(mounts):
        with model.hooks(fwd_hooks=fwd_hooks):
            yield model


class _BiasReplacer(NamedTuple):
    mount: tuple[str, str, nn.Module]
    fwd_hook: tuple[str, Callable]
    cache_name: str
    restore: Callable[[], None]


def _make_bias_replacer(parent: nn.Module, parent_path: str, bias_attr: str, intercept: str, batch_size: int, seq_len: int) -> _BiasReplacer | None:
    param = getattr(parent, bias_attr, None)
    if param is None:
        return None
    original = param.data.clone()
    leaf = param.data.detach()[None, None].expand(batch_size, seq_len, *param.shape).clone().requires_grad_(True)
    param.data.zero_()
    bias_hook = HookPoint()
    child = f"hook_{bias_attr}"
    return _BiasReplacer(
        mount=(parent_path, child, bias_hook),
        fwd_hook=(intercept, lambda tensor, hook=None, **_: tensor + bias_hook(leaf)),
        cache_name=f"{parent_path}.{child}",
        restore=lambda: getattr(parent, bias_attr).data.copy_(original),
    )


@contextmanager
def _bias_phase(model: HookedTransformer, replacers: list[_BiasReplacer | None]):
    active = [r for r in replacers if r is not None]
    if not active:
        yield []
        return
    try:
        with model.mount_hooked_modules([r.mount for r in active]):
            with model.hooks(fwd_hooks=[r.fwd_hook for r in active]):
                yield [r.cache_name for r in active]
    finally:
        for r in active:
            r.restore()


@contextmanager
def replace_model_biases_with_leaves(model: HookedTransformer, batch_size: int, seq_len: int, device_mesh=None):
    """``attn.b_O`` -> ``blocks.{i}.attn.hook_b_O`` (added back at ``blocks.{i}.hook_attn_out``), ``mlp.b_out`` ->
    ``blocks.{i}.mlp.hook_b_out`` (at ``blocks.{i}.hook_mlp_out``). Enter BEFORE ``apply_saes`` so that a transcoder
    writing to the same hook point sees the bias already restored. Yields the mounted hook names."""
    reps: list[_BiasReplacer | None] = []
    for i, block in enumerate(model.blocks):
        reps.append(_make_bias_replacer(block.attn, f"blocks.{i}.attn", "b_O", f"blocks.{i}.hook_attn_out", batch_size, seq_len))
        reps.append(_make_bias_replacer(block.mlp, f"blocks.{i}.mlp", "b_out", f"blocks.{i}.hook_mlp_out", batch_size, seq_len))
    with _bias_phase(model, reps) as names:
        yield names


@contextmanager
def replace_sae_biases_with_leaves(model: HookedTransformer, saes: list[SparseDictionary], batch_size: int, seq_len: int, device_mesh=None):
    """``b_D`` -> ``<hook_point_out>.sae.hook_b_D`` (added back at the dictionary's ``hook_reconstructed``); for
    attention dictionaries also ``b_Q`` / ``b_K`` at ``hook_q`` / ``hook_k``. Enter AFTER ``apply_saes`` (the
    dictionaries must already be mounted)."""
    reps: list[_BiasReplacer | None] = []
    for sae in saes:
        if not isinstance(sae, _SPLICEABLE):
            continue
        path = f"{sae.cfg.hook_point_out}.sae"
        if isinstance(sae, LowRankSparseAttention):
            reps.append(_make_bias_replacer(sae, path, "b_Q", f"{path}.hook_q", batch_size, seq_len))
            reps.append(_make_bias_replacer(sae, path, "b_K", f"{path}.hook_k", batch_size, seq_len))
        if sae.cfg.use_decoder_bias:
            reps.append(_make_bias_replacer(sae, path, "b_D", f"{path}.hook_reconstructed", batch_size, seq_len))
    with _bias_phase(model, reps) as names:
        yield names
