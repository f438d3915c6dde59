"""Hook points: named identity modules whose inputs can be observed or replaced.

The reference project builds its dictionaries on ``transformer_lens.hook_points.HookedRootModule``
(models/sparse_dictionary.py:32,217 there). This is an independent, dependency-free equivalent with the
part of that interface the framework uses: ``HookPoint`` (forward and backward hooks, an ``hook(tensor, hook=)``
signature), ``HookedRootModule.setup()``, ``hook_dict``, ``hooks(...)`` context manager,
``run_with_hooks``, ``run_with_cache`` and ``reset_hooks``.
"""

from __future__ import annotations

from contextlib import contextmanager
from typing import Any, Callable, Iterable, Sequence

import torch
from torch import nn

HookFn = Callable[..., Any]
NameFilter = str | Sequence[str] | Callable[[str], bool] | None


class HookPoint(nn.Module):
    """Identity module. Forward hooks receive ``(tensor, hook=self)`` and may return a replacement."""

    def __init__(self):
        super().__init__()
        self.name: str | None = None
        self.fwd_hooks: list[tuple[HookFn, bool]] = []  # (fn, is_permanent)
        self.bwd_hooks: list[tuple[HookFn, bool]] = []
        self.ctx: dict[str, Any] = {}

    def add_hook(self, hook: HookFn, dir: str = "fwd", is_permanent: bool = False, prepend: bool = False) -> None:
        target = self.fwd_hooks if dir == "fwd" else self.bwd_hooks
        if dir not in ("fwd", "bwd"):
            raise ValueError(f"Invalid direction {dir}")
        if prepend:
            target.insert(0, (hook, is_permanent))
        else:
            target.append((hook, is_permanent))

    def add_perma_hook(self, hook: HookFn, dir: str = "fwd") -> None:
        self.add_hook(hook, dir=dir, is_permanent=True)

    def remove_hooks(self, dir: str = "both", including_permanent: bool = False) -> None:
        def keep(hs):
            return [h for h in hs if h[1] and not including_permanent]

        if dir in ("fwd", "both"):
            self.fwd_hooks = keep(self.fwd_hooks)
        if dir in ("bwd", "both"):
            self.bwd_hooks = keep(self.bwd_hooks)

    def clear_context(self) -> None:
        self.ctx = {}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        for fn, _ in self.fwd_hooks:
            out = fn(x, hook=self)
            if out is not None:
                x = out
        if self.bwd_hooks and isinstance(x, torch.Tensor) and x.requires_grad:
            hooks = list(self.bwd_hooks)

            def _bwd(grad, hooks=hooks):
                for fn, _ in hooks:
                    out = fn(grad, hook=self)
                    if out is not None:
                        grad = out
                return grad

            x = x.view_as(x)
            x.register_hook(_bwd)
        return x

    def layer(self) -> int:
        """Layer index parsed from a name like ``blocks.3.hook_resid_post``."""
        assert self.name is not None
        return int(self.name.split(".")[1])


class HookedRootModule(nn.Module):
    """A module whose ``HookPoint`` descendants are addressable by their dotted name."""

    def __init__(self, *args, **kwargs):
        super().__init__()
        self.is_caching = False
        self.hook_dict: dict[str, HookPoint] = {}
        self.mod_dict: dict[str, nn.Module] = {}

    def setup(self) -> None:
        """Index sub-modules; call at the end of ``__init__`` (and again after adding hook points)."""
        self.mod_dict = {}
        self.hook_dict = {}
        for name, module in self.named_modules():
            if name == "":
                continue
            self.mod_dict[name] = module
            if isinstance(module, HookPoint):
                module.name = name
                self.hook_dict[name] = module

    def hook_points(self) -> Iterable[HookPoint]:
        return self.hook_dict.values()

    def reset_hooks(self, clear_contexts: bool = True, direction: str = "both", including_permanent: bool = False):
        for hp in self.hook_points():
            hp.remove_hooks(direction, including_permanent=including_permanent)
            if clear_contexts:
                hp.clear_context()
        self.is_caching = False

    def _match(self, names: NameFilter) -> list[str]:
        if names is None:
            return list(self.hook_dict)
        if isinstance(names, str):
            return [names] if names in self.hook_dict else []
        if callable(names):
            return [n for n in self.hook_dict if names(n)]
        return [n for n in names if n in self.hook_dict]

    def add_hook(self, name: NameFilter, hook: HookFn, dir: str = "fwd", is_permanent: bool = False, prepend: bool = False):
        if isinstance(name, str) and name not in self.hook_dict:
            raise KeyError(f"No hook point named {name!r}")
        for n in self._match(name):
            self.hook_dict[n].add_hook(hook, dir=dir, is_permanent=is_permanent, prepend=prepend)

    @contextmanager
    def hooks(
        self,
        fwd_hooks: Sequence[tuple[NameFilter, HookFn]] = (),
        bwd_hooks: Sequence[tuple[NameFilter, HookFn]] = (),
        reset_hooks_end: bool = True,
        clear_contexts: bool = False,
    ):
        try:
            for name, fn in fwd_hooks:
                self.add_hook(name, fn, dir="fwd")
            for name, fn in bwd_hooks:
                self.add_hook(name, fn, dir="bwd")
            yield self
        finally:
            if reset_hooks_end:
                self.reset_hooks(clear_contexts, including_permanent=False)

    def run_with_hooks(self, *args, fwd_hooks=(), bwd_hooks=(), reset_hooks_end=True, clear_contexts=False, **kwargs):
        with self.hooks(fwd_hooks, bwd_hooks, reset_hooks_end, clear_contexts):
            return self(*args, **kwargs)

    def get_caching_hooks(self, names_filter: NameFilter = None, incl_bwd: bool = False, cache: dict | None = None):
        cache = {} if cache is None else cache

        def save(tensor, hook):
            cache[hook.name] = tensor.detach()

        def save_bwd(tensor, hook):
            cache[hook.name + "_grad"] = tensor.detach()

        names = self._match(names_filter)
        fwd = [(n, save) for n in names]
        bwd = [(n, save_bwd) for n in names] if incl_bwd else []
        return cache, fwd, bwd

    def run_with_cache(self, *args, names_filter: NameFilter = None, incl_bwd: bool = False, **kwargs):
        cache, fwd, bwd = self.get_caching_hooks(names_filter, incl_bwd)
        with self.hooks(fwd, bwd):
            out = self(*args, **kwargs)
            if incl_bwd:
                out.backward()
        return out, cache
