"""Dataclass pytrees: map a function over every tensor held (directly or in nested containers / nested pytrees)
by a dataclass instance and rebuild an instance of the same class.

Same role as core/pytree.py of the reference project (:44-86), implemented on ``dataclasses`` introspection
instead of cattrs.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Callable, Self

import torch
from torch import Tensor


def _map(x: Any, fn_tensor: Callable[[Tensor], Any] | None, fn_any: Callable[[Any], Any] | None) -> Any:
    if isinstance(x, PyTree):
        return fn_any(x) if fn_any is not None else x.tree_map_tensor(fn_tensor)  # type: ignore[arg-type]
    if isinstance(x, Tensor):
        return fn_any(x) if fn_any is not None else fn_tensor(x)  # type: ignore[misc]
    if isinstance(x, dict):
        return {k: _map(v, fn_tensor, fn_any) for k, v in x.items()}
    if isinstance(x, tuple) and hasattr(x, "_fields"):
        return type(x)(*(_map(v, fn_tensor, fn_any) for v in x))
    if isinstance(x, (list, tuple)):
        return type(x)(_map(v, fn_tensor, fn_any) for v in x)
    return x


class PyTree:
    """Mixin for ``@dataclass`` classes."""

    def __to_pytree__(self) -> dict[str, Any]:
        assert dataclasses.is_dataclass(self), f"{type(self).__name__} must be a dataclass to be a PyTree"
        return {f.name: getattr(self, f.name) for f in dataclasses.fields(self)}

    @classmethod
    def __from_pytree__(cls, data: dict[str, Any]) -> Self:
        init = {f.name for f in dataclasses.fields(cls) if f.init}  # type: ignore[arg-type]
        obj = cls(**{k: v for k, v in data.items() if k in init})
        for k, v in data.items():
            if k not in init:
                object.__setattr__(obj, k, v)
        return obj

    def tree_map_tensor(self, fn: Callable[[Tensor], Tensor]) -> Self:
        return type(self).__from_pytree__({k: _map(v, fn, None) for k, v in self.__to_pytree__().items()})

    def tree_map(self, fn: Callable[["Tensor | PyTree"], "Tensor | PyTree"]) -> Self:
        """``fn`` sees tensors and nested pytrees (not descended into automatically)."""
        return type(self).__from_pytree__({k: _map(v, None, fn) for k, v in self.__to_pytree__().items()})

    def to(self, device: torch.device | str) -> Self:
        return self.tree_map(lambda t: t.to(device))

    def full_tensor(self) -> Self:
        """Gather distributed tensors (objects exposing ``full_tensor``); plain tensors pass through."""
        return self.tree_map(lambda t: t.full_tensor() if hasattr(t, "full_tensor") and not isinstance(t, PyTree) else (t.full_tensor() if isinstance(t, PyTree) else t))
