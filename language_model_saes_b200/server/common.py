"""Small helpers of the server (server/utils/common.py of the reference project)."""

from __future__ import annotations

import re
import threading
from functools import wraps
from typing import Any, Callable

import numpy as np
import torch


class synchronized:
    """Serialise calls that have the same keyword arguments (loading one model twice at once is wasteful); calls with
    different arguments run in parallel. Attributes of the wrapped callable (``cache_clear`` ...) pass through."""

    def __init__(self, func: Callable):
        self._func = func
        self._locks: dict[frozenset, threading.Lock] = {}
        self._guard = threading.Lock()
        wraps(func)(self)

    def __call__(self, *args, **kwargs):
        assert len(args) == 0, "Positional arguments are not supported"
        key = frozenset(kwargs.items())
        with self._guard:
            lock = self._locks.setdefault(key, threading.Lock())
        with lock:
            return self._func(**kwargs)

    def __getattr__(self, name: str):
        return getattr(self._func, name)


def make_serializable(obj: Any) -> Any:
    if isinstance(obj, torch.Tensor):
        return obj.detach().cpu().tolist()
    if isinstance(obj, np.ndarray):
        return obj.tolist()
    if isinstance(obj, (np.integer, np.floating)):
        return obj.item()
    if isinstance(obj, dict):
        return {k: make_serializable(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [make_serializable(v) for v in obj]
    return obj


def natural_sort_key(name: str) -> list[tuple[int, int | str]]:
    """``"L2"`` sorts before ``"L10"``."""
    return [(0, int(p)) if p.isdigit() else (1, p.lower()) for p in re.split(r"(\d+)", name) if p]


def packed(data: Any):
    """msgpack response."""
    import msgpack
    from fastapi import Response

    return Response(content=msgpack.packb(make_serializable(data)), media_type="application/x-msgpack")
