"""Hierarchical timer with the ``timer.time(name)`` interface of the reference project
(utils/timer.py:35-509 there), measured differently.

The reference synchronises the whole device at every start and stop. Here a region is bracketed by two CUDA
events recorded on the current stream (no device-wide sync on the hot path); elapsed times are resolved
lazily, when a summary or a value is asked for. On CPU the wall clock is used. Each region also opens an
NVTX range of the same name. The timer is disabled by default and then costs one attribute check.
"""

from __future__ import annotations

import functools
import time as _time
from contextlib import contextmanager
from typing import Callable

import torch


class TimerNode:
    __slots__ = ("name", "path", "parent", "children", "total_ms", "count", "pending", "wall_start")

    def __init__(self, name: str, path: str, parent: str | None):
        self.name = name
        self.path = path
        self.parent = parent
        self.children: list[str] = []
        self.total_ms = 0.0
        self.count = 0
        self.pending: list[tuple[torch.cuda.Event, torch.cuda.Event]] = []
        self.wall_start: float | None = None


class Timer:
    _instance: "Timer | None" = None

    def __new__(cls):
        if cls._instance is None:
            inst = super().__new__(cls)
            inst._enabled = False
            inst._nodes = {}
            inst._stack = []
            inst._open = {}
            inst.use_cuda_events = True
            inst.use_nvtx = False
            cls._instance = inst
        return cls._instance

    # ---- control -----------------------------------------------------------------------------
    def enable(self):
        self._enabled = True

    def disable(self):
        self._enabled = False

    @property
    def enabled(self) -> bool:
        return self._enabled

    def reset(self):
        self._nodes = {}
        self._stack = []
        self._open = {}

    # ---- measurement -------------------------------------------------------------------------
    def _path(self, name: str) -> str:
        return f"{self._stack[-1]}/{name}" if self._stack else name

    def start(self, name: str):
        if not self._enabled:
            return
        path = self._path(name)
        node = self._nodes.get(path)
        if node is None:
            parent = self._stack[-1] if self._stack else None
            node = TimerNode(name, path, parent)
            self._nodes[path] = node
            if parent is not None:
                self._nodes[parent].children.append(path)
        self._stack.append(path)
        if self.use_cuda_events and torch.cuda.is_available():
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._open[path] = ev
            if self.use_nvtx:
                torch.cuda.nvtx.range_push(name)
        else:
            node.wall_start = _time.perf_counter()

    def stop(self, name: str):
        if not self._enabled or not self._stack:
            return
        path = self._stack.pop()
        node = self._nodes[path]
        node.count += 1
        if path in self._open:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            node.pending.append((self._open.pop(path), end))
            if self.use_nvtx:
                torch.cuda.nvtx.range_pop()
            if len(node.pending) > 4096:
                self._resolve(node)
        elif node.wall_start is not None:
            node.total_ms += (_time.perf_counter() - node.wall_start) * 1e3
            node.wall_start = None

    def _resolve(self, node: TimerNode):
        if node.pending:
            node.pending[-1][1].synchronize()
            for s, e in node.pending:
                node.total_ms += s.elapsed_time(e)
            node.pending = []

    @contextmanager
    def _region(self, name: str):
        self.start(name)
        try:
            yield
        finally:
            self.stop(name)

    def time(self, name: str):
        """Context manager and decorator: ``with timer.time("x"): ...`` or ``@timer.time("x")``."""
        timer = self

        class _Both:
            def __enter__(self_inner):
                timer.start(name)

            def __exit__(self_inner, *exc):
                timer.stop(name)
                return False

            def __call__(self_inner, func: Callable):
                @functools.wraps(func)
                def wrapper(*args, **kwargs):
                    if not timer._enabled:
                        return func(*args, **kwargs)
                    timer.start(name)
                    try:
                        return func(*args, **kwargs)
                    finally:
                        timer.stop(name)

                return wrapper

        return _Both()

    def profile(self, func: Callable | None = None, *, name: str | None = None, print_summary: bool = True):
        """Decorator that enables the timer for one call of ``func`` and prints the summary afterwards."""

        def decorator(f: Callable):
            @functools.wraps(f)
            def wrapper(*args, **kwargs):
                was = self._enabled
                self.reset()
                self.enable()
                try:
                    with self.time(name or f.__name__):
                        return f(*args, **kwargs)
                finally:
                    if print_summary:
                        print(self.summary())
                    self._enabled = was

            return wrapper

        return decorator(func) if func is not None else decorator

    # ---- queries -----------------------------------------------------------------------------
    def _find(self, name: str, parent_context: str | None = None) -> list[TimerNode]:
        out = []
        for path, node in self._nodes.items():
            if node.name == name and (parent_context is None or (node.parent or "").endswith(parent_context)):
                out.append(node)
        return out

    def get_time(self, name: str, parent_context: str | None = None) -> float:
        """Accumulated seconds of every region with this name."""
        total = 0.0
        for n in self._find(name, parent_context):
            self._resolve(n)
            total += n.total_ms
        return total / 1e3

    def get_count(self, name: str, parent_context: str | None = None) -> int:
        return sum(n.count for n in self._find(name, parent_context))

    def get_average_time(self, name: str, parent_context: str | None = None) -> float:
        c = self.get_count(name, parent_context)
        return self.get_time(name, parent_context) / c if c else 0.0

    def get_all_timers(self) -> dict[str, float]:
        for n in self._nodes.values():
            self._resolve(n)
        return {p: n.total_ms / 1e3 for p, n in self._nodes.items()}

    def get_all_counts(self) -> dict[str, int]:
        return {p: n.count for p, n in self._nodes.items()}

    def get_all_average_times(self) -> dict[str, float]:
        t = self.get_all_timers()
        return {p: (t[p] / n.count if n.count else 0.0) for p, n in self._nodes.items()}

    def get_active_timers(self) -> list[str]:
        return list(self._stack)

    def reset_timer(self, name: str, parent_context: str | None = None):
        for n in self._find(name, parent_context):
            n.total_ms, n.count, n.pending = 0.0, 0, []

    def summary(self) -> str:
        times = self.get_all_timers()
        lines = ["Timer summary (seconds, count, % of parent)"]

        def walk(path: str, depth: int, parent_time: float | None):
            n = self._nodes[path]
            t = times[path]
            pct = f" {100.0 * t / parent_time:5.1f}%" if parent_time else ""
            avg = t / n.count if n.count else 0.0
            lines.append(f"{'  ' * depth}{n.name}: {t:.4f}s  x{n.count}  avg {avg * 1e3:.3f}ms{pct}")
            for c in n.children:
                walk(c, depth + 1, t)

        for path, n in self._nodes.items():
            if n.parent is None:
                walk(path, 0, None)
        return "\n".join(lines)


timer = Timer()
