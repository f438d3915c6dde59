"""Rank-aware logging and metric tables.

API parity with utils/logging.py of the reference project (setup_logging :10-43, log_metrics :63-132,
DistributedLoggerAdapter :135-179): one root configuration with a rank prefix, loggers under one package
namespace, an adapter that only emits on global rank 0, and a grouped table rendering of metric dicts.
"""

from __future__ import annotations

import logging
import sys

import torch.distributed as dist

_ROOT = "lmsaes_b200"


def is_master() -> bool:
    return not dist.is_initialized() or dist.get_rank() == 0


def setup_logging(level: str = "INFO", format_string: str | None = None, enable_distributed: bool = True) -> logging.Logger:
    if format_string is None:
        prefix = f"[Rank {dist.get_rank()}] " if enable_distributed and dist.is_initialized() else ""
        format_string = prefix + "%(asctime)s - %(name)s - %(levelname)s - %(message)s"
    logging.basicConfig(
        level=getattr(logging, level.upper()),
        format=format_string,
        datefmt="%Y-%m-%d %H:%M:%S",
        handlers=[logging.StreamHandler(sys.stdout)],
        force=True,
    )
    return logging.getLogger(_ROOT)


def get_logger(name: str) -> logging.Logger:
    return logging.getLogger(f"{_ROOT}.{name}")


def _fmt(value) -> str:
    if isinstance(value, bool):
        return str(value)
    if isinstance(value, float):
        return f"{value:.2e}" if (value != 0 and abs(value) < 1e-3) else f"{value:.4f}"
    if isinstance(value, int):
        return f"{value:,}"
    return str(value)


def format_metrics_dict(metrics: dict, title: str = "Metrics", max_width: int = 80) -> str:
    """Group ``category/metric`` keys by category and align the values in a plain-text table."""
    if not metrics:
        return f"{title}: (empty)"
    groups: dict[str, dict[str, object]] = {}
    for key, value in metrics.items():
        cat, _, name = key.partition("/")
        if not name:
            cat, name = "general", key
        groups.setdefault(cat, {})[name] = value
    bar = "=" * max_width
    lines = ["", bar, title.center(max_width), bar]
    for cat, items in groups.items():
        lines.append("")
        lines.append(f"[{cat.upper().replace('_', ' ')}]")
        width = max(len(k) for k in items)
        lines.extend(f"  {k:<{width}} : {_fmt(v)}" for k, v in items.items())
    lines.append(bar)
    return "\n".join(lines)


def log_metrics(logger: logging.Logger, metrics: dict, step: int | None = None, title: str = "Training Metrics"):
    if not is_master():
        return
    if step is not None:
        title = f"{title} - Step {step}"
    logger.info(format_metrics_dict(metrics, title))


class DistributedLoggerAdapter(logging.LoggerAdapter):
    """Forwards to the wrapped logger on global rank 0 only."""

    def __init__(self, logger: logging.Logger, extra: dict | None = None):
        super().__init__(logger, extra or {})

    def process(self, msg, kwargs):
        return f"[Master] {msg}", kwargs

    def log(self, level, msg, *args, **kwargs):
        if is_master():
            super().log(level, msg, *args, **kwargs)


def get_distributed_logger(name: str) -> DistributedLoggerAdapter:
    return DistributedLoggerAdapter(get_logger(name))
