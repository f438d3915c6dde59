"""Dataset -> stream of raw records, each tagged with its position in the dataset
(``meta.context_idx``), the dataset name and optional metadata (activation/processors/huggingface.py:20-102 of the
reference project)."""

from __future__ import annotations

import itertools
from typing import Any, Iterable, Optional

from torch.utils.data import DataLoader
from tqdm import tqdm

from .core import BaseActivationProcessor


def identity_collate_fn(x):
    """Module-level so that DataLoader workers can pickle it."""
    return x


class HuggingFaceDatasetLoader(BaseActivationProcessor[Any, Iterable[dict[str, Any]]]):
    def __init__(self, batch_size: int, num_workers: int = 0, with_info: bool = False, show_progress: bool = True):
        self.batch_size = batch_size
        self.num_workers = num_workers
        self.with_info = with_info
        self.show_progress = show_progress

    def process(self, data, *, dataset_name: str | None = None, metadata: Optional[dict[str, Any]] = None, **kwargs):
        loader: Iterable[list[dict[str, Any]]] = DataLoader(
            data, batch_size=self.batch_size, shuffle=False, pin_memory=False, collate_fn=identity_collate_fn,
            num_workers=self.num_workers,
        )  # fmt: skip
        if self.show_progress:
            loader = tqdm(loader, desc="Loading dataset")
        flat = itertools.chain.from_iterable(loader)
        if not self.with_info:
            return flat
        extra = {**({"dataset_name": dataset_name} if dataset_name else {}), **(metadata or {})}
        return ({**rec, "meta": {"context_idx": i, **extra}} for i, rec in enumerate(flat))
