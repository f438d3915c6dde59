"""Operations on ``dict[str, Tensor]`` whose tensors share their leading dimensions
(utils/tensor_dict.py:11-100 of the reference project)."""

from __future__ import annotations

from typing import Any

import torch


def _expand_index(idx: torch.Tensor, like: torch.Tensor, dim: int) -> torch.Tensor:
    """Index of the key's shape, broadcast over the trailing dimensions of ``like``."""
    extra = like.ndim - idx.ndim
    view = idx.reshape(*idx.shape, *([1] * extra))
    return view.expand(*idx.shape, *like.shape[idx.ndim :]) if extra else view


def sort_dict_of_tensor(tensor_dict: dict[str, torch.Tensor], sort_dim: int = 0, sort_key: str = "elt", descending: bool = True,
                        device_mesh=None) -> dict[str, torch.Tensor]:  # fmt: skip
    """Sort every tensor along ``sort_dim`` by the order of ``tensor_dict[sort_key]``. Tensors of higher rank than the
    key are moved as whole slices. All tensors are local shards here, so ``device_mesh`` needs no handling."""
    key = tensor_dict[sort_key]
    order = key.argsort(dim=sort_dim, descending=descending)
    return {k: torch.gather(v, sort_dim, _expand_index(order, v, sort_dim)) for k, v in tensor_dict.items()}


def topk_dict_of_tensor(tensor_dict: dict[str, torch.Tensor], k: int, sort_key: str = "elt") -> dict[str, torch.Tensor]:
    """Keep the ``k`` largest rows (dim 0, per trailing position of the key), sorted descending: the same result as a
    full sort followed by ``[:k]`` at the cost of a selection."""
    key = tensor_dict[sort_key]
    k = min(k, key.shape[0])
    order = key.topk(k, dim=0, sorted=True).indices
    return {name: torch.gather(v, 0, _expand_index(order, v, 0)) for name, v in tensor_dict.items()}


def concat_dict_of_tensor(*dicts: dict[str, torch.Tensor], dim: int = 0) -> dict[str, torch.Tensor]:
    return {k: torch.cat([d[k] for d in dicts], dim=dim) for k in dicts[0].keys()}


def move_dict_of_tensor_to_device(tensor_dict: dict[str, Any], device: torch.device | str) -> dict[str, Any]:
    return {k: v.to(device, non_blocking=True) if isinstance(v, torch.Tensor) else v for k, v in tensor_dict.items()}


def batch_size(tensor_dict: dict[str, Any]) -> int:
    """Leading dimension shared by the tensors of a batch."""
    sizes = {v.shape[0] for v in tensor_dict.values() if isinstance(v, torch.Tensor) and v.ndim > 0}
    assert len(sizes) == 1, f"inconsistent batch sizes: {sizes}"
    return sizes.pop()
