"""Named tensor dimensions and token-mask reductions.

Same role as utils/tensor_specs.py of the reference project (:8-84): a tensor's dimension names are inferred
from its rank, and reductions address dimensions by name so that [batch, d] and [batch, context, d] inputs
share one code path.
"""

from __future__ import annotations

import torch
from torch import Tensor


class TensorSpecs:
    """Dimension names by tensor rank for a single-layer dictionary."""

    @staticmethod
    def feature_acts(tensor: Tensor) -> tuple[str, ...]:
        return _by_rank(tensor, {2: ("batch", "sae"), 3: ("batch", "context", "sae")})

    @staticmethod
    def reconstructed(tensor: Tensor) -> tuple[str, ...]:
        return _by_rank(tensor, {2: ("batch", "model"), 3: ("batch", "context", "model")})

    @staticmethod
    def label(tensor: Tensor) -> tuple[str, ...]:
        return TensorSpecs.reconstructed(tensor)

    @staticmethod
    def loss(tensor: Tensor) -> tuple[str, ...]:
        return _by_rank(tensor, {1: ("batch",), 2: ("batch", "context")})


def _by_rank(tensor: Tensor, table: dict[int, tuple[str, ...]]) -> tuple[str, ...]:
    try:
        return table[tensor.ndim]
    except KeyError:
        raise ValueError(f"Cannot infer tensor specs for tensor with {tensor.ndim} dimensions.") from None


_REDUCERS = {
    "sum": lambda t, dims: t.sum(dim=dims),
    "mean": lambda t, dims: t.mean(dim=dims),
    "max": lambda t, dims: t.amax(dim=dims),
    "min": lambda t, dims: t.amin(dim=dims),
}


def reduce(tensor: Tensor, specs: tuple[str, ...], reduction_map: dict[str, str]) -> tuple[Tensor, tuple[str, ...]]:
    """Reduce the named dimensions present in ``specs``; absent names are ignored."""
    assert tensor.ndim == len(specs), f"Tensor has {tensor.ndim} dimensions, but specs have {len(specs)}"
    for name, how in reduction_map.items():
        if name in specs:
            d = specs.index(name)
            tensor = _REDUCERS[how](tensor, (d,))
            specs = specs[:d] + specs[d + 1 :]
    return tensor, specs


def apply_token_mask(
    tensor: Tensor, specs: tuple[str, ...], mask: Tensor | None = None, reduction: str = "sum"
) -> tuple[Tensor, tuple[str, ...]]:
    """Sum / mean over the token dimensions (batch, context), counting only tokens whose mask is 1."""
    assert tensor.ndim == len(specs), f"Tensor has {tensor.ndim} dimensions, but specs have {len(specs)}"
    if mask is None:
        return reduce(tensor, specs, {"batch": reduction, "context": reduction})
    token_dims = tuple(i for i, s in enumerate(specs) if s in ("batch", "context"))
    token_shape = tuple(tensor.shape[i] for i in token_dims)
    assert tuple(mask.shape) == token_shape, f"Mask has shape {tuple(mask.shape)}, token part is {token_shape}"
    view = [tensor.shape[i] if i in token_dims else 1 for i in range(tensor.ndim)]
    m = mask.to(tensor.dtype).reshape(view)
    out = (tensor * m).sum(dim=token_dims)
    if reduction == "mean":
        out = out / mask.sum().to(out.dtype)
    return out, tuple(s for s in specs if s not in ("batch", "context"))
