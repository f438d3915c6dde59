"""Small helpers: dtype names, token padding, activation-norm estimation.

Covers utils/misc.py of the reference project (dtype maps :62-104, calculate_activation_norm :122-159,
pad_and_truncate_tokens :162-188, ensure_tokenized :197-208).
"""

from __future__ import annotations

import warnings
from typing import Iterable

import torch
import torch.distributed as dist

_CANONICAL = {
    "float16": torch.float16,
    "float32": torch.float32,
    "float64": torch.float64,
    "int8": torch.int8,
    "int16": torch.int16,
    "int32": torch.int32,
    "int64": torch.int64,
    "bool": torch.bool,
    "bfloat16": torch.bfloat16,
}
_ALIASES = {
    "bf16": torch.bfloat16,
    "float": torch.float32,
    "fp16": torch.float16,
    "fp32": torch.float32,
    "fp64": torch.float64,
    "int": torch.int32,
    "half": torch.float16,
    "double": torch.float64,
}
str_dtype_map: dict[str, torch.dtype] = {**_CANONICAL, **_ALIASES}
str_dtype_map.update({f"torch.{k}": v for k, v in {**_CANONICAL, "float": torch.float32, "int": torch.int32}.items()})
_dtype_to_str = {v: k for k, v in _CANONICAL.items()}


def convert_str_to_torch_dtype(name: str) -> torch.dtype:
    try:
        return str_dtype_map[name]
    except KeyError:
        raise ValueError(f"Unsupported data type: {name}. Supported: {sorted(str_dtype_map)}") from None


def convert_torch_dtype_to_str(dtype: torch.dtype) -> str:
    try:
        return _dtype_to_str[dtype]
    except KeyError:
        raise ValueError(f"Unsupported data type: {dtype}. Supported: {sorted(_dtype_to_str.values())}") from None


def tensor_id(t: torch.Tensor) -> tuple[int, int, tuple[int, ...], tuple[int, ...]]:
    """Hashable identity of a tensor *view* (distinct views of one buffer differ)."""
    return (t.data_ptr(), int(t.storage_offset()), tuple(t.shape), tuple(t.stride()))


def is_master() -> bool:
    return not dist.is_initialized() or dist.get_rank() == 0


def pad_and_truncate_tokens(tokens: torch.Tensor, seq_len: int, pad_token_id: int = 0) -> torch.Tensor:
    """Right-pad with ``pad_token_id`` or cut the last dimension to exactly ``seq_len``."""
    n = tokens.size(-1)
    if n >= seq_len:
        return tokens[..., :seq_len]
    pad = tokens.new_full((*tokens.shape[:-1], seq_len - n), pad_token_id)
    return torch.cat([tokens, pad], dim=-1)


def get_slice_length(s: slice, length: int) -> int:
    return len(range(*s.indices(length)))


def ensure_tokenized(prompt, tokenizer, device: torch.device | str = "cpu") -> torch.Tensor:
    """str | tensor | list[int] -> 1-D tensor of token ids."""
    if isinstance(prompt, str):
        return tokenizer(prompt, return_tensors="pt").input_ids[0].to(device)
    if isinstance(prompt, torch.Tensor):
        return (prompt.squeeze(0) if prompt.ndim == 2 else prompt).to(device)
    if isinstance(prompt, (list, tuple)):
        return torch.tensor(list(prompt), dtype=torch.long, device=device)
    raise TypeError(f"Unsupported prompt type: {type(prompt)}")


def calculate_activation_norm(
    activation_stream: Iterable[dict[str, torch.Tensor]],
    hook_points: list[str],
    batch_num: int = 8,
    device_mesh=None,
) -> dict[str, float]:
    """Mean L2 norm per hook point over the first ``batch_num`` batches of the stream.

    Under a mesh with a ``head`` dimension each head rank measures its own slice of the hook points and the
    results are merged over the head group (reference: utils/misc.py:122-159). Under data parallelism the
    per-rank means are averaged so that every rank normalises with the same constant.
    """
    from ..parallel.mesh import mesh_dim_size, mesh_group, mesh_local_rank

    hook_points = list(hook_points)
    head = mesh_dim_size(device_mesh, "head")
    if head > 1:
        per = len(hook_points) // head
        r = mesh_local_rank(device_mesh, "head")
        hook_points = hook_points[r * per : (r + 1) * per]
    assert hook_points, "No hook points provided"
    sums = {k: 0.0 for k in hook_points}
    counts = {k: 0 for k in hook_points}
    it = iter(activation_stream)
    for _ in range(batch_num):
        try:
            batch = next(it)
        except StopIteration:
            warnings.warn("Activation stream ended before the requested number of norm batches was read.")
            break
        for k in hook_points:
            n = batch[k].float().norm(p=2, dim=-1)
            sums[k] += float(n.sum())
            counts[k] += n.numel()
    if mesh_dim_size(device_mesh, "data") > 1:
        g = mesh_group(device_mesh, "data")
        gathered: list = [None] * dist.get_world_size(g)
        dist.all_gather_object(gathered, (sums, counts), group=g)
        sums = {k: sum(s[k] for s, _ in gathered) for k in hook_points}
        counts = {k: sum(c[k] for _, c in gathered) for k in hook_points}
    norms = {k: sums[k] / max(counts[k], 1) for k in hook_points}
    if head > 1:
        g = mesh_group(device_mesh, "head")
        gathered = [None] * dist.get_world_size(g)
        dist.all_gather_object(gathered, norms, group=g)
        norms = {k: v for d in gathered for k, v in d.items()}
    return norms
