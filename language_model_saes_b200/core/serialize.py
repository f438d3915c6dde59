"""Versioned (de)serialisation of dataclass object graphs that contain tensors.

Same contract as core/serialize.py of the reference project (:11-140): ``dump(obj)`` gives
``{"_version": FORMAT_VERSION, "data": <plain nested structure with tensors>}``; ``load(blob, cls)`` rebuilds
``cls``; a class can declare ``@migrate(before="N")`` static methods that rewrite raw dicts written by older
format versions, applied in ascending order while loading. Classes may customise their encoding with
``__unstructure__(self) -> Any`` and ``__structure__(cls, data) -> obj``. ``dumps`` / ``loads`` wrap the blob in a
``torch.save`` byte string (for databases and files).
"""

from __future__ import annotations

import dataclasses
import io
import types
import typing
from contextvars import ContextVar
from typing import Any, Callable, TypeVar, get_args, get_origin, get_type_hints

import torch

FORMAT_VERSION = "2"
T = TypeVar("T")
_loading_source_version: ContextVar[str | None] = ContextVar("_loading_source_version", default=None)


def migrate(*, before: str) -> Callable[[Callable[[Any], Any]], Any]:
    """Mark a static method ``(raw: dict) -> dict`` as the migration to run for blobs older than ``before``."""

    def decorator(func):
        target = func.__func__ if isinstance(func, staticmethod) else func
        target.__migrate_before__ = before
        return staticmethod(target)

    return decorator


def _collect_migrations(cls: type) -> list[tuple[str, Callable[[Any], Any]]]:
    out = []
    for attr in vars(cls).values():
        if isinstance(attr, staticmethod) and getattr(attr.__func__, "__migrate_before__", None) is not None:
            out.append((attr.__func__.__migrate_before__, attr.__func__))
    return sorted(out, key=lambda e: int(e[0]))


def unstructure(obj: Any) -> Any:
    if hasattr(obj, "__unstructure__") and not isinstance(obj, type):
        return obj.__unstructure__()
    if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        return {f.name: unstructure(getattr(obj, f.name)) for f in dataclasses.fields(obj)}
    if isinstance(obj, dict):
        return {k: unstructure(v) for k, v in obj.items()}
    if isinstance(obj, tuple) and hasattr(obj, "_fields"):
        return {k: unstructure(v) for k, v in obj._asdict().items()}
    if isinstance(obj, (list, tuple, set, frozenset)):
        return [unstructure(v) for v in obj]
    return obj


def _substitute(tp: Any, typevar_map: dict[Any, Any]) -> Any:
    """Replace type variables inside ``tp`` (``V`` -> ``list[int]``, ``tuple[V, ...]`` -> ``tuple[list[int], ...]``)."""
    if not typevar_map:
        return tp
    if isinstance(tp, typing.TypeVar):
        return typevar_map.get(tp, Any)
    args = get_args(tp)
    if not args:
        return tp
    new_args = tuple(a if a is Ellipsis else _substitute(a, typevar_map) for a in args)
    origin = get_origin(tp)
    try:
        return origin[new_args] if origin not in (typing.Union, types.UnionType) else typing.Union[new_args]
    except TypeError:
        return tp


def structure(data: Any, cls: Any) -> Any:
    if cls is Any or cls is None or data is None or isinstance(cls, typing.TypeVar):
        return data
    origin = get_origin(cls)
    if origin in (typing.Union, types.UnionType):
        args = [a for a in get_args(cls) if a is not type(None)]
        if len(args) == 1:
            return structure(data, args[0])
        for a in args:
            try:
                if isinstance(a, type) and isinstance(data, a):
                    return data
            except TypeError:
                pass
        for a in args:
            try:
                return structure(data, a)
            except Exception:  # noqa: BLE001
                continue
        return data
    if origin in (list, set, frozenset):
        (a,) = get_args(cls) or (Any,)
        return origin(structure(v, a) for v in data)
    if origin is tuple:
        args = get_args(cls)
        if len(args) == 2 and args[1] is Ellipsis:
            return tuple(structure(v, args[0]) for v in data)
        return tuple(structure(v, a) for v, a in zip(data, args)) if args else tuple(data)
    if origin is dict:
        ka, va = get_args(cls) or (Any, Any)
        return {structure(k, ka) if ka in (int, str, float) else k: structure(v, va) for k, v in data.items()}
    typevar_map: dict[Any, Any] = {}
    if origin is not None:
        # a parametrised generic dataclass (Box[int]): remember what its type variables stand for
        params = getattr(origin, "__parameters__", ())
        typevar_map = dict(zip(params, get_args(cls)))
        cls = origin
    if isinstance(cls, type):
        version = _loading_source_version.get()
        if version is not None and isinstance(data, dict):
            for before, fn in _collect_migrations(cls):
                if int(version) < int(before):
                    data = fn(data)
        if "__structure__" in cls.__dict__:
            return cls.__structure__(data)
        if dataclasses.is_dataclass(cls):
            hints = get_type_hints(cls)
            kwargs, later = {}, {}
            for f in dataclasses.fields(cls):
                if f.name in data:
                    (kwargs if f.init else later)[f.name] = structure(data[f.name], _substitute(hints.get(f.name, Any), typevar_map))
            obj = cls(**kwargs)
            for k, v in later.items():
                object.__setattr__(obj, k, v)
            return obj
        if hasattr(cls, "_fields") and isinstance(data, dict):
            return cls(**data)
        if cls in (int, float, str, bool) and not isinstance(data, cls):
            return cls(data)
    return data


def dump(obj: Any) -> dict[str, Any]:
    return {"_version": FORMAT_VERSION, "data": unstructure(obj)}


def load(blob: Any, cls: type[T]) -> T:
    token = _loading_source_version.set(str(blob["_version"]))
    try:
        return structure(blob["data"], cls)
    finally:
        _loading_source_version.reset(token)


def dumps(obj: Any) -> bytes:
    buf = io.BytesIO()
    torch.save(dump(obj), buf)
    return buf.getvalue()


def loads(data: bytes, cls: type[T], device: torch.device | str = "cpu") -> T:
    return load(torch.load(io.BytesIO(data), map_location=device, weights_only=False), cls)


__all__ = ["FORMAT_VERSION", "dump", "dumps", "load", "loads", "migrate", "structure", "unstructure"]
