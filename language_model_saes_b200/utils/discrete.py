"""String <-> small-integer dictionaries for metadata that has to live in tensors (utils/discrete.py:6-140 of the
reference project). With a process group every rank ends up with the same table: unseen strings are all-gathered,
rank 0 of the group numbers them (sorted, so the numbering does not depend on set order) and broadcasts the update."""

from __future__ import annotations

from typing import Optional

import torch.distributed as dist


class DiscreteMapper:
    def __init__(self) -> None:
        self.value_to_int: dict[str, int] = {}
        self.int_to_value: list[str] = []

    @property
    def counter(self) -> int:
        return len(self.int_to_value)

    def _add(self, value: str) -> int:
        idx = self.value_to_int.get(value)
        if idx is None:
            idx = self.value_to_int[value] = len(self.int_to_value)
            self.int_to_value.append(value)
        return idx

    def encode(self, values: list[str], group: Optional[dist.ProcessGroup] = None) -> list[int]:
        if group is not None and dist.get_world_size(group) > 1:
            unseen = sorted({v for v in values if v not in self.value_to_int})
            gathered: list = [None] * dist.get_world_size(group)
            dist.all_gather_object(gathered, unseen, group=group)
            # every rank computes the same sorted union, so no broadcast is needed to agree on the numbering
            for v in sorted({v for part in gathered for v in (part or [])}):
                self._add(v)
            return [self.value_to_int[v] for v in values]
        return [self._add(v) for v in values]

    def decode(self, integers: list[int]) -> list[str]:
        return [self.int_to_value[i] for i in integers]

    def get_mapping(self) -> dict[str, int]:
        return dict(self.value_to_int)


class KeyedDiscreteMapper:
    """One ``DiscreteMapper`` per metadata key, created on first use."""

    def __init__(self) -> None:
        self.mappers: dict[str, DiscreteMapper] = {}

    def add_mapper(self, key: str, mapper: DiscreteMapper) -> None:
        self.mappers[key] = mapper

    def get_mapper(self, key: str) -> DiscreteMapper:
        return self.mappers[key]

    def encode(self, key: str, values: list[str], group: Optional[dist.ProcessGroup] = None) -> list[int]:
        if key not in self.mappers:
            self.mappers[key] = DiscreteMapper()
        return self.mappers[key].encode(values, group=group)

    def decode(self, key: str, integers: list[int]) -> list[str]:
        if key not in self.mappers:
            raise KeyError(f"no mapper for key {key!r}")
        return self.mappers[key].decode(integers)

    def keys(self) -> list[str]:
        return list(self.mappers.keys())
