"""Stream processors: objects that turn one iterable of records into another."""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Generic, Iterable, TypeVar

InputT = TypeVar("InputT")
OutputT = TypeVar("OutputT", bound=Iterable)


class BaseActivationProcessor(Generic[InputT, OutputT], ABC):
    """``process(data, **kwargs)`` consumes a stream lazily and yields a new one; instances are callable."""

    @abstractmethod
    def process(self, data: InputT, **kwargs) -> OutputT:
        raise NotImplementedError

    def __call__(self, data: InputT, **kwargs) -> OutputT:
        return self.process(data, **kwargs)
