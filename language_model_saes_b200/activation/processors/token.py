"""Raw records -> token tensors, and padding / truncation to a fixed context length
(activation/processors/token.py:11-80 of the reference project)."""

from __future__ import annotations

from typing import Any, Iterable

from ...utils.misc import pad_and_truncate_tokens
from .core import BaseActivationProcessor


class RawDatasetTokenProcessor(BaseActivationProcessor[Iterable[dict[str, Any]], Iterable[dict[str, Any]]]):
    def __init__(self, prepend_bos: bool | None = None):
        self.prepend_bos = prepend_bos

    def process(self, data: Iterable[dict[str, Any]], *, model, **kwargs) -> Iterable[dict[str, Any]]:
        for d in data:
            tokens = model.to_tokens(d, prepend_bos=self.prepend_bos)
            out = {"tokens": tokens[0]}
            if "meta" in d:
                out["meta"] = d["meta"]
            yield out


class PadAndTruncateTokensProcessor(BaseActivationProcessor[Iterable[dict[str, Any]], Iterable[dict[str, Any]]]):
    def __init__(self, seq_len: int):
        self.seq_len = seq_len

    def process(self, data: Iterable[dict[str, Any]], *, pad_token_id: int = 0, **kwargs) -> Iterable[dict[str, Any]]:
        for d in data:
            assert "tokens" in d, "PadAndTruncateTokensProcessor needs a 'tokens' field"
            yield {**d, "tokens": pad_and_truncate_tokens(d["tokens"], self.seq_len, pad_token_id=pad_token_id)}
