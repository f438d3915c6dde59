"""Text samples with per-token activations, grouped into display segments
(analysis/samples.py:17-219 of the reference project)."""

from __future__ import annotations

import bisect
from dataclasses import dataclass
from typing import Any

import torch


def process_token(token: str) -> str:
    """Make whitespace control characters visible."""
    return token.replace("\n", "⏎").replace("\t", "→").replace("\r", "↵")


@dataclass
class Segment:
    text: str
    activation: float

    def display(self, abs_threshold: float) -> str:
        return f"<<{self.text}>>" if self.activation > abs_threshold else self.text

    def display_max(self, abs_threshold: float) -> str:
        return f"{self.text}\n" if self.activation > abs_threshold else ""


@dataclass
class ZPatternSegment:
    """Which earlier tokens contribute to one activating token of an attention feature."""

    contributing_indices: list[int]
    contributions: list[float]
    max_contribution: float


@dataclass
class TokenizedSample:
    segments: list[Segment]
    max_activation: float
    """Maximum activation of the feature over the whole analysis (not of this sample)."""
    z_pattern_data: dict[int, ZPatternSegment] | None = None

    @property
    def sample_max_activation(self) -> float:
        return max(seg.activation for seg in self.segments)

    def _context(self, i: int, n: int = 3) -> str:
        return "".join(s.text for s in self.segments[max(0, i - n) : i])

    def to_max_activation_surrounding(self, visible_range: int) -> "TokenizedSample":
        assert self.z_pattern_data is None, "Z pattern data is not supported for max activation surrounding tokens"
        acts = [s.activation for s in self.segments]
        i = acts.index(max(acts))
        return TokenizedSample(self.segments[max(0, i - visible_range) : i + visible_range], self.max_activation)

    def display_highlighted(self, threshold: float = 0.7) -> str:
        return "".join(s.display(threshold * self.max_activation) for s in self.segments)

    def display_plain(self) -> str:
        return "".join(s.text for s in self.segments)

    def display_max(self, threshold: float = 0.7) -> str:
        """One line per distinct strongly-activating token: ``(three tokens of context) token``; attention features
        get their strongest contributing tokens in front: ``[(ctx) tok; ...] => (ctx) token``."""
        out, seen = "", set()
        for i, seg in enumerate(self.segments):
            if seg.activation <= threshold * self.max_activation or seg.text == "" or seg.text in seen:
                continue
            seen.add(seg.text)
            if self.z_pattern_data is not None and i in self.z_pattern_data:
                z = self.z_pattern_data[i]
                srcs = [
                    f"({process_token(self._context(j))}) {process_token(self.segments[j].text)}"
                    for j, c in zip(z.contributing_indices, z.contributions)
                    if c > threshold * z.max_contribution
                ]
                out += f"[{'; '.join(srcs)}] => "
            out += f"({process_token(self._context(i))}) {process_token(seg.text)}\n"
        return out

    def display_next(self, threshold: float = 0.7) -> str:
        """The last distinct token that directly follows a strongly-activating token."""
        out, seen, after_active = "", set(), False
        for seg in self.segments:
            if after_active and seg.text != "" and seg.text not in seen:
                seen.add(seg.text)
                out = process_token(seg.text) + "\n"
            after_active = seg.activation > threshold * self.max_activation
        return out

    def add_z_pattern_data(self, z_pattern_indices: torch.Tensor, z_pattern_values: torch.Tensor, origins: list[dict[str, Any] | None]):
        """``z_pattern_indices [2, nnz]`` = (query position, key position)."""
        self.z_pattern_data = {}
        for q in z_pattern_indices[0].unique_consecutive().tolist():
            if origins[q] is None:
                continue
            sel = z_pattern_indices[0] == q
            vals = z_pattern_values[sel]
            self.z_pattern_data[int(q)] = ZPatternSegment(z_pattern_indices[1, sel].tolist(), vals.tolist(), vals.max().item())

    def has_z_pattern_data(self) -> bool:
        return self.z_pattern_data is not None

    @staticmethod
    def construct(text: str, activations: torch.Tensor, origins: list[dict[str, Any] | None], max_activation: float) -> "TokenizedSample":
        """Cut ``text`` at every token boundary found in ``origins`` (entries ``{"key": "text", "range": (a, b)}``); a
        segment's activation is the maximum over the tokens that start inside it and end within it."""
        toks = sorted(
            (o["range"][0], o["range"][1], float(a))
            for o, a in zip(origins, activations.tolist())
            if o and o.get("key") == "text" and "range" in o
        )
        cuts = sorted({p for s, e, _ in toks for p in (s, e)})
        starts = [t[0] for t in toks]
        segments = []
        for a, b in zip(cuts[:-1], cuts[1:]):
            best = 0.0
            for s, e, act in toks[bisect.bisect_left(starts, a) :]:
                if s > b:
                    break
                if e <= b:
                    best = max(best, act)
            segments.append(Segment(text[a:b], best))
        return TokenizedSample(segments, max_activation)
