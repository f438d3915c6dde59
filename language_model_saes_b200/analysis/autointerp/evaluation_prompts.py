"""Prompts that test an explanation: *detection* (does this excerpt contain the feature?) and *fuzzing* (are the
highlighted tokens the right ones?), after analysis/autointerp/evaluation_prompts.py of the reference project."""

from __future__ import annotations

from typing import Any

from ..samples import TokenizedSample
from .autointerp_base import AutoInterpConfig

_ANSWER_NOTE = (
    'Answer with a single JSON object: {"steps": [{"thought": "..."}, ...], "evaluation_results": [true, false, ...]} '
    "with exactly one boolean per example, in the order given."
)


def generate_detection_prompt(cfg: AutoInterpConfig, explanation: dict[str, Any], examples: list[TokenizedSample]) -> tuple[str, str]:
    system = (
        "You check an explanation of a language-model feature. You are given the explanation and several plain text "
        "excerpts. For each excerpt decide whether the feature, as explained, would fire on at least one of its "
        "tokens (true) or on none (false). Judge only by the explanation. "
        + ("Give a short reason per excerpt in `steps`. " if cfg.include_cot else "Leave `steps` empty. ")
        + _ANSWER_NOTE
    )
    body = "\n".join(f"Example {i + 1}: {ex.display_plain()}" for i, ex in enumerate(examples))
    user = f"Explanation: {explanation['final_explanation']}\n\n{body}\n\nWhich examples contain the feature?"
    return system, user


def generate_fuzzing_prompt(cfg: AutoInterpConfig, explanation: dict[str, Any], examples: list[tuple[TokenizedSample, bool]]) -> tuple[str, str]:
    system = (
        "You check an explanation of a language-model feature. You are given the explanation and several excerpts in "
        "which some tokens are wrapped in << and >>. In some excerpts the wrapped tokens are where the feature truly "
        "fires; in others random tokens were wrapped instead. For each excerpt decide whether the wrapped tokens are "
        "consistent with the explanation (true) or not (false). "
        + ("Give a short reason per excerpt in `steps`. " if cfg.include_cot else "Leave `steps` empty. ")
        + _ANSWER_NOTE
    )
    body = "\n".join(f"Example {i + 1}: {ex.display_highlighted(cfg.activation_threshold)}" for i, (ex, _) in enumerate(examples))
    user = f"Explanation: {explanation['final_explanation']}\n\n{body}\n\nWhich examples are marked correctly?"
    return system, user
