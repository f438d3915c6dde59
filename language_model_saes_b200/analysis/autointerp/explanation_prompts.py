"""Prompts that ask a chat model to explain a feature from its activating examples. Two styles, as in
analysis/autointerp/explanation_prompts.py of the reference project: a structured JSON answer with reasoning steps,
and a terse one-phrase answer in the style used by public feature browsers (which also sees the top logits)."""

from __future__ import annotations

from typing import Any

from ..samples import TokenizedSample
from .autointerp_base import AutoInterpConfig

_JSON_SCHEMA_NOTE = """Answer with a single JSON object with these keys:
  "steps": a list of {"thought": "..."} objects, your reasoning in order (may be empty if no reasoning was requested);
  "final_explanation": one or two sentences that state what the feature responds to;
  "activation_consistency": an integer 1-5, how uniformly the examples fit the explanation (5 = all of them);
  "complexity": an integer 1-5, how abstract the concept is (1 = a single token or character, 5 = an abstract idea)."""


def _numbered(blocks: list[str]) -> str:
    return "\n".join(f"Example {i + 1}:\n{b}" for i, b in enumerate(blocks))


def generate_explanation_prompt(cfg: AutoInterpConfig, activating_examples: list[TokenizedSample]) -> tuple[str, str]:
    """(system, user) prompts for the structured explainer."""
    has_z = any(ex.has_z_pattern_data() for ex in activating_examples)
    system = (
        "You study the internal features of a neural language model. A feature is a direction in the model's "
        "activations that fires on some tokens. You are shown text excerpts in which one feature fires; the tokens "
        f"on which it fires strongly are wrapped in << and >>. Below each excerpt the strongest tokens are listed again "
        "as `(preceding context) token`."
    )
    if has_z:
        system += (
            " This feature reads from earlier positions through attention: a line `[(ctx) source; ...] => (ctx) token` "
            "lists the earlier tokens that contribute most to the activation on `token`. Take into account what is "
            "being moved from the sources to the target."
        )
    system += (
        " Find the common property of the highlighted tokens: the token itself, what precedes it, what it predicts, "
        "or a broader theme. Prefer the simplest description that covers the examples; do not list the examples back.\n"
    )
    if cfg.include_cot:
        system += "Think step by step and record each step before you conclude.\n"
    else:
        system += "Do not spell out reasoning steps; give the conclusion directly.\n"
    system += _JSON_SCHEMA_NOTE
    blocks = []
    for ex in activating_examples:
        t = cfg.activation_threshold
        blocks.append(f"{ex.display_highlighted(t)}\nStrongest tokens:\n{ex.display_max(t)}")
    user = "These are the excerpts for the feature.\n\n" + _numbered(blocks) + "\nExplain the feature."
    return system, user


def generate_explanation_prompt_neuronpedia(cfg: AutoInterpConfig, activating_examples: list[TokenizedSample],
                                            top_logits: dict[str, list[dict[str, Any]]] | None = None) -> tuple[str, str]:  # fmt: skip
    """(system, user) prompts for the terse explainer: the answer is a short phrase, no JSON."""
    system = (
        "You label features of a neural language model for a public feature browser. For one feature you get: the "
        "tokens on which it fires most (with a little preceding context), the tokens that follow them, and optionally "
        "the vocabulary items whose logits the feature raises most. Reply with a label of at most about ten words, "
        "lower case, no full sentence, no quotation marks, no preamble such as 'this feature'. If the firing tokens "
        "share an obvious surface form, name it; if instead the feature is best described by what it predicts next, "
        "say `predicts ...`; otherwise name the shared topic."
    )
    t = cfg.activation_threshold
    parts = []
    max_tokens = "".join(ex.display_max(t) for ex in activating_examples)
    parts.append("Firing tokens, as (context) token:\n" + max_tokens)
    nxt = "".join(ex.display_next(t) for ex in activating_examples)
    if nxt:
        parts.append("Tokens that follow a firing token:\n" + nxt)
    if top_logits is not None and top_logits.get("top_positive"):
        parts.append("Most promoted output tokens:\n" + "\n".join(str(e["token"]) for e in top_logits["top_positive"]))
    return system, "\n".join(parts) + "\nLabel:"
