"""Configuration of automatic feature interpretation (analysis/autointerp/autointerp_base.py:14-60 of the reference
project: same fields and defaults)."""

from enum import Enum
from typing import Optional

from pydantic import Field

from ...config import BaseConfig


class ExplainerType(str, Enum):
    OPENAI = "openai"
    NEURONPEDIA = "neuronpedia"


class ScorerType(str, Enum):
    DETECTION = "detection"
    FUZZING = "fuzzing"
    GENERATION = "generation"
    SIMULATION = "simulation"


class AutoInterpConfig(BaseConfig):
    explainer_type: ExplainerType = ExplainerType.OPENAI
    openai_api_key: Optional[str] = None
    openai_model: str = "gpt-3.5-turbo"
    openai_base_url: Optional[str] = None
    openai_proxy: Optional[str] = None

    n_activating_examples: int = 7
    n_non_activating_examples: int = 20
    activation_threshold: float = 0.7
    """Tokens above this fraction of the feature's maximum activation are highlighted."""
    max_length: int = 50

    scorer_type: list[ScorerType] = Field(default_factory=lambda: [ScorerType.DETECTION, ScorerType.FUZZING])
    detection_n_examples: int = 5
    fuzzing_n_examples: int = 5
    fuzzing_decile_correct: int = 5
    fuzzing_decile_incorrect: int = 2

    include_cot: bool = True
    overwrite_existing: bool = False
