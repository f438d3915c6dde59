"""Automatic interpretation of dictionary features with a chat model."""

from ..samples import Segment, TokenizedSample, process_token
from .autointerp_base import AutoInterpConfig, ExplainerType, ScorerType
from .evaluation_prompts import generate_detection_prompt, generate_fuzzing_prompt
from .explanation_prompts import generate_explanation_prompt, generate_explanation_prompt_neuronpedia
from .feature_interpreter import FeatureInterpreter

__all__ = [
    "generate_explanation_prompt", "generate_explanation_prompt_neuronpedia", "generate_detection_prompt", "generate_fuzzing_prompt",
    "FeatureInterpreter", "AutoInterpConfig", "ExplainerType", "ScorerType", "Segment", "TokenizedSample", "process_token",
]  # fmt: skip
