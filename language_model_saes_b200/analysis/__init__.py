"""Feature analysis: activation statistics and samples, direct logit attribution, automatic interpretation."""

from .direct_logit_attributor import DirectLogitAttributor, DirectLogitAttributorConfig
from .feature_analyzer import FeatureAnalyzer, FeatureAnalyzerConfig
from .samples import Segment, TokenizedSample, ZPatternSegment, process_token

__all__ = [
    "DirectLogitAttributor", "DirectLogitAttributorConfig", "FeatureAnalyzer", "FeatureAnalyzerConfig",
    "Segment", "TokenizedSample", "ZPatternSegment", "process_token",
]  # fmt: skip
