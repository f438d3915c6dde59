"""Per-dictionary-type post-processing of feature analyses; importing the package registers all processors."""

from .base import PostAnalysisProcessor, get_post_analysis_processor, register_post_analysis_processor
from .clt import CLTPostAnalysisProcessor
from .crosscoder import CrosscoderPostAnalysisProcessor
from .generic import GenericPostAnalysisProcessor
from .lorsa import LorsaPostAnalysisProcessor

__all__ = [
    "PostAnalysisProcessor", "get_post_analysis_processor", "register_post_analysis_processor",
    "CLTPostAnalysisProcessor", "CrosscoderPostAnalysisProcessor", "GenericPostAnalysisProcessor", "LorsaPostAnalysisProcessor",
]  # fmt: skip
