"""Processor for dictionaries that add nothing to the common record (analysis/post_analysis/generic.py of the
reference project)."""

from .base import PostAnalysisProcessor, register_post_analysis_processor


class GenericPostAnalysisProcessor(PostAnalysisProcessor):
    pass


register_post_analysis_processor("sae", GenericPostAnalysisProcessor)
register_post_analysis_processor("generic", GenericPostAnalysisProcessor)
