"""Cross-layer transcoders add, per feature of the analysed source layer, the decoder norm towards every target
layer (analysis/post_analysis/clt.py:20-64 of the reference project)."""

from ...models.clt import CrossLayerTranscoder
from .base import PostAnalysisProcessor, register_post_analysis_processor


class CLTPostAnalysisProcessor(PostAnalysisProcessor):
    def _process_tensors(self, sae, act_times, n_analyzed_tokens, max_feature_acts, sample_result, mapper, device_mesh=None,
                         activation_factory=None, activation_factory_process_kwargs=None, clt_layer=None):  # fmt: skip
        assert isinstance(sae, CrossLayerTranscoder), "CLTPostAnalysisProcessor only supports CrossLayerTranscoder SAE"
        norms = sae.decoder_norm_per_feature(layer=clt_layer).float().cpu().numpy()  # [n_targets, F_local]
        return sample_result, [{"decoder_norms": norms[:, i]} for i in range(norms.shape[1])]


register_post_analysis_processor("clt", CLTPostAnalysisProcessor)
