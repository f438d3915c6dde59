"""Crosscoders add per-feature decoder norms per head and the head-by-head cosine / inner-product matrices of the
decoder directions (analysis/post_analysis/crosscoder.py:21-131 of the reference project)."""

import torch

from ...models.crosscoder import Crosscoder
from ...parallel.dist_ops import Sharded, full_tensor
from .base import PostAnalysisProcessor, register_post_analysis_processor


class CrosscoderPostAnalysisProcessor(PostAnalysisProcessor):
    def _process_tensors(self, sae, act_times, n_analyzed_tokens, max_feature_acts, sample_result, mapper, device_mesh=None,
                         activation_factory=None, activation_factory_process_kwargs=None, clt_layer=None):  # fmt: skip
        assert isinstance(sae, Crosscoder), "CrosscoderPostAnalysisProcessor only supports Crosscoder SAE"
        w_d = sae.W_D.detach()  # [local heads, F_local, d]
        if sae.head_size > 1:
            w_d = full_tensor(Sharded(w_d, 0, sae.head_group))  # every head's rows of this feature shard
        norms = torch.linalg.vector_norm(w_d.float(), dim=-1)  # [heads, F_local]
        inner = torch.einsum("ifd,jfd->fij", w_d.float(), w_d.float())
        sims = inner / torch.einsum("if,jf->fij", norms, norms)
        n = len(act_times)
        assert norms.shape[-1] == n and sims.shape[0] == n and inner.shape[0] == n, (
            f"feature dimension mismatch: norms {tuple(norms.shape)}, similarities {tuple(sims.shape)}, expected {n} features"
        )
        norms, sims, inner = norms.float().cpu(), sims.float().cpu(), inner.float().cpu()
        return sample_result, [
            {
                "decoder_norms": norms[:, i].tolist(),
                "decoder_similarity_matrices": sims[i].tolist(),
                "decoder_inner_product_matrices": inner[i].tolist(),
            }
            for i in range(n)
        ]


register_post_analysis_processor("crosscoder", CrosscoderPostAnalysisProcessor)
