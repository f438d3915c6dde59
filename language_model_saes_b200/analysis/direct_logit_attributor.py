"""Direct logit attribution: push every decoder direction through the final norm and the unembedding, keep the
top / bottom tokens (analysis/direct_logit_attributor.py:15-164 of the reference project)."""

from __future__ import annotations

from functools import singledispatch

import torch

from ..backend.hooked_transformer import HookedTransformer
from ..backend.language_model import LanguageModel
from ..config import BaseConfig
from ..models.clt import CrossLayerTranscoder
from ..models.crosscoder import Crosscoder
from ..models.lorsa import LowRankSparseAttention
from ..models.sae import SparseAutoEncoder
from ..models.sparse_dictionary import SparseDictionary


class DirectLogitAttributorConfig(BaseConfig):
    top_k: int = 10
    clt_layer: int | None = None


def _logits_of_directions(directions: torch.Tensor, model: HookedTransformer, chunk: int = 8192) -> torch.Tensor:
    """``[n, d_model] -> [n, d_vocab]``, chunked over directions so that the fp32 logits of a large dictionary never
    exist at once next to the unembedding."""
    outs = []
    for part in directions.split(chunk):
        h = part[:, None, :].to(model.W_U.dtype)
        if model.cfg.normalization_type is not None:
            h = model.ln_final(h)
        outs.append((h @ model.W_U + model.b_U)[:, 0])
    return torch.cat(outs)


@singledispatch
def decoder_directions(sae, layer_idx: int | None = None) -> tuple[list[torch.Tensor], int]:
    """Directions whose logit effects are summed, and the number of features."""
    raise NotImplementedError(f"Unsupported SAE type: {type(sae)}")


@decoder_directions.register
def _(sae: SparseAutoEncoder, layer_idx: int | None = None):
    return [sae.W_D], sae.cfg.d_sae


@decoder_directions.register
def _(sae: Crosscoder, layer_idx: int | None = None):
    return [sae.W_D[-1]], sae.cfg.d_sae


@decoder_directions.register
def _(sae: LowRankSparseAttention, layer_idx: int | None = None):
    return [sae.W_O], sae.cfg.n_ov_heads


@decoder_directions.register
def _(sae: CrossLayerTranscoder, layer_idx: int | None = None):
    assert layer_idx is not None, "layer_idx is required for CrossLayerTranscoder"
    return [sae.W_D[i][layer_idx] for i in range(layer_idx, sae.cfg.n_layers)], sae.cfg.d_sae


class DirectLogitAttributor:
    def __init__(self, cfg: DirectLogitAttributorConfig):
        self.cfg = cfg

    @torch.no_grad()
    def direct_logit_attribute(self, sae: SparseDictionary, model: LanguageModel, layer_idx: int | None = None) -> list[dict]:
        assert isinstance(model, HookedTransformer), "DirectLogitAttributor needs the hooked-transformer backend"
        dirs, n = decoder_directions(sae, layer_idx if layer_idx is not None else self.cfg.clt_layer)
        k = self.cfg.top_k
        top_v, top_i, bot_v, bot_i = [], [], [], []
        # top-k per chunk of features: the [n, d_vocab] logits are reduced as they are produced
        for lo in range(0, n, 8192):
            logits = sum(_logits_of_directions(d[lo : lo + 8192], model) for d in dirs).float()
            tv, ti = logits.topk(k, dim=-1)
            bv, bi = logits.topk(k, dim=-1, largest=False)
            top_v.append(tv.cpu()), top_i.append(ti.cpu()), bot_v.append(bv.cpu()), bot_i.append(bi.cpu())
        top_v, top_i, bot_v, bot_i = (torch.cat(t) for t in (top_v, top_i, bot_v, bot_i))
        assert top_v.shape == (n, k), f"expected ({n}, {k}) top logits, got {tuple(top_v.shape)}"
        tok = model.tokenizer
        vocab: dict[int, str] = {}

        def s(i: int) -> str:
            if i not in vocab:
                vocab[i] = tok.decode([i]) if tok is not None else str(i)
            return vocab[i]

        return [
            {
                "top_positive": [{"token": s(i), "logit": v} for i, v in zip(top_i[f].tolist(), top_v[f].tolist())],
                "top_negative": [{"token": s(i), "logit": v} for i, v in zip(bot_i[f].tolist(), bot_v[f].tolist())],
            }
            for f in range(n)
        ]
