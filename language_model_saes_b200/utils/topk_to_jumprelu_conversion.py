"""Turn a (batch-)top-k cross-layer transcoder into a JumpReLU one with a single global threshold
(utils/topk_to_jumprelu_conversion.py:21-98 of the reference project).

The threshold is the smallest pre-activation that the batch-level top-``k * batch`` selection kept on one calibration
batch (over all layers and features, across feature shards). With ``sparsity_include_decoder_norm`` the threshold is
divided by each feature's decoder norm and the flag is cleared, so that encoding no longer needs the decoders.
"""

from __future__ import annotations

import math
from typing import Iterable

import torch

from ..activation_functions import JumpReLU
from ..models.clt import CrossLayerTranscoder
from ..models.sparse_dictionary import SparseDictionary
from ..parallel.collectives import distributed_threshold
from .logging import get_distributed_logger

logger = get_distributed_logger("utils.topk_to_jumprelu_conversion")


@torch.no_grad()
def topk_to_jumprelu_conversion(sae: SparseDictionary, activations_stream: Iterable[dict[str, torch.Tensor]], device_mesh=None) -> SparseDictionary:
    assert isinstance(sae, CrossLayerTranscoder), "Current implementation only supports CLT models"
    assert "topk" in sae.cfg.act_fn, "CLT model must use topk activation function"
    stream = iter(activations_stream)
    batch = sae.normalize_activations(next(stream))
    x, enc_kwargs, _ = sae.prepare_input(batch)
    _, hidden_pre = sae.encode(x, **enc_kwargs, return_hidden_pre=True)
    # (with ``sparsity_include_decoder_norm`` the encoder already returns the pre-activations times the decoder norms: the
    # values the selection ran on)
    score = hidden_pre.clamp(min=0.0).float()
    n_tokens = score[..., 0, 0].numel()
    k = sae.cfg.top_k * n_tokens
    # one row holding every (token, layer, local feature) score; the feature shard is the "last dim" of the selection
    threshold = float(distributed_threshold(score.reshape(1, -1), k, sae.tp_group if sae.tp_size > 1 else None).item())
    logger.info(f"Computed threshold: {threshold}")
    before = sae(x)

    sae.cfg.act_fn = "jumprelu"
    sae.activation_function = sae.activation_function_factory(device_mesh)
    assert isinstance(sae.activation_function, JumpReLU)
    log_thr = sae.activation_function.log_jumprelu_threshold.data
    if sae.cfg.sparsity_include_decoder_norm:
        log_thr.copy_((threshold / sae.decoder_norm_per_feature().float()).log().to(log_thr.dtype))
        sae.cfg.sparsity_include_decoder_norm = False
        logger.info("Also converting sparsity_include_decoder_norm to False so we do not need decoders to get encode results.")
    else:
        log_thr.fill_(math.log(threshold))
    after = sae(x)
    logger.info(f"Mean difference between original and converted reconstruction: {float((before - after).float().mean())}")

    val = next(stream, None)
    if val is not None:
        val = sae.normalize_activations(val)
        x, enc_kwargs, _ = sae.prepare_input(val)
        acts = sae.encode(x, **enc_kwargs)
        l0 = acts.gt(0).float().sum()
        if sae.tp_size > 1:
            torch.distributed.all_reduce(l0, group=sae.tp_group)
        logger.info(f"converted sae got L0 of {float(l0) / acts[..., 0, 0].numel()}, should be {sae.cfg.top_k}")
    return sae
