"""Language-model backends: the activation source of the whole framework.

Interface and behaviour follow backend/language_model.py of the reference project: ``LanguageModelConfig``
(:126-183, incl. ``lm_config.json`` save / load), the ``LanguageModel`` ABC (:186-242: ``trace``,
``to_activations``, ``preprocess_raw_data``, special token ids) and its backends — a hooked-transformer backend
(:245-579; here built on ``backend.hooked_transformer`` instead of TransformerLens), a HuggingFace backend that
reads residual streams from ``output_hidden_states`` and therefore only supports ``blocks.N.hook_resid_post``
(:582-643), a Qwen-VL backend with image tokens (:646-729) and a tokenizer-only backend (:732-892).
``mask = token != pad and token != bos`` (:396-397). Raw records may carry ``text`` or pre-tokenised ``tokens``.
"""

from __future__ import annotations

import json
import os
import re
from abc import ABC, abstractmethod
from typing import Any, Literal, Optional

import torch
import torch.distributed as dist

from ..config import BaseModelConfig
from ..parallel.mesh import mesh_dim_size, mesh_group
from ..utils.misc import pad_and_truncate_tokens
from .hooked_transformer import HookedTransformer, HookedTransformerConfig


def to_tokens(tokenizer, text, max_length: int, device="cpu", prepend_bos: bool = True) -> torch.Tensor:
    tokens = tokenizer(text, return_tensors="pt", padding=True, truncation=True, max_length=max_length)["input_ids"].to(device)
    bos = tokenizer.bos_token_id
    if bos is None:
        return tokens
    has = bool(torch.all(tokens[:, 0] == bos))
    if prepend_bos and not has:
        tokens = torch.cat([torch.full((tokens.shape[0], 1), bos, dtype=tokens.dtype, device=device), tokens], dim=1)
    elif not prepend_bos and has:
        tokens = tokens[:, 1:]
    return tokens


def set_tokens(tokenizer, bos_token_id, eos_token_id, pad_token_id):
    """Fill in missing special tokens (eos -> "<|endoftext|>", pad -> eos, bos -> eos unless ids are given)."""
    if tokenizer.eos_token is None:
        tokenizer.eos_token = "<|endoftext|>" if eos_token_id is None else tokenizer.decode(eos_token_id)
    if tokenizer.pad_token is None:
        tokenizer.pad_token = tokenizer.eos_token if pad_token_id is None else tokenizer.decode(pad_token_id)
    if tokenizer.bos_token is None:
        tokenizer.bos_token = tokenizer.eos_token if bos_token_id is None else tokenizer.decode(bos_token_id)
    return tokenizer


def _match_str_tokens_to_input(text: str, str_tokens: list[str]) -> list[Optional[dict[str, Any]]]:
    """Character range of every token string inside ``text`` (None for special / undecodable tokens)."""
    out: list[Optional[dict[str, Any]]] = []
    cur = 0
    for tok in str_tokens:
        pos = cur if text.startswith(tok, cur) else text.find(tok, cur)
        if pos != -1:
            out.append({"key": "text", "range": (pos, pos + len(tok))})
            cur = pos + len(tok)
        else:
            if not ((tok.startswith("<") and tok.endswith(">")) or "�" in tok):
                raise ValueError(f"Token {tok} not found in input text `{text}`")
            out.append(None)
    return out


def _get_layer_indices_from_hook_points(hook_points: list[str]) -> list[int]:
    ms = [re.match(r"^blocks\.(\d+)\.hook_resid_post$", hp) for hp in hook_points]
    assert all(m is not None for m in ms), "hook_points must be residual stream hook points"
    return [int(m.group(1)) for m in ms]  # type: ignore[union-attr]


class LanguageModelConfig(BaseModelConfig):
    model_name: str = "gpt2"
    model_from_pretrained_path: str | None = None
    cache_dir: str | None = None
    local_files_only: bool = False
    max_length: int = 2048
    backend: Literal["huggingface", "transformer_lens", "hooked", "tokenizer_only", "auto"] = "auto"
    prepend_bos: bool = True
    bos_token_id: int | None = None
    eos_token_id: int | None = None
    pad_token_id: int | None = None
    random_init: bool = False
    """Build the architecture from its config with random weights instead of loading a checkpoint."""

    @staticmethod
    def from_pretrained_sae(pretrained_name_or_path: str, **kwargs):
        """Read the ``lm_config.json`` stored next to a pretrained dictionary (local directory or hub)."""
        from ..models.sparse_dictionary import PretrainedSAEType, auto_infer_pretrained_sae_type

        kind = auto_infer_pretrained_sae_type(pretrained_name_or_path)
        if kind == PretrainedSAEType.LOCAL:
            path = os.path.join(pretrained_name_or_path, "lm_config.json")
            if not os.path.exists(path):
                path = os.path.join(os.path.dirname(pretrained_name_or_path), "lm_config.json")
        elif kind == PretrainedSAEType.HUGGINGFACE:
            from huggingface_hub import hf_hub_download

            repo_id, name = pretrained_name_or_path.split(":")
            path = hf_hub_download(repo_id=repo_id, filename=f"{name}/lm_config.json")
        else:
            from sae_lens.loading.pretrained_saes_directory import get_pretrained_saes_directory

            repo_id, _ = pretrained_name_or_path.split(":")
            return LanguageModelConfig(model_name=get_pretrained_saes_directory()[repo_id].model, **kwargs)
        with open(path, "r") as f:
            return LanguageModelConfig.model_validate({**json.load(f), **kwargs})

    def save_lm_config(self, sae_path: str):
        assert os.path.exists(sae_path), f"{sae_path} does not exist. Unable to save LanguageModelConfig."
        with open(os.path.join(sae_path, "lm_config.json"), "w") as f:
            json.dump(self.model_dump(), f, indent=4)


class LanguageModel(ABC):
    @abstractmethod
    def trace(self, raw: dict[str, Any], n_context: Optional[int] = None) -> list[list[Any]]:
        """Origin (``{"key", "range"}`` or None) of every token of every sample of ``raw``."""

    @abstractmethod
    def to_activations(self, raw: dict[str, Any], hook_points: list[str], n_context: Optional[int] = None) -> dict[str, torch.Tensor]:
        """Activations ``[batch, n_tokens, d]`` at the hook points, plus ``tokens``, ``mask``, ``attention_mask``."""

    @abstractmethod
    def preprocess_raw_data(self, raw: dict[str, Any]) -> dict[str, Any]: ...

    @property
    @abstractmethod
    def eos_token_id(self) -> int | None: ...

    @property
    @abstractmethod
    def bos_token_id(self) -> int | None: ...

    @property
    @abstractmethod
    def pad_token_id(self) -> int | None: ...


class _TokenizerMixin:
    tokenizer: Any
    lm_cfg: LanguageModelConfig

    @property
    def eos_token_id(self) -> int | None:
        return self.lm_cfg.eos_token_id if self.tokenizer is None else self.tokenizer.eos_token_id

    @property
    def bos_token_id(self) -> int | None:
        return self.lm_cfg.bos_token_id if self.tokenizer is None else self.tokenizer.bos_token_id

    @property
    def pad_token_id(self) -> int | None:
        return self.lm_cfg.pad_token_id if self.tokenizer is None else self.tokenizer.pad_token_id

    def preprocess_raw_data(self, raw: dict[str, Any]) -> dict[str, Any]:
        return raw

    def _tokens_of(self, raw: dict[str, Any], device) -> torch.Tensor:
        """Token ids of a batch of raw records: pre-tokenised ``tokens`` win over ``text``."""
        if "tokens" in raw:
            toks = raw["tokens"]
            if isinstance(toks, torch.Tensor):
                return toks.to(device)
            rows = [torch.as_tensor(t, dtype=torch.long) for t in toks]
            n = max(r.numel() for r in rows)
            pad = self.pad_token_id if self.pad_token_id is not None else 0
            return torch.stack([pad_and_truncate_tokens(r, n, pad) for r in rows]).to(device)
        assert self.tokenizer is not None, "text input needs a tokenizer"
        return to_tokens(self.tokenizer, raw["text"], max_length=self.lm_cfg.max_length, device=device, prepend_bos=self.lm_cfg.prepend_bos)

    def _common_context(self, tokens: torch.Tensor, n_context: Optional[int], device_mesh) -> torch.Tensor:
        """Pad / truncate to ``n_context``; under data parallelism without it, to the longest batch of the group."""
        if device_mesh is not None and n_context is None and mesh_dim_size(device_mesh, "data") > 1:
            g = mesh_group(device_mesh, "data")
            lens: list = [None] * dist.get_world_size(g)
            dist.all_gather_object(lens, tokens.shape[1], group=g)
            n_context = max(lens)
        if n_context is not None:
            pad = self.pad_token_id if self.pad_token_id is not None else 0
            tokens = pad_and_truncate_tokens(tokens, n_context, pad_token_id=pad)
        return tokens.contiguous()

    def _masks(self, tokens: torch.Tensor) -> torch.Tensor:
        keep = torch.ones_like(tokens, dtype=torch.bool)
        if self.pad_token_id is not None:
            keep &= tokens.ne(self.pad_token_id)
        if self.bos_token_id is not None:
            keep &= tokens.ne(self.bos_token_id)
        return keep.int()

    def trace(self, raw: dict[str, Any], n_context: Optional[int] = None) -> list[list[Any]]:
        assert self.tokenizer is not None
        enc = self.tokenizer(raw["text"], return_tensors="pt", padding=True, truncation=True,
                             max_length=self.lm_cfg.max_length, return_offsets_mapping=True)  # fmt: skip
        offsets = enc["offset_mapping"].tolist()
        tokens = enc["input_ids"]
        has = self.bos_token_id is not None and bool(torch.all(tokens[:, 0] == self.bos_token_id))
        if self.lm_cfg.prepend_bos and not has:
            offsets = [[None] + o for o in offsets]
        elif not self.lm_cfg.prepend_bos and has:
            offsets = [o[1:] for o in offsets]
        if n_context is not None:
            offsets = [(o[:n_context] + [None] * max(0, n_context - len(o))) for o in offsets]
        return [[{"key": "text", "range": tuple(o)} if o is not None else None for o in row] for row in offsets]


class HookedLanguageModel(_TokenizerMixin, HookedTransformer, LanguageModel):
    """Hooked-transformer backend: any hook point of ``backend.hooked_transformer`` can be read, the forward pass
    stops at the last requested hook, and the circuits code can splice dictionaries into it."""

    def __init__(self, cfg: LanguageModelConfig, device_mesh=None, *, architecture: HookedTransformerConfig | None = None, tokenizer=None):
        self.lm_cfg = cfg
        self.device_mesh = device_mesh
        device = f"cuda:{torch.cuda.current_device()}" if cfg.device == "cuda" else cfg.device
        self.device = torch.device(device)
        if architecture is not None:
            architecture.device, architecture.dtype = device, cfg.dtype
            HookedTransformer.__init__(self, architecture, tokenizer)
        else:
            from transformers import AutoConfig, AutoModelForCausalLM, AutoTokenizer

            src = cfg.model_from_pretrained_path or cfg.model_name
            if cfg.random_init:
                hf_cfg = AutoConfig.from_pretrained(src, cache_dir=cfg.cache_dir, local_files_only=cfg.local_files_only)
                HookedTransformer.__init__(self, self.config_from_hf(hf_cfg, device=device, dtype=cfg.dtype), None)
            else:
                hf = AutoModelForCausalLM.from_pretrained(src, cache_dir=cfg.cache_dir, local_files_only=cfg.local_files_only, dtype=cfg.dtype)
                HookedTransformer.__init__(self, self.config_from_hf(hf.config, device=device, dtype=cfg.dtype), None)
                self.load_hf_state_dict(hf.state_dict(), hf.config.model_type)
                del hf
            try:
                tokenizer = AutoTokenizer.from_pretrained(src, cache_dir=cfg.cache_dir, use_fast=True, local_files_only=cfg.local_files_only)
            except Exception:  # noqa: BLE001
                tokenizer = None
        self.tokenizer = set_tokens(tokenizer, cfg.bos_token_id, cfg.eos_token_id, cfg.pad_token_id) if tokenizer is not None else None
        self.eval()

    @classmethod
    def from_hooked_transformer(cls, model: HookedTransformer, device_mesh=None, **overrides: Any) -> "HookedLanguageModel":
        """Re-class an existing ``HookedTransformer``; config fields that cannot be inferred come from ``overrides``."""
        model.__class__ = cls
        tok = model.tokenizer
        inferred = dict(model_name=model.cfg.model_name, max_length=model.cfg.n_ctx, dtype=model.cfg.dtype,
                        device=str(next(model.parameters()).device),
                        bos_token_id=getattr(tok, "bos_token_id", None), eos_token_id=getattr(tok, "eos_token_id", None),
                        pad_token_id=getattr(tok, "pad_token_id", None))  # fmt: skip
        model.lm_cfg = LanguageModelConfig(**(inferred | overrides))
        model.device_mesh = device_mesh
        model.device = next(model.parameters()).device
        return model  # type: ignore[return-value]

    # ---- circuit tracing (the functions live in ``circuits``; the reference exposes them as model methods) ----
    def apply_saes(self, saes):
        """Context manager: splice sparse dictionaries into the forward pass (``circuits.hooks.apply_saes``)."""
        from ..circuits.hooks import apply_saes

        return apply_saes(self, saes)

    def detach_at(self, hook_points: list[str]):
        """Context manager: cut the autograd graph at hook points (``circuits.hooks.detach_at``)."""
        from ..circuits.hooks import detach_at

        return detach_at(self, hook_points)

    def attribute(self, inputs, replacement_modules, **kwargs):
        """Attribution graph of one prompt (``circuits.attribution.attribute``)."""
        from ..circuits.attribution import attribute

        return attribute(self, inputs, replacement_modules, **kwargs)

    def qk_trace(self, inputs, replacement_modules, lorsa_features, **kwargs):
        """QK tracing of attention-dictionary features (``circuits.attribution.qk_trace``)."""
        from ..circuits.attribution import qk_trace

        return qk_trace(self, inputs, replacement_modules, lorsa_features, **kwargs)

    @torch.no_grad()
    def to_activations(self, raw: dict[str, Any], hook_points: list[str], n_context: Optional[int] = None) -> dict[str, torch.Tensor]:
        tokens = self._common_context(self._tokens_of(raw, self.device), n_context, self.device_mesh)
        _, acts = self.run_with_cache_until(tokens, names_filter=hook_points, return_type=None)
        mask = self._masks(tokens)
        return {hp: acts[hp] for hp in hook_points} | {"tokens": tokens, "mask": mask, "attention_mask": mask.clone()}


TransformerLensLanguageModel = HookedLanguageModel


class HuggingFaceLanguageModel(_TokenizerMixin, LanguageModel):
    """Plain ``transformers`` model; residual streams are read from ``output_hidden_states`` (only
    ``blocks.N.hook_resid_post``). Returns no ``mask`` beyond pad / bos filtering."""

    def __init__(self, cfg: LanguageModelConfig, device_mesh=None, model=None, tokenizer=None):
        from transformers import AutoConfig, AutoModelForCausalLM, AutoTokenizer

        self.lm_cfg = cfg
        self.device_mesh = device_mesh
        self.device = torch.device(f"cuda:{torch.cuda.current_device()}" if cfg.device == "cuda" else cfg.device)
        src = cfg.model_from_pretrained_path or cfg.model_name
        if model is None:
            if cfg.random_init:
                model = AutoModelForCausalLM.from_config(AutoConfig.from_pretrained(src, local_files_only=cfg.local_files_only))
            else:
                model = AutoModelForCausalLM.from_pretrained(src, cache_dir=cfg.cache_dir, local_files_only=cfg.local_files_only, dtype=cfg.dtype)
        self.model = model.to(self.device, cfg.dtype).eval()
        if tokenizer is None:
            try:
                tokenizer = AutoTokenizer.from_pretrained(src, cache_dir=cfg.cache_dir, local_files_only=cfg.local_files_only)
            except Exception:  # noqa: BLE001
                tokenizer = None
        self.tokenizer = set_tokens(tokenizer, cfg.bos_token_id, cfg.eos_token_id, cfg.pad_token_id) if tokenizer is not None else None

    @torch.no_grad()
    def to_activations(self, raw: dict[str, Any], hook_points: list[str], n_context: Optional[int] = None) -> dict[str, torch.Tensor]:
        layers = _get_layer_indices_from_hook_points(hook_points)
        tokens = self._common_context(self._tokens_of(raw, self.device), n_context, self.device_mesh)
        out = self.model(input_ids=tokens, output_hidden_states=True)
        mask = self._masks(tokens)
        return {hp: out.hidden_states[l + 1] for hp, l in zip(hook_points, layers)} | {
            "tokens": tokens, "mask": mask, "attention_mask": mask.clone()}  # fmt: skip


class QwenVLLanguageModel(HuggingFaceLanguageModel):
    """Qwen-VL style vision-language model: records may carry ``images``; image placeholder tokens are traced back
    to their image (``{"key": "image", "image_idx": i}``) instead of a text range."""

    def __init__(self, cfg: LanguageModelConfig, device_mesh=None, model=None, tokenizer=None, processor=None):
        super().__init__(cfg, device_mesh, model=model, tokenizer=tokenizer)
        if processor is None:
            from transformers import AutoProcessor

            processor = AutoProcessor.from_pretrained(cfg.model_from_pretrained_path or cfg.model_name, local_files_only=cfg.local_files_only)
        self.processor = processor
        self.image_token_id = getattr(getattr(self.model, "config", None), "image_token_id", None)

    def preprocess_raw_data(self, raw: dict[str, Any]) -> dict[str, Any]:
        if "images" not in raw:
            return raw
        text = [t if "<|image_pad|>" in t else "<|vision_start|><|image_pad|><|vision_end|>" * len(imgs) + t
                for t, imgs in zip(raw["text"], raw["images"])]  # fmt: skip
        return {**raw, "text": text}

    @torch.no_grad()
    def to_activations(self, raw: dict[str, Any], hook_points: list[str], n_context: Optional[int] = None) -> dict[str, torch.Tensor]:
        if "images" not in raw:
            return super().to_activations(raw, hook_points, n_context)
        layers = _get_layer_indices_from_hook_points(hook_points)
        images = [img for imgs in raw["images"] for img in imgs]
        enc = self.processor(text=raw["text"], images=images or None, return_tensors="pt", padding=True).to(self.device)
        out = self.model(**enc, output_hidden_states=True)
        tokens = enc["input_ids"]
        mask = self._masks(tokens)
        return {hp: out.hidden_states[l + 1] for hp, l in zip(hook_points, layers)} | {
            "tokens": tokens, "mask": mask, "attention_mask": enc["attention_mask"].int()}  # fmt: skip

    def trace(self, raw: dict[str, Any], n_context: Optional[int] = None) -> list[list[Any]]:
        if "images" not in raw:
            return super().trace(raw, n_context)
        images = [img for imgs in raw["images"] for img in imgs]
        enc = self.processor(text=raw["text"], images=images or None, return_tensors="pt", padding=True)
        out = []
        for row, text in zip(enc["input_ids"].tolist(), raw["text"]):
            strs = [self.tokenizer.decode([t]) for t in row]
            img_i, origins = -1, []
            text_pos = _match_str_tokens_to_input(text, [s for t, s in zip(row, strs) if t != self.image_token_id])
            it = iter(text_pos)
            prev_img = False
            for t in row:
                if t == self.image_token_id:
                    if not prev_img:
                        img_i += 1
                    origins.append({"key": "image", "image_idx": img_i})
                    prev_img = True
                else:
                    origins.append(next(it))
                    prev_img = False
            out.append(origins[:n_context] if n_context else origins)
        return out


class TokenizerOnlyLanguageModel(_TokenizerMixin, LanguageModel):
    """No weights: tokenisation and tracing only (used by the server / sample rendering without a GPU)."""

    def __init__(self, cfg: LanguageModelConfig, tokenizer=None):
        self.lm_cfg = cfg
        if tokenizer is None:
            from transformers import AutoTokenizer

            tokenizer = AutoTokenizer.from_pretrained(cfg.model_from_pretrained_path or cfg.model_name, cache_dir=cfg.cache_dir,
                                                      local_files_only=cfg.local_files_only)  # fmt: skip
        self.tokenizer = set_tokens(tokenizer, cfg.bos_token_id, cfg.eos_token_id, cfg.pad_token_id)

    def to_activations(self, raw, hook_points, n_context=None):
        raise NotImplementedError("TokenizerOnlyLanguageModel has no weights")

    def to_tokens(self, raw: dict[str, Any], prepend_bos: bool | None = None) -> torch.Tensor:
        return to_tokens(self.tokenizer, raw["text"], self.lm_cfg.max_length, prepend_bos=self.lm_cfg.prepend_bos if prepend_bos is None else prepend_bos)
