"""A decoder-only transformer with named hook points (own implementation, no transformer_lens dependency).

Hook names follow the convention the reference project's configs and circuits code address
(``blocks.{l}.hook_resid_pre | hook_resid_mid | hook_resid_post | hook_attn_out | hook_mlp_out``,
``blocks.{l}.ln1.hook_normalized | ln1.hook_scale`` (same for ``ln2``), ``blocks.{l}.attn.hook_q | hook_k | hook_v |
hook_z | hook_attn_scores | hook_pattern``, ``blocks.{l}.mlp.hook_pre | hook_post``, ``hook_embed``,
``ln_final.hook_normalized``). Architectures: GPT-NeoX (parallel residual, partial rotary, LayerNorm), Llama /
Qwen (sequential, RMSNorm, gated MLP, grouped-query attention), GPT-2 (learned positions). Weights can be random
(``from_config``) or converted from a HuggingFace ``transformers`` model of those families (``from_hf``).

Also here: ``run_with_cache_until`` (stop the forward pass at the last requested hook; backend/tl_addons.py:28-89
of the reference), ``run_with_ref_cache`` (cache without detaching, :92-157) and ``mount_hooked_modules`` (:160-196).
"""

from __future__ import annotations

import math
from contextlib import contextmanager
from dataclasses import dataclass, field
from typing import Any, Literal, Sequence

import torch
import torch.nn.functional as F
from torch import nn

from ..hooks import HookedRootModule, HookPoint, NameFilter


@dataclass
class HookedTransformerConfig:
    n_layers: int
    d_model: int
    n_heads: int
    d_vocab: int
    n_ctx: int = 2048
    d_head: int | None = None
    d_mlp: int | None = None
    n_key_value_heads: int | None = None
    act_fn: Literal["gelu", "gelu_new", "silu", "relu"] = "gelu"
    normalization_type: Literal["LN", "RMS"] = "LN"
    positional_embedding_type: Literal["rotary", "standard", "none"] = "rotary"
    rotary_dim: int | None = None
    rotary_base: float = 10000.0
    rotary_adjacent_pairs: bool = False
    parallel_attn_mlp: bool = False
    gated_mlp: bool = False
    attn_bias: bool = True
    mlp_bias: bool = True
    eps: float = 1e-5
    use_qk_norm: bool = False
    tie_word_embeddings: bool = False
    init_std: float = 0.02
    device: str = "cpu"
    dtype: torch.dtype = torch.float32
    model_name: str = "custom"
    extra: dict[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        if self.d_head is None:
            self.d_head = self.d_model // self.n_heads
        if self.d_mlp is None:
            self.d_mlp = 4 * self.d_model
        if self.rotary_dim is None:
            self.rotary_dim = self.d_head


class StopAtHook(Exception):
    """Raised by the early-stop hook of ``run_with_cache_until``; carries nothing."""


class Norm(nn.Module):
    def __init__(self, cfg: HookedTransformerConfig, length: int | None = None):
        super().__init__()
        self.kind, self.eps = cfg.normalization_type, cfg.eps
        n = length or cfg.d_model
        self.w = nn.Parameter(torch.ones(n, device=cfg.device, dtype=cfg.dtype))
        self.b = nn.Parameter(torch.zeros(n, device=cfg.device, dtype=cfg.dtype)) if self.kind == "LN" else None
        self.hook_scale = HookPoint()
        self.hook_normalized = HookPoint()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        if self.kind == "LN":
            xf = xf - xf.mean(-1, keepdim=True)
        scale = self.hook_scale((xf.pow(2).mean(-1, keepdim=True) + self.eps).sqrt())
        out = self.hook_normalized((xf / scale).to(x.dtype))
        out = out * self.w
        return out + self.b if self.b is not None else out


class Attention(nn.Module):
    """Multi-head / grouped-query causal attention with per-head weight tensors
    ``W_Q [n_heads, d_model, d_head]``, ``W_K, W_V [n_kv_heads, d_model, d_head]``, ``W_O [n_heads, d_head, d_model]``."""

    def __init__(self, cfg: HookedTransformerConfig):
        super().__init__()
        self.cfg = cfg
        H, Hkv, d, dh = cfg.n_heads, cfg.n_key_value_heads or cfg.n_heads, cfg.d_model, cfg.d_head
        mk = lambda *s: nn.Parameter(torch.empty(*s, device=cfg.device, dtype=cfg.dtype))  # noqa: E731
        self.W_Q, self.W_K, self.W_V, self.W_O = mk(H, d, dh), mk(Hkv, d, dh), mk(Hkv, d, dh), mk(H, dh, d)
        self.b_Q, self.b_K, self.b_V, self.b_O = mk(H, dh), mk(Hkv, dh), mk(Hkv, dh), mk(d)
        if cfg.use_qk_norm:
            self.ln_q, self.ln_k = Norm(cfg, dh), Norm(cfg, dh)
        for name in ("q", "k", "v", "z", "attn_scores", "pattern", "result", "rot_q", "rot_k"):
            setattr(self, f"hook_{name}", HookPoint())
        if cfg.positional_embedding_type == "rotary":
            sin, cos = self._rotary_tables(cfg.rotary_dim, cfg.n_ctx, cfg.rotary_base)
            self.register_buffer("rotary_sin", sin, persistent=False)
            self.register_buffer("rotary_cos", cos, persistent=False)

    def _rotary_tables(self, rd: int, n_ctx: int, base: float):
        pos = torch.arange(n_ctx, dtype=torch.float32, device=self.cfg.device)
        freq = base ** (torch.arange(rd // 2, dtype=torch.float32, device=self.cfg.device) / (rd / 2))
        freq = freq.repeat_interleave(2) if self.cfg.rotary_adjacent_pairs else freq.repeat(2)
        ang = pos[:, None] / freq[None, :]
        return torch.sin(ang), torch.cos(ang)

    def _rotate(self, x: torch.Tensor, offset: int = 0) -> torch.Tensor:
        rd = self.cfg.rotary_dim
        xr, xp = x[..., :rd], x[..., rd:]
        n = x.size(1)
        cos = self.rotary_cos[None, offset : offset + n, None, :].to(x.dtype)
        sin = self.rotary_sin[None, offset : offset + n, None, :].to(x.dtype)
        if self.cfg.rotary_adjacent_pairs:
            flip = torch.stack((-xr[..., 1::2], xr[..., ::2]), dim=-1).flatten(-2)
        else:
            h = rd // 2
            flip = torch.cat((-xr[..., h:], xr[..., :h]), dim=-1)
        return torch.cat([xr * cos + flip * sin, xp], dim=-1)

    def qkv(self, q_in: torch.Tensor, k_in: torch.Tensor, v_in: torch.Tensor):
        q = self.hook_q(torch.einsum("bsd,hde->bshe", q_in, self.W_Q) + self.b_Q)
        k = self.hook_k(torch.einsum("bsd,hde->bshe", k_in, self.W_K) + self.b_K)
        v = self.hook_v(torch.einsum("bsd,hde->bshe", v_in, self.W_V) + self.b_V)
        if self.cfg.use_qk_norm:
            q, k = self.ln_q(q), self.ln_k(k)
        if self.cfg.positional_embedding_type == "rotary":
            q, k = self.hook_rot_q(self._rotate(q)), self.hook_rot_k(self._rotate(k))
        return q, k, v

    def _needs_pattern(self) -> bool:
        return bool(self.hook_attn_scores.fwd_hooks or self.hook_pattern.fwd_hooks or self.hook_attn_scores.bwd_hooks
                    or self.hook_pattern.bwd_hooks)  # fmt: skip

    def forward(self, query_input: torch.Tensor, key_input: torch.Tensor | None = None, value_input: torch.Tensor | None = None,
                attention_mask: torch.Tensor | None = None) -> torch.Tensor:  # fmt: skip
        key_input = query_input if key_input is None else key_input
        value_input = query_input if value_input is None else value_input
        q, k, v = self.qkv(query_input, key_input, value_input)
        H, Hkv = self.cfg.n_heads, k.size(2)
        if Hkv != H:
            k = k.repeat_interleave(H // Hkv, dim=2)
            v = v.repeat_interleave(H // Hkv, dim=2)
        q_, k_, v_ = (t.permute(0, 2, 1, 3) for t in (q, k, v))
        if self._needs_pattern() or attention_mask is not None:
            s = q_.size(-2)
            scores = q_ @ k_.transpose(-1, -2) / math.sqrt(self.cfg.d_head)
            causal = torch.tril(torch.ones(s, s, dtype=torch.bool, device=scores.device))
            if attention_mask is not None:
                causal = causal[None, None] & attention_mask[:, None, None, :].bool()
            scores = self.hook_attn_scores(scores.masked_fill(~causal, float("-inf")))
            pattern = self.hook_pattern(torch.nan_to_num(F.softmax(scores, dim=-1)))
            z = pattern.to(v_.dtype) @ v_
        else:
            z = F.scaled_dot_product_attention(q_, k_, v_, is_causal=True)
        z = self.hook_z(z.permute(0, 2, 1, 3))
        return torch.einsum("bshe,hed->bsd", z, self.W_O) + self.b_O

    @torch.no_grad()
    def head_outputs(self, x: torch.Tensor) -> torch.Tensor:
        """Per-head contribution to the output ``[batch, seq, n_heads, d_model]`` (no bias)."""
        q, k, v = self.qkv(x, x, x)
        H, Hkv = self.cfg.n_heads, k.size(2)
        if Hkv != H:
            k, v = k.repeat_interleave(H // Hkv, dim=2), v.repeat_interleave(H // Hkv, dim=2)
        z = F.scaled_dot_product_attention(q.permute(0, 2, 1, 3), k.permute(0, 2, 1, 3), v.permute(0, 2, 1, 3), is_causal=True)
        return torch.einsum("bhse,hed->bshd", z, self.W_O)


class MLP(nn.Module):
    def __init__(self, cfg: HookedTransformerConfig):
        super().__init__()
        self.cfg = cfg
        d, m = cfg.d_model, cfg.d_mlp
        mk = lambda *s: nn.Parameter(torch.empty(*s, device=cfg.device, dtype=cfg.dtype))  # noqa: E731
        self.W_in, self.b_in, self.W_out, self.b_out = mk(d, m), mk(m), mk(m, d), mk(d)
        if cfg.gated_mlp:
            self.W_gate = mk(d, m)
        self.hook_pre = HookPoint()
        self.hook_post = HookPoint()
        self.act = {"gelu": F.gelu, "gelu_new": lambda x: F.gelu(x, approximate="tanh"), "silu": F.silu, "relu": F.relu}[cfg.act_fn]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        pre = self.hook_pre(x @ self.W_in + self.b_in)
        if self.cfg.gated_mlp:
            post = self.hook_post(self.act(x @ self.W_gate) * pre)
        else:
            post = self.hook_post(self.act(pre))
        return post @ self.W_out + self.b_out


class TransformerBlock(nn.Module):
    def __init__(self, cfg: HookedTransformerConfig):
        super().__init__()
        self.cfg = cfg
        self.ln1, self.attn, self.ln2, self.mlp = Norm(cfg), Attention(cfg), Norm(cfg), MLP(cfg)
        for name in ("resid_pre", "resid_mid", "resid_post", "attn_in", "mlp_in", "attn_out", "mlp_out"):
            setattr(self, f"hook_{name}", HookPoint())

    def forward(self, resid: torch.Tensor, attention_mask: torch.Tensor | None = None) -> torch.Tensor:
        resid = self.hook_resid_pre(resid)
        attn_out = self.hook_attn_out(self.attn(self.ln1(self.hook_attn_in(resid)), attention_mask=attention_mask))
        if self.cfg.parallel_attn_mlp:
            mlp_out = self.hook_mlp_out(self.mlp(self.ln2(self.hook_mlp_in(resid))))
            return self.hook_resid_post(resid + attn_out + mlp_out)
        mid = self.hook_resid_mid(resid + attn_out)
        mlp_out = self.hook_mlp_out(self.mlp(self.ln2(self.hook_mlp_in(mid))))
        return self.hook_resid_post(mid + mlp_out)


class HookedTransformer(HookedRootModule):
    def __init__(self, cfg: HookedTransformerConfig, tokenizer=None):
        super().__init__()
        self.cfg = cfg
        self.tokenizer = tokenizer
        mk = lambda *s: nn.Parameter(torch.empty(*s, device=cfg.device, dtype=cfg.dtype))  # noqa: E731
        self.W_E = mk(cfg.d_vocab, cfg.d_model)
        if cfg.positional_embedding_type == "standard":
            self.W_pos = mk(cfg.n_ctx, cfg.d_model)
        self.hook_embed = HookPoint()
        self.hook_pos_embed = HookPoint()
        self.blocks = nn.ModuleList([TransformerBlock(cfg) for _ in range(cfg.n_layers)])
        self.ln_final = Norm(cfg)
        self.W_U = mk(cfg.d_model, cfg.d_vocab)
        self.b_U = mk(cfg.d_vocab)
        self.setup()
        self.init_weights()

    @classmethod
    def from_config(cls, cfg: HookedTransformerConfig, tokenizer=None, seed: int | None = None) -> "HookedTransformer":
        if seed is not None:
            torch.manual_seed(seed)
        return cls(cfg, tokenizer)

    @torch.no_grad()
    def init_weights(self) -> None:
        """N(0, init_std) for weight matrices, zeros for biases, ones for norm scales."""
        for name, p in self.named_parameters():
            leaf = name.rsplit(".", 1)[-1]
            if leaf == "w":
                p.fill_(1.0)
            elif leaf == "b" or leaf.startswith("b_"):
                p.zero_()
            elif p.ndim >= 2:
                p.normal_(0.0, self.cfg.init_std)
            else:
                p.zero_()

    # ---- accessors used by initialisers / attribution ---------------------------------------------
    def attention_module(self, layer: int) -> Attention:
        return self.blocks[layer].attn

    def mlp_module(self, layer: int) -> MLP:
        return self.blocks[layer].mlp

    # ---- forward -----------------------------------------------------------------------------
    def embed(self, tokens: torch.Tensor) -> torch.Tensor:
        x = self.hook_embed(self.W_E[tokens])
        if self.cfg.positional_embedding_type == "standard":
            x = x + self.hook_pos_embed(self.W_pos[: tokens.size(1)][None])
        return x

    def forward(self, tokens: torch.Tensor, return_type: str | None = "logits", loss_per_token: bool = False,
                attention_mask: torch.Tensor | None = None, start_at_layer: int | None = None,
                stop_at_layer: int | None = None):  # fmt: skip
        """``tokens [batch, pos]`` (or a residual stream when ``start_at_layer`` is given) -> logits / loss."""
        resid = tokens if start_at_layer is not None else self.embed(tokens)
        lo = start_at_layer or 0
        hi = self.cfg.n_layers if stop_at_layer is None else stop_at_layer
        for block in self.blocks[lo:hi]:
            resid = block(resid, attention_mask=attention_mask)
        if stop_at_layer is not None:
            return resid
        if return_type is None:
            return None
        logits = self.ln_final(resid) @ self.W_U + self.b_U
        if return_type == "logits":
            return logits
        logp = F.log_softmax(logits[:, :-1].float(), dim=-1)
        nll = -logp.gather(-1, tokens[:, 1:, None]).squeeze(-1)
        loss = nll if loss_per_token else nll.mean()
        return loss if return_type == "loss" else (logits, loss)

    def to_tokens(self, text, prepend_bos: bool | None = True, max_length: int | None = None) -> torch.Tensor:
        assert self.tokenizer is not None, "no tokenizer attached"
        enc = self.tokenizer(text, return_tensors="pt", padding=True, truncation=max_length is not None, max_length=max_length)
        toks = enc["input_ids"].to(self.W_E.device)
        bos = self.tokenizer.bos_token_id
        if bos is not None:
            has = bool((toks[:, 0] == bos).all())
            if prepend_bos and not has:
                toks = torch.cat([torch.full((toks.size(0), 1), bos, device=toks.device, dtype=toks.dtype), toks], dim=1)
            elif prepend_bos is False and has:
                toks = toks[:, 1:]
        return toks

    # ---- caching helpers -----------------------------------------------------------------------
    def run_with_cache_until(self, *args, names_filter: NameFilter = None, until: str | None = None, **kwargs):
        """Forward pass that caches the requested hooks and stops as soon as it can: right after ``until`` has fired
        when that is given, otherwise once every requested hook has fired (hook points are registered in the order the
        modules were defined, which is not the order they run in, so "the last one" is found by counting); later
        layers are never executed."""
        names = self._match(names_filter)
        cache: dict[str, torch.Tensor] = {}
        pending = set(names)

        def save(t, hook):
            cache[hook.name] = t.detach()
            pending.discard(hook.name)
            if until is None and not pending:
                raise StopAtHook

        def stop(t, hook):
            raise StopAtHook

        hooks = [(n, save) for n in names] + ([(until, stop)] if until is not None else [])
        out = None
        with self.hooks(fwd_hooks=hooks):
            try:
                out = self(*args, **kwargs)
            except StopAtHook:
                pass
        return out, cache

    def run_with_ref_cache(self, *args, names_filter: NameFilter = None, retain_grad: bool = False, **kwargs):
        """Like ``run_with_cache`` but the cached tensors stay attached to the autograd graph."""
        cache: dict[str, torch.Tensor] = {}

        def save(t, hook):
            if retain_grad and t.requires_grad:
                t.retain_grad()
            cache[hook.name] = t

        with self.hooks(fwd_hooks=[(n, save) for n in self._match(names_filter)]):
            out = self(*args, **kwargs)
        return out, cache

    @contextmanager
    def mount_hooked_modules(self, mounts: Sequence[tuple[str, str, nn.Module]]):
        """Temporarily attach extra modules (e.g. dictionaries) under existing hook-bearing modules so that their
        hook points become addressable as ``<parent>.<name>....``; ``mounts`` = (parent hook name, name, module)."""
        added = []
        try:
            for parent_name, name, module in mounts:
                parent = self.mod_dict[parent_name] if parent_name else self
                parent.add_module(name, module)
                added.append((parent, name))
            self.setup()
            yield self
        finally:
            for parent, name in added:
                delattr(parent, name)
            self.setup()

    # ---- conversion from HuggingFace checkpoints -----------------------------------------------
    @classmethod
    def config_from_hf(cls, hf_cfg, device: str = "cpu", dtype: torch.dtype = torch.float32) -> HookedTransformerConfig:
        mt = hf_cfg.model_type
        common = dict(n_layers=hf_cfg.num_hidden_layers, d_model=hf_cfg.hidden_size, n_heads=hf_cfg.num_attention_heads,
                      d_vocab=hf_cfg.vocab_size, n_ctx=getattr(hf_cfg, "max_position_embeddings", 2048), device=device,
                      dtype=dtype, model_name=getattr(hf_cfg, "_name_or_path", mt) or mt)  # fmt: skip
        if mt == "gpt_neox":
            dh = hf_cfg.hidden_size // hf_cfg.num_attention_heads
            return HookedTransformerConfig(**common, d_mlp=hf_cfg.intermediate_size, act_fn="gelu", normalization_type="LN",
                                           rotary_dim=int(dh * getattr(hf_cfg, "rotary_pct", 0.25)),
                                           rotary_base=getattr(hf_cfg, "rotary_emb_base", 10000.0),
                                           parallel_attn_mlp=getattr(hf_cfg, "use_parallel_residual", True),
                                           eps=hf_cfg.layer_norm_eps, init_std=getattr(hf_cfg, "initializer_range", 0.02))  # fmt: skip
        if mt in ("llama", "qwen2", "qwen3", "mistral"):
            return HookedTransformerConfig(**common, d_mlp=hf_cfg.intermediate_size, act_fn="silu", normalization_type="RMS",
                                           d_head=getattr(hf_cfg, "head_dim", None), n_key_value_heads=getattr(hf_cfg, "num_key_value_heads", None),
                                           rotary_base=getattr(hf_cfg, "rope_theta", 10000.0), gated_mlp=True, mlp_bias=False,
                                           attn_bias=mt == "qwen2", eps=hf_cfg.rms_norm_eps, use_qk_norm=mt == "qwen3",
                                           tie_word_embeddings=getattr(hf_cfg, "tie_word_embeddings", False),
                                           init_std=getattr(hf_cfg, "initializer_range", 0.02))  # fmt: skip
        if mt == "gpt2":
            return HookedTransformerConfig(n_layers=hf_cfg.n_layer, d_model=hf_cfg.n_embd, n_heads=hf_cfg.n_head, d_vocab=hf_cfg.vocab_size,
                                           n_ctx=hf_cfg.n_positions, act_fn="gelu_new", positional_embedding_type="standard",
                                           eps=hf_cfg.layer_norm_epsilon, device=device, dtype=dtype, model_name="gpt2",
                                           tie_word_embeddings=True, init_std=hf_cfg.initializer_range)  # fmt: skip
        raise ValueError(f"unsupported HuggingFace model type {mt!r}")

    @classmethod
    def from_hf(cls, hf_model, tokenizer=None, device: str = "cpu", dtype: torch.dtype = torch.float32) -> "HookedTransformer":
        cfg = cls.config_from_hf(hf_model.config, device=device, dtype=dtype)
        model = cls(cfg, tokenizer)
        model.load_hf_state_dict(hf_model.state_dict(), hf_model.config.model_type)
        return model

    @torch.no_grad()
    def load_hf_state_dict(self, sd: dict[str, torch.Tensor], model_type: str) -> None:
        cfg = self.cfg
        H, Hkv, dh, d = cfg.n_heads, cfg.n_key_value_heads or cfg.n_heads, cfg.d_head, cfg.d_model
        put = lambda p, t: p.copy_(t.to(p.dtype))  # noqa: E731
        for name, p in self.named_parameters():
            leaf = name.rsplit(".", 1)[-1]
            if leaf == "b" or leaf.startswith("b_"):
                p.zero_()
        if model_type == "gpt_neox":
            put(self.W_E, sd["gpt_neox.embed_in.weight"])
            for l, b in enumerate(self.blocks):
                pre = f"gpt_neox.layers.{l}."
                put(b.ln1.w, sd[pre + "input_layernorm.weight"]); put(b.ln1.b, sd[pre + "input_layernorm.bias"])
                put(b.ln2.w, sd[pre + "post_attention_layernorm.weight"]); put(b.ln2.b, sd[pre + "post_attention_layernorm.bias"])
                W = sd[pre + "attention.query_key_value.weight"].view(H, 3, dh, d)
                B = sd[pre + "attention.query_key_value.bias"].view(H, 3, dh)
                for i, (w_, b_) in enumerate(((b.attn.W_Q, b.attn.b_Q), (b.attn.W_K, b.attn.b_K), (b.attn.W_V, b.attn.b_V))):
                    put(w_, W[:, i].transpose(1, 2)); put(b_, B[:, i])
                put(b.attn.W_O, sd[pre + "attention.dense.weight"].T.reshape(H, dh, d)); put(b.attn.b_O, sd[pre + "attention.dense.bias"])
                put(b.mlp.W_in, sd[pre + "mlp.dense_h_to_4h.weight"].T); put(b.mlp.b_in, sd[pre + "mlp.dense_h_to_4h.bias"])
                put(b.mlp.W_out, sd[pre + "mlp.dense_4h_to_h.weight"].T); put(b.mlp.b_out, sd[pre + "mlp.dense_4h_to_h.bias"])
            put(self.ln_final.w, sd["gpt_neox.final_layer_norm.weight"]); put(self.ln_final.b, sd["gpt_neox.final_layer_norm.bias"])
            put(self.W_U, sd["embed_out.weight"].T)
        elif model_type in ("llama", "qwen2", "qwen3", "mistral"):
            put(self.W_E, sd["model.embed_tokens.weight"])
            for l, b in enumerate(self.blocks):
                pre = f"model.layers.{l}."
                put(b.ln1.w, sd[pre + "input_layernorm.weight"]); put(b.ln2.w, sd[pre + "post_attention_layernorm.weight"])
                put(b.attn.W_Q, sd[pre + "self_attn.q_proj.weight"].view(H, dh, d).transpose(1, 2))
                put(b.attn.W_K, sd[pre + "self_attn.k_proj.weight"].view(Hkv, dh, d).transpose(1, 2))
                put(b.attn.W_V, sd[pre + "self_attn.v_proj.weight"].view(Hkv, dh, d).transpose(1, 2))
                put(b.attn.W_O, sd[pre + "self_attn.o_proj.weight"].T.reshape(H, dh, d))
                for nm, tgt, n in (("q", b.attn.b_Q, H), ("k", b.attn.b_K, Hkv), ("v", b.attn.b_V, Hkv)):
                    key = pre + f"self_attn.{nm}_proj.bias"
                    if key in sd:
                        put(tgt, sd[key].view(n, dh))
                if cfg.use_qk_norm:
                    put(b.attn.ln_q.w, sd[pre + "self_attn.q_norm.weight"]); put(b.attn.ln_k.w, sd[pre + "self_attn.k_norm.weight"])
                put(b.mlp.W_in, sd[pre + "mlp.up_proj.weight"].T); put(b.mlp.W_gate, sd[pre + "mlp.gate_proj.weight"].T)
                put(b.mlp.W_out, sd[pre + "mlp.down_proj.weight"].T)
            put(self.ln_final.w, sd["model.norm.weight"])
            put(self.W_U, (sd["lm_head.weight"] if "lm_head.weight" in sd else sd["model.embed_tokens.weight"]).T)
        elif model_type == "gpt2":
            g = lambda k: sd[k] if k in sd else sd["transformer." + k]  # noqa: E731
            put(self.W_E, g("wte.weight")); put(self.W_pos, g("wpe.weight"))
            for l, b in enumerate(self.blocks):
                pre = f"h.{l}."
                put(b.ln1.w, g(pre + "ln_1.weight")); put(b.ln1.b, g(pre + "ln_1.bias"))
                put(b.ln2.w, g(pre + "ln_2.weight")); put(b.ln2.b, g(pre + "ln_2.bias"))
                W = g(pre + "attn.c_attn.weight").view(d, 3, H, dh)
                B = g(pre + "attn.c_attn.bias").view(3, H, dh)
                for i, (w_, b_) in enumerate(((b.attn.W_Q, b.attn.b_Q), (b.attn.W_K, b.attn.b_K), (b.attn.W_V, b.attn.b_V))):
                    put(w_, W[:, i].permute(1, 0, 2)); put(b_, B[i])
                put(b.attn.W_O, g(pre + "attn.c_proj.weight").view(H, dh, d)); put(b.attn.b_O, g(pre + "attn.c_proj.bias"))
                put(b.mlp.W_in, g(pre + "mlp.c_fc.weight")); put(b.mlp.b_in, g(pre + "mlp.c_fc.bias"))
                put(b.mlp.W_out, g(pre + "mlp.c_proj.weight")); put(b.mlp.b_out, g(pre + "mlp.c_proj.bias"))
            put(self.ln_final.w, g("ln_f.weight")); put(self.ln_final.b, g("ln_f.bias"))
            put(self.W_U, g("wte.weight").T)
        else:
            raise ValueError(f"unsupported HuggingFace model type {model_type!r}")


def pythia_shaped_config(size: Literal["70m", "160m"], device: str = "cpu", dtype: torch.dtype = torch.float32) -> HookedTransformerConfig:
    """Architectures of the Pythia models used by the benchmark configurations (random weights)."""
    dims = {"70m": (6, 512, 8), "160m": (12, 768, 12)}[size]
    return HookedTransformerConfig(n_layers=dims[0], d_model=dims[1], n_heads=dims[2], d_vocab=50304, n_ctx=2048, act_fn="gelu",
                                   normalization_type="LN", rotary_dim=(dims[1] // dims[2]) // 4, parallel_attn_mlp=True,
                                   device=device, dtype=dtype, model_name=f"pythia-{size}-shaped")  # fmt: skip
