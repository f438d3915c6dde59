"""Cross-layer transcoder (CLT): L encoders, and a decoder from every source layer to every later target layer.

Behaviour follows models/clt.py of the reference project: config (:67-120); parameters ``W_E [L, d, F]``,
``b_E [L, F]``, ``W_D.<t> [t+1, F, d]``, ``b_D.<t> [d]`` (:157-178); activation functions ``relu``,
``jumprelu`` (threshold ``[L, F]``), ``topk`` (per token and layer), ``layertopk`` (per token over layers x
features, k entries), ``batchtopk`` (per layer over batch x features, k*batch entries), ``batchlayertopk``
(over everything, k*batch entries) (:232-387); initialisation bounds (:389-466); encode (:526-573);
``y_t = sum_{s<=t} a_s W_D[t][s] + b_D[t]`` (:629-709) with dense, CSR and COO decoding (:711-798);
``decoder_norm()`` returning ones and the real per-feature norm ``sqrt(sum_t ||W_D[t][s, f]||^2)`` (:801-876);
dataset-norm folding (:907-937); own loss without Aux-K / Lp (:1023-1104).

Under feature (``model``) parallelism the contributions of all target layers are stacked first and reduced
across shards with ONE all-reduce (the reference issues one per target layer).
"""

from __future__ import annotations

import math
from typing import Any, Callable, Literal

import torch
import torch.distributed as dist
from torch import nn

from ..activation_functions import JumpReLU
from ..parallel.collectives import all_reduce_sum, distributed_topk
from ..parallel.mesh import DeviceMesh, DimMap
from ..ops.select_kernels import positive_topk
from ..utils.math import topk
from ..utils.tensor_specs import TensorSpecs
from ..utils.timer import timer
from .sae import shard_generator
from .sparse_dictionary import SparseDictionary, SparseDictionaryConfig, register_sae_config, register_sae_model


class CrossLayerTranscoderSpecs(TensorSpecs):
    @staticmethod
    def feature_acts(tensor: torch.Tensor) -> tuple[str, ...]:
        return {3: ("batch", "layers", "sae"), 4: ("batch", "context", "layers", "sae")}[tensor.ndim]

    @staticmethod
    def reconstructed(tensor: torch.Tensor) -> tuple[str, ...]:
        return {3: ("layers", "batch", "model"), 4: ("layers", "batch", "context", "model")}[tensor.ndim]

    @staticmethod
    def label(tensor: torch.Tensor) -> tuple[str, ...]:
        return CrossLayerTranscoderSpecs.reconstructed(tensor)

    @staticmethod
    def loss(tensor: torch.Tensor) -> tuple[str, ...]:
        return {2: ("layers", "batch"), 3: ("layers", "batch", "context")}[tensor.ndim]


@register_sae_config("clt")
class CLTConfig(SparseDictionaryConfig):
    sae_type: str = "clt"
    act_fn: Literal["relu", "jumprelu", "topk", "batchtopk", "batchlayertopk", "layertopk"] = "relu"
    init_cross_layer_decoder_all_zero: bool = False
    hook_points_in: list[str]
    hook_points_out: list[str]
    decode_with_csr: bool = False
    sparsity_threshold_for_csr: float = 0.05

    @property
    def n_layers(self) -> int:
        return len(self.hook_points_in)

    @property
    def n_decoders(self) -> int:
        return self.n_layers * (self.n_layers + 1) // 2

    @property
    def associated_hook_points(self) -> list[str]:
        return self.hook_points_in + self.hook_points_out

    @property
    def hooks_in(self) -> list[str]:
        return self.hook_points_in

    @property
    def hooks_out(self) -> list[str]:
        return self.hook_points_out

    def model_post_init(self, __context):
        super().model_post_init(__context)
        assert len(self.hook_points_in) == len(self.hook_points_out), "Number of input and output hook points must match"


@register_sae_model("clt")
class CrossLayerTranscoder(SparseDictionary):
    specs: type[TensorSpecs] = CrossLayerTranscoderSpecs

    def __init__(self, cfg: CLTConfig, device_mesh: DeviceMesh | None = None):
        super().__init__(cfg, device_mesh)
        self.cfg: CLTConfig = cfg
        L, d, F = cfg.n_layers, cfg.d_model, cfg.d_sae
        (F_l,) = DimMap({"model": 0}).local_shape((F,), device_mesh)
        self.d_sae_local = F_l
        dev, dt = cfg.device, cfg.dtype
        self.W_E = nn.Parameter(torch.empty(L, F_l, d, device=dev, dtype=dt).transpose(1, 2))
        self.b_E = nn.Parameter(torch.empty(L, F_l, device=dev, dtype=dt))
        self.W_D = nn.ParameterList([nn.Parameter(torch.empty(t + 1, F_l, d, device=dev, dtype=dt)) for t in range(L)])
        self.b_D = nn.ParameterList([nn.Parameter(torch.empty(d, device=dev, dtype=dt)) for _ in range(L)])
        self.decoders_for_layer_from: tuple[int, list[torch.Tensor]] | None = None
        self.setup()

    def dim_maps(self) -> dict[str, DimMap]:
        maps: dict[str, DimMap] = {"W_E": DimMap({"model": 2}), "b_E": DimMap({"model": 1}), "decoder_norms": DimMap({"model": 1})}
        for t in range(self.cfg.n_layers):
            maps[f"W_D.{t}"] = DimMap({"model": 1})
            maps[f"b_D.{t}"] = DimMap({})
        maps["W_D"] = DimMap({"model": 1})
        maps["b_D"] = DimMap({})
        return super().dim_maps() | maps

    # ---- activation functions ----------------------------------------------------------------
    def activation_function_factory(self, device_mesh: DeviceMesh | None = None) -> Callable[[torch.Tensor], torch.Tensor]:
        act = self.cfg.act_fn.lower()
        if act == "relu":
            return lambda x: x * x.gt(0).to(x.dtype)
        if act == "jumprelu":
            return JumpReLU(self.cfg.jumprelu_threshold_window, shape=(self.cfg.n_layers, self.cfg.d_sae),
                            dims_to_keep_in_bwd=(-2, -1), device=self.cfg.device, dtype=self.cfg.dtype,
                            device_mesh=device_mesh)  # fmt: skip
        # (dims searched over, number kept as a function of the batch size)
        table = {
            "topk": ((-1,), lambda b: self.current_k),
            "layertopk": ((-2, -1), lambda b: self.current_k),
            "batchtopk": (None, lambda b: self.current_k * b),  # all token dims + features, per layer
            "batchlayertopk": ("all", lambda b: self.current_k * b),
        }
        if act not in table:
            raise ValueError(f"Not implemented activation function {self.cfg.act_fn}")
        dims_spec, count = table[act]

        def select(x: torch.Tensor) -> torch.Tensor:
            x = x * x.gt(0).to(x.dtype)
            n_tokens = x[..., 0, 0].numel()
            if dims_spec is None:
                dims = tuple(range(x.ndim - 2)) + (x.ndim - 1,)
            elif dims_spec == "all":
                dims = tuple(range(x.ndim - 2)) + (x.ndim - 2, x.ndim - 1)
            else:
                dims = tuple(d % x.ndim for d in dims_spec)
            k = count(n_tokens)
            if len(dims) > 1:  # batch-level selections: radix-select threshold on a GPU
                out = positive_topk(x, k, dims, self.tp_group if self.tp_size > 1 else None)
                if out is not None:
                    return out
            if self.tp_size > 1:
                return distributed_topk(x, k, self.tp_group, dim=dims)
            n_sel = 1
            for d_ in dims:
                n_sel *= x.shape[d_]
            return topk(x, k=min(k, n_sel), dim=dims)

        return select

    # ---- initialisation ----------------------------------------------------------------------
    @torch.no_grad()
    def init_parameters(self, **kwargs):
        """Encoders ~ U(+-1/sqrt(d_sae)); decoders ~ U(+-1/sqrt(L d_model)); biases zero."""
        super().init_parameters(**kwargs)
        g = shard_generator(self.device_mesh, self.b_E.device)
        eb = 1.0 / math.sqrt(self.cfg.d_sae)
        db = 1.0 / math.sqrt(self.cfg.n_layers * self.cfg.d_model)
        self.W_E.transpose(1, 2).uniform_(-eb, eb, generator=g)
        self.b_E.zero_()
        for t, w in enumerate(self.W_D):
            w.uniform_(-db, db, generator=g)
            if self.cfg.init_cross_layer_decoder_all_zero:
                w[:-1] = 0
            self.b_D[t].zero_()

    @torch.no_grad()
    def init_encoder_bias_with_mean_hidden_pre(self, batch: dict[str, torch.Tensor]):
        x = self.prepare_input(batch)[0]
        _, hidden_pre = self.encode(x, return_hidden_pre=True)
        mean = hidden_pre.reshape(-1, *hidden_pre.shape[-2:]).mean(dim=0)
        if self.dp_size > 1:
            dist.all_reduce(mean, group=self.dp_group)
            mean /= self.dp_size
        self.b_E.sub_(mean)

    # ---- norms -------------------------------------------------------------------------------
    def decoder_norm(self, keepdim: bool = False):
        """Ones, by design of the reference: gating and penalties use ``decoder_norm_per_feature``."""
        return torch.ones(self.cfg.n_decoders, device=self.b_E.device, dtype=self.cfg.dtype)

    def encoder_norm(self, keepdim: bool = False):
        return torch.norm(self.W_E, p=2, dim=1, keepdim=keepdim)

    def decoder_bias_norm(self):
        return torch.ones(self.cfg.n_layers, device=self.b_E.device, dtype=self.cfg.dtype)

    @torch.no_grad()
    def keep_only_decoders_for_layer_from(self, layer_from: int):
        """Cache the decoder slices leaving ``layer_from`` (single-layer analysis)."""
        self.decoders_for_layer_from = (layer_from, [w[layer_from] for t, w in enumerate(self.W_D) if t >= layer_from])

    @torch.no_grad()
    def decoder_norm_per_feature(self, layer: int | None = None) -> torch.Tensor:
        """``[L, F_l]``: for source layer s and feature f, the norm over all its target layers of the decoder
        rows, ``sqrt(sum_{t>=s} ||W_D[t][s, f, :]||^2)``. With ``layer`` given: row t holds
        ``||W_D[t][layer, f, :]||`` for t >= layer (zeros elsewhere)."""
        out = torch.zeros(self.cfg.n_layers, self.d_sae_local, dtype=self.cfg.dtype, device=self.b_E.device)
        if layer is not None:
            if self.decoders_for_layer_from is not None:
                kept_from, kept = self.decoders_for_layer_from
                assert kept_from == layer
                for off, w in enumerate(kept):
                    out[layer + off] = w.pow(2).sum(dim=-1).sqrt()
            else:
                for t in range(layer, self.cfg.n_layers):
                    out[t] = self.W_D[t][layer].pow(2).sum(dim=-1).sqrt()
            return out
        for t, w in enumerate(self.W_D):
            out[: t + 1] += w.pow(2).sum(dim=-1)
        return out.sqrt()

    @torch.no_grad()
    def decoder_norm_per_decoder(self) -> torch.Tensor:
        """``[n_decoders]`` mean row norm of each (source -> target) decoder, in (target, source) order."""
        vals = [w[s].pow(2).sum(dim=-1).sqrt().mean() for w in self.W_D for s in range(w.shape[0])]
        out = torch.stack(vals)
        if self.tp_size > 1:
            dist.all_reduce(out, group=self.tp_group)
            out /= self.tp_size
        return out

    @torch.no_grad()
    def standardize_parameters_of_dataset_norm(self):
        assert self.cfg.norm_activation == "dataset-wise" and self.dataset_average_activation_norm is not None
        norms = self.dataset_average_activation_norm
        root = math.sqrt(self.cfg.d_model)
        f_in = [root / norms[hp] for hp in self.cfg.hook_points_in]
        f_out = [root / norms[hp] for hp in self.cfg.hook_points_out]
        for s in range(self.cfg.n_layers):
            self.b_E.data[s].div_(f_in[s])
            if isinstance(self.activation_function, JumpReLU):
                self.activation_function.log_jumprelu_threshold.data[s] -= math.log(f_in[s])
        for t in range(self.cfg.n_layers):
            self.b_D[t].data.div_(f_out[t])
            for s in range(t + 1):
                self.W_D[t].data[s].mul_(f_in[s] / f_out[t])
        self.cfg.norm_activation = "inference"

    # ---- forward -----------------------------------------------------------------------------
    def encode(self, x: torch.Tensor, return_hidden_pre: bool = False, **kwargs):
        """``x [..., L, d]`` -> feature activations ``[..., L, F_l]``."""
        with timer.time("encoder_matmul"):
            hidden_pre = torch.einsum("...ld,lds->...ls", x.to(self.W_E.dtype), self.W_E) + self.b_E
        gate = self.decoder_norm_per_feature() if self.cfg.sparsity_include_decoder_norm else None
        if gate is not None:
            hidden_pre = hidden_pre * gate
        with timer.time("activation_function"):
            feature_acts = self.activation_function(hidden_pre)
        if gate is not None:
            feature_acts = feature_acts / gate
        return (feature_acts, hidden_pre) if return_hidden_pre else feature_acts

    def encode_single_layer(self, x: torch.Tensor, layer: int, return_hidden_pre: bool = False, **kwargs):
        """Features of one source layer from that layer's input ``[..., d]`` (analysis path)."""
        hidden_pre = x.to(self.W_E.dtype) @ self.W_E[layer] + self.b_E[layer]
        if self.cfg.sparsity_include_decoder_norm:
            hidden_pre = hidden_pre * self.decoder_norm_per_feature(layer=layer)[layer:].pow(2).sum(0).sqrt()
        if isinstance(self.activation_function, JumpReLU):
            thr = self.activation_function.get_jumprelu_threshold()[layer]
            feature_acts = hidden_pre * hidden_pre.gt(thr)
        else:
            feature_acts = self.activation_function(hidden_pre.unsqueeze(-2)).squeeze(-2)
        return (feature_acts, hidden_pre) if return_hidden_pre else feature_acts

    def get_decoder_weights(self, layer_to: int) -> torch.Tensor:
        return self.W_D[layer_to]

    def _contribution(self, feature_acts, layer_to: int) -> torch.Tensor:
        """``sum_{s<=t} a_s @ W_D[t][s]`` for one target layer, without bias or cross-shard reduction."""
        w = self.W_D[layer_to]
        if isinstance(feature_acts, (list, tuple)):  # one sparse [tokens, F] matrix per source layer
            out = None
            for s in range(layer_to + 1):
                c = torch.sparse.mm(feature_acts[s].to(torch.float32), w[s].to(torch.float32))
                out = c if out is None else out + c
            return out.to(self.cfg.dtype)
        a = feature_acts[..., : layer_to + 1, :]
        return torch.einsum("...lf,lfd->...d", a, w.to(a.dtype))

    def decode(self, feature_acts, batch_first: bool = False, **kwargs) -> torch.Tensor:
        """``[..., L, F_l]`` (or a list of L sparse matrices) -> ``[L, ..., d]`` (``batch_first``: ``[..., L, d]``)."""
        acts = feature_acts
        if not isinstance(acts, (list, tuple)) and self.cfg.decode_with_csr and (
            self.current_k / (self.cfg.d_sae * self.cfg.n_layers) < self.cfg.sparsity_threshold_for_csr
        ):
            # one gather kernel for every (source, target) pair instead of L (L + 1) / 2 CSR products
            from ..ops.clt_kernels import clt_sparse_decode

            partial = clt_sparse_decode(acts, list(self.W_D), None).to(acts.dtype)
        else:
            partial = torch.stack([self._contribution(acts, t) for t in range(self.cfg.n_layers)], dim=0)
        stacked = all_reduce_sum(partial, self.tp_group)
        stacked = stacked + torch.stack(list(self.b_D)).reshape(self.cfg.n_layers, *([1] * (stacked.ndim - 2)), -1)
        if batch_first:
            return stacked.movedim(0, -2)
        return stacked

    def prepare_input(self, batch: dict[str, torch.Tensor], **kwargs) -> tuple[torch.Tensor, dict[str, Any], dict[str, Any]]:
        missing = [hp for hp in self.cfg.hook_points_in if hp not in batch]
        if missing:
            raise ValueError(f"Missing hook point {missing[0]} in batch")
        return torch.stack([batch[hp] for hp in self.cfg.hook_points_in], dim=-2), {}, {}

    def prepare_input_single_layer(self, batch: dict[str, torch.Tensor], layer: int, **kwargs):
        hp = self.cfg.hook_points_in[layer]
        if hp not in batch:
            raise ValueError(f"Missing hook point {hp} in batch")
        return batch[hp], {}, {}

    def prepare_label(self, batch: dict[str, torch.Tensor], **kwargs) -> torch.Tensor:
        missing = [hp for hp in self.cfg.hook_points_out if hp not in batch]
        if missing:
            raise ValueError(f"Missing hook point {missing[0]} in batch")
        return torch.stack([batch[hp] for hp in self.cfg.hook_points_out], dim=0)

    @torch.no_grad()
    def compute_training_metrics(self, *, l0: torch.Tensor, explained_variance_legacy: torch.Tensor, **kwargs) -> dict[str, float]:
        out: dict[str, float] = {}
        ev = explained_variance_legacy.reshape(-1)
        if ev.numel() == self.cfg.n_layers:
            out.update({f"metrics/explained_variance_L{l}": float(ev[l]) for l in range(self.cfg.n_layers)})
        if l0.ndim >= 1 and l0.shape[-1] == self.cfg.n_layers:
            per_layer = l0.reshape(-1, self.cfg.n_layers).mean(0)
            n = max(int(kwargs.get("n_tokens", 1)), 1) if l0.ndim == 1 else 1
            out.update({f"metrics/l0_layer{l}": float(per_layer[l]) / n for l in range(self.cfg.n_layers)})
        return out

    # ---- loss --------------------------------------------------------------------------------
    @timer.time("compute_loss")
    def compute_loss(
        self,
        batch: dict[str, torch.Tensor],
        label: torch.Tensor | None = None,
        *,
        sparsity_loss_type: Literal["power", "tanh", "tanh-quad", None] = None,
        tanh_stretch_coefficient: float = 4.0,
        frequency_scale: float = 0.01,
        p: int = 1,
        l1_coefficient: float = 1.0,
        return_aux_data: bool = True,
        **kwargs,
    ):
        """MSE summed over d_model and averaged over layers and tokens, plus an optional sparsity penalty on
        ``feature_acts * decoder_norm_per_feature`` (no Aux-K / Lp terms for this model)."""
        x, ekw, dkw = self.prepare_input(batch)
        label = self.prepare_label(batch, **kwargs)
        with timer.time("encode"):
            feature_acts, hidden_pre = self.encode(x, return_hidden_pre=True, **ekw)
        with timer.time("decode"):
            reconstructed = self.decode(feature_acts, **dkw)
        l_rec = (reconstructed - label).pow(2).sum(dim=-1).mean()
        loss = l_rec
        l_s = None
        if sparsity_loss_type is not None:
            gated = feature_acts * self.decoder_norm_per_feature()
            if sparsity_loss_type == "power":
                l_s = self._sum_over_features(gated.abs().pow(p).sum(dim=-1)).pow(1.0 / p)
            elif sparsity_loss_type == "tanh":
                l_s = self._sum_over_features(torch.tanh(tanh_stretch_coefficient * gated).sum(dim=-1))
            elif sparsity_loss_type == "tanh-quad":
                freq = torch.tanh(tanh_stretch_coefficient * gated).reshape(-1, gated.shape[-1]).mean(0)
                l_s = self._sum_over_features((freq * (1 + freq / frequency_scale)).sum(dim=-1))
            else:
                raise ValueError(f"sparsity_loss_type {sparsity_loss_type} not supported.")
            l_s = l1_coefficient * l_s
            loss = loss + l_s.mean()
        if not return_aux_data:
            return loss
        mask = batch.get("mask")
        return {
            "loss": loss, "l_rec": l_rec, "l_s": l_s, "l_p": None, "l_aux": None, "label": label, "mask": mask,
            "n_tokens": batch["tokens"].numel() if mask is None else int(mask.sum()),
            "feature_acts": feature_acts, "reconstructed": reconstructed, "hidden_pre": hidden_pre,
            "l1_coefficient": l1_coefficient,
        }  # fmt: skip
