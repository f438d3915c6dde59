"""Attribution graphs for one prompt through a model whose activations are replaced by sparse dictionaries.

Algorithms follow circuits/attribution.py of the reference project (NodeRefs :46-142, intermediates attribution
:200-228, input x gradient scores :230-279, greedy collection :281-342, pruning :367-452, cache collection :455-533,
``attribute`` :536-780, QK tracing :803-942 / :1043-1183, Hessian :944-1010).

The central trick: the prompt is replicated ``batch_size`` times, non-linearities (feature activations, norms,
attention patterns) are cut out of the autograd graph, and for a batch of targets the scalar
``sum_j target_j[row j]`` is back-propagated once. Row ``j`` of every source gradient is then the gradient of target
``j`` alone, i.e. ``batch_size`` rows of the (linear) Jacobian per backward pass.
"""

from __future__ import annotations

import functools
import logging
from contextlib import nullcontext
from dataclasses import dataclass, field
from typing import Any, Iterator, Literal, Self, Sequence

import torch
from tqdm import tqdm

from ..backend.hooked_transformer import HookedTransformer
from ..core.pytree import PyTree
from ..core.serialize import migrate
from ..models.lorsa import LowRankSparseAttention
from ..models.sparse_dictionary import SparseDictionary
from ..utils.misc import ensure_tokenized
from ..utils.timer import timer
from .hooks import apply_saes, detach_at, replace_model_biases_with_leaves, replace_sae_biases_with_leaves
from .indexed_tensor import NodeDimension, NodeIndexed, NodeIndexedMatrix, NodeIndexedVector, NodeInfo

logger = logging.getLogger(__name__)


def _gather(ref: torch.Tensor, indices: torch.Tensor) -> torch.Tensor:
    """``ref[:, i0, i1, ...]`` for every row of ``indices`` -> ``[batch, n, ...]``."""
    return ref[(slice(None), *indices.unbind(dim=1))]


@dataclass
class NodeRefs:
    """Graph tensors (``mapping[key] [batch, ...]``, still attached to autograd) and the nodes taken from them."""

    mapping: dict[str, torch.Tensor]
    dimension: NodeDimension

    @classmethod
    def from_nodes_and_refs(cls, entries: Sequence[tuple[str, torch.Tensor, torch.Tensor]]) -> Self:
        """From ``(key, indices [n, d_index], ref)`` triples."""
        if len(entries) == 0:
            raise ValueError("Cannot build NodeRefs from empty entries without an explicit device.")
        return cls({k: ref for k, _, ref in entries}, NodeDimension.from_node_infos([NodeInfo(k, idx) for k, idx, _ in entries]))

    @property
    def device(self) -> torch.device:
        return next(iter(self.mapping.values())).device

    @property
    def dtype(self) -> torch.dtype:
        return next(iter(self.mapping.values())).dtype

    @property
    def device_mesh(self):
        return None

    @property
    def batch_size(self) -> int:
        return next(iter(self.mapping.values())).shape[0]

    def refs(self) -> list[torch.Tensor]:
        return list(self.mapping.values())

    @functools.cached_property
    def _entries(self) -> list[tuple[str, torch.Tensor, torch.Tensor]]:
        return [(ni.key, ni.indices, self.mapping[ni.key]) for ni in self.dimension.node_infos]

    @functools.cached_property
    def _identity(self) -> list[bool]:
        """Per slot: do the indices enumerate the whole ref (then gathering is the identity)?"""
        return [ni.is_identity and tuple(ref.shape[1 : 1 + ni.indices.shape[1]]) == tuple((ni.indices.max(0).values + 1).tolist())
                for ni, (_, _, ref) in zip(self.dimension.node_infos, self._entries)]  # fmt: skip

    @functools.cached_property
    def values(self) -> list[torch.Tensor]:
        """Per slot ``[batch, n_nodes, ...]``."""
        return [ref.flatten(1, idx.shape[1]) if full and idx.shape[1] > 1 else (ref if full else _gather(ref, idx))
                for (_, idx, ref), full in zip(self._entries, self._identity)]  # fmt: skip

    def iter_batches(self, batch_size: int) -> Iterator["NodeRefs"]:
        for lo in range(0, len(self.dimension), batch_size):
            off = torch.arange(lo, min(lo + batch_size, len(self.dimension)), device=self.dimension.device)
            yield self[self.dimension.offsets_to_nodes(off)]

    def __add__(self, other: "NodeRefs") -> "NodeRefs":
        return NodeRefs({**self.mapping, **other.mapping}, self.dimension + other.dimension)

    def __getitem__(self, index: NodeDimension) -> "NodeRefs":
        return NodeRefs({k: v for k, v in self.mapping.items() if k in index.keys}, index)

    def __iter__(self):
        return iter(self._entries)


@dataclass
class IntermediateRefs:
    """Feature nodes seen from both sides of the cut: ``upstream`` (pre-detach, a target of backward passes) and
    ``downstream`` (the fresh leaf, a source)."""

    upstream: NodeRefs
    downstream: NodeRefs


@dataclass
class QKTracingResult(PyTree):
    """Per attention feature: top sources through the query side, through the key side, and top (q source, k source)
    pairs of the bilinear attention score."""

    q_marginal: NodeIndexed[list[NodeIndexed[torch.Tensor]]]
    k_marginal: NodeIndexed[list[NodeIndexed[torch.Tensor]]]
    pairs: NodeIndexed[list[NodeIndexed[torch.Tensor]]]

    @migrate(before="2")
    @staticmethod
    def _v1_to_v2(data: dict[str, Any]) -> dict[str, Any]:
        """Version 1 stored only the pairs; marginals become zero vectors over the pair's nodes."""

        def size(dim_raw: dict[str, Any]) -> int:
            return sum(int(n["indices"].shape[0]) for n in dim_raw.values()) if dim_raw else 0

        q = [{"value": torch.zeros(size(s["dimensions"][0])), "dimensions": [s["dimensions"][0]]} for s in data["value"]]
        k = [{"value": torch.zeros(size(s["dimensions"][1])), "dimensions": [s["dimensions"][1]]} for s in data["value"]]
        return {"q_marginal": {"value": q, "dimensions": data["dimensions"]}, "k_marginal": {"value": k, "dimensions": data["dimensions"]}, "pairs": data}


@dataclass
class AttributionResult(PyTree):
    activations: NodeIndexedVector
    attribution: NodeIndexedMatrix
    targets: NodeDimension | None = None
    logits: torch.Tensor | None = None
    probs: torch.Tensor | None = None
    prompt_token_ids: list[int] = field(default_factory=list)
    prompt_tokens: list[str] = field(default_factory=list)
    logit_token_ids: list[int] | None = None
    logit_tokens: list[str] | None = None
    qk_trace_results: QKTracingResult | None = None


def get_normalized_matrix(matrix: NodeIndexedMatrix) -> NodeIndexedMatrix:
    """Rows of absolute values scaled to sum to 1."""
    a = matrix.data.abs()
    return NodeIndexedMatrix.from_data(a / a.sum(dim=1, keepdim=True).clamp(min=1e-8), matrix.dimensions)


@timer.time("compute_intermediates_attribution")
def compute_intermediates_attribution(attribution: NodeIndexedMatrix, targets: NodeDimension, intermediates: NodeDimension,
                                      max_iter: int) -> NodeIndexedMatrix:  # fmt: skip
    """Total (direct + through collected intermediates) normalised influence of every source on every target:
    ``T + T_i (I + A + A^2 + ...) I_all`` summed path length by path length until nothing is left to propagate."""
    attribution = get_normalized_matrix(attribution)
    influence = attribution[targets, None]
    if len(intermediates) == 0:
        return influence
    t2i = attribution[targets, intermediates]
    i2all = attribution[intermediates, None]
    i2i = attribution[intermediates, intermediates]
    for _ in range(max_iter):
        step = t2i @ i2all
        if not torch.any(step.data):
            break
        influence = influence + step
        t2i = t2i @ i2i
    return influence


@timer.time("attribution_scores")
def attribution_scores(grad_refs: Sequence[torch.Tensor | None], sources: NodeRefs) -> torch.Tensor:
    """Input x gradient summed over the non-node dimensions -> ``[batch, n_sources]``. ``grad_refs`` is aligned with
    ``sources.refs()`` (one gradient per distinct ref)."""
    grad_of = dict(zip(sources.mapping.keys(), grad_refs))
    parts = []
    for (key, idx, _), full, value in zip(sources._entries, sources._identity, sources.values):  # noqa: SLF001
        g = grad_of[key]
        if g is None:
            parts.append(value.new_zeros(value.shape[:2]))
            continue
        g = (g.flatten(1, idx.shape[1]) if idx.shape[1] > 1 else g) if full else _gather(g, idx)
        prod = value.detach() * g
        parts.append(prod.flatten(2).sum(-1) if prod.ndim > 2 else prod)
    return torch.cat(parts, dim=1) if len(parts) > 1 else parts[0]


@timer.time("greedily_collect_attribution")
def greedily_collect_attribution(targets: NodeRefs, sources: NodeRefs, intermediates: IntermediateRefs, max_intermediates: int,
                                 reduction_weight: torch.Tensor, max_iter: int = 100) -> tuple[NodeIndexedMatrix, NodeDimension]:  # fmt: skip
    """Rows for the targets first; then repeatedly pick the ``batch`` not-yet-collected feature nodes with the largest
    (weighted, path-summed) influence on the targets and add their rows."""
    all_sources = sources + intermediates.downstream
    attribution = NodeIndexedMatrix.from_dimensions((targets.dimension, all_sources.dimension), device=targets.device, dtype=targets.dtype)
    batch = targets.batch_size

    @timer.time("per_target_attribution")
    def rows_for(t: NodeRefs) -> torch.Tensor:
        stacked = torch.cat(t.values, dim=1)  # [batch, n_targets]
        n = stacked.shape[1]
        root = stacked[:n].diagonal()
        grads = torch.autograd.grad(root.sum(), all_sources.refs(), retain_graph=True, materialize_grads=True)
        return attribution_scores(grads, all_sources)[:n]

    for tb in targets.iter_batches(batch):
        attribution[tb.dimension, None] = rows_for(tb).to(attribution.data.dtype)

    collected = NodeDimension.empty(targets.device)
    weight = NodeIndexedVector.from_data(reduction_weight, (targets.dimension,))
    for i in tqdm(range(0, max_intermediates, batch), desc="OV Attribution"):
        n_pick = min(batch, max_intermediates - i, len(intermediates.downstream.dimension) - len(collected))
        if n_pick <= 0:
            break
        total = compute_intermediates_attribution(attribution, targets.dimension, collected, max_iter)
        influence = weight @ total[None, intermediates.downstream.dimension]
        _, picked = influence.topk(k=n_pick, ignore_dimension=collected)
        collected = collected + picked
        attribution.add_targets(picked, rows_for(intermediates.upstream[picked]).to(attribution.data.dtype))
    return attribution, collected


def ln_detach_hooks(model: HookedTransformer) -> list[str]:
    """Scale hook of every normalisation layer: with the scale frozen a norm is linear."""
    names = []
    for i, block in enumerate(model.blocks):
        for mod in ("ln1", "ln2", "ln1_post", "ln2_post"):
            if isinstance(getattr(block, mod, None), torch.nn.Module):
                names.append(f"blocks.{i}.{mod}.hook_scale")
    return names + ["ln_final.hook_scale"]


def attn_detach_hooks(model: HookedTransformer) -> list[str]:
    """Attention patterns (and QK-norm scales): with the pattern frozen attention is linear in the values."""
    names = []
    for i, block in enumerate(model.blocks):
        if isinstance(getattr(block, "attn", None), torch.nn.Module):
            names.append(f"blocks.{i}.attn.hook_pattern")
            if model.cfg.use_qk_norm:
                names += [f"blocks.{i}.attn.ln_q.hook_scale", f"blocks.{i}.attn.ln_k.hook_scale"]
    return names


def _find_influence_threshold(scores: torch.Tensor, threshold: float) -> torch.Tensor:
    """Smallest score among the largest ones that together hold ``threshold`` of the total."""
    if scores.numel() == 0:
        return torch.tensor(0.0, device=scores.device, dtype=scores.dtype)
    s = torch.sort(scores.reshape(-1), descending=True).values
    cum = torch.cumsum(s, 0) / s.sum().clamp(min=1e-8)
    i = min(int(torch.searchsorted(cum, torch.tensor(threshold, device=cum.device, dtype=cum.dtype))), s.numel() - 1)
    return s[i]


@timer.time("prune_attribution")
def prune_attribution(attribution: NodeIndexedMatrix, reduction_weight: torch.Tensor, node_threshold: float = 0.6,
                      edge_threshold: float = 0.8, targets: NodeDimension | None = None) -> NodeIndexedMatrix:  # fmt: skip
    """Zero the rows / columns of low-influence feature and error nodes and low-influence edges.

    Rows are targets (default: key ``"logits"``) followed by collected feature nodes; columns are embeddings, error
    nodes (keys ending in ``.error``) and feature nodes. Targets and embeddings always stay. A node stays if it is in
    the set holding ``node_threshold`` of the total influence AND still has a kept edge; edges likewise with
    ``edge_threshold``; iterated until stable.
    """
    if not 0.0 <= node_threshold <= 1.0:
        raise ValueError("node_threshold must be between 0.0 and 1.0")
    if not 0.0 <= edge_threshold <= 1.0:
        raise ValueError("edge_threshold must be between 0.0 and 1.0")
    rows, cols = attribution.dimensions
    if targets is None:
        targets = rows.filter_keys(lambda k: k == "logits")
    intermediates = rows - targets
    optional_sources = cols.filter_keys(lambda k: isinstance(k, str) and k.endswith(".error")) + intermediates
    weight = NodeIndexedVector.from_data(reduction_weight, (targets,))
    node_scores = weight @ compute_intermediates_attribution(attribution, targets, intermediates, max_iter=100)
    influence = node_scores[intermediates]
    influence.add_nodes(targets, reduction_weight.to(influence.data.dtype))
    edge_scores = NodeIndexedMatrix.from_data(get_normalized_matrix(attribution).data * influence[rows].data[:, None], attribution.dimensions)
    node_mask = node_scores.map(lambda x: x >= _find_influence_threshold(x, node_threshold))
    edge_mask = edge_scores.map(lambda x: x >= _find_influence_threshold(x, edge_threshold))

    def tighten():
        node_mask[optional_sources] = node_mask[optional_sources] & edge_mask[None, optional_sources].any(0)
        node_mask[intermediates] = node_mask[intermediates] & edge_mask[intermediates, None].any(1)

    before = node_mask.clone()
    tighten()
    while not torch.equal(node_mask.data, before.data):
        before = node_mask.clone()
        edge_mask.masked_fill_dim_(1, ~node_mask[optional_sources], False)
        edge_mask.masked_fill_dim_(0, ~node_mask[intermediates], False)
        tighten()
    out = attribution.clone()
    out.masked_fill_dim_(1, ~node_mask[optional_sources], 0)
    out.masked_fill_dim_(0, ~node_mask[intermediates], 0)
    out.masked_fill_(~edge_mask, 0)
    return out


@timer.time("collect_cache")
def collect_cache(model: HookedTransformer, tokens: torch.Tensor, replacement_modules: list[SparseDictionary], with_bias_leaves: bool = False):
    """One forward pass of ``tokens [batch, seq]`` with the dictionaries spliced in and every non-linearity cut;
    returns ``(logits, cache)`` where the cache holds graph-attached tensors: embeddings, error terms, feature
    activations before / after the cut, attention-dictionary scores and rotated q / k, norm scales and bias leaves."""
    assert tokens.ndim == 2, "tokens must be [batch, seq]"
    b, s = tokens.shape
    outs = [rm.cfg.hook_point_out for rm in replacement_modules]
    lorsas = [rm for rm in replacement_modules if isinstance(rm, LowRankSparseAttention)]
    model_bias_ctx = replace_model_biases_with_leaves(model, b, s) if with_bias_leaves else nullcontext([])
    sae_bias_ctx = replace_sae_biases_with_leaves(model, replacement_modules, b, s) if with_bias_leaves else nullcontext([])
    cut = (
        ["hook_embed"]
        + [o + ".error" for o in outs]
        + [o + ".sae.hook_feature_acts" for o in outs]
        + [rm.cfg.hook_point_out + ".sae.hook_attn_pattern" for rm in lorsas]
        + [rm.cfg.hook_point_out + sfx for rm in lorsas if rm.cfg.use_post_qk_ln for sfx in (".sae.ln_q.hook_scale", ".sae.ln_k.hook_scale")]
        + ln_detach_hooks(model)
        + attn_detach_hooks(model)
    )
    with model_bias_ctx as model_bias_names, apply_saes(model, replacement_modules), sae_bias_ctx as sae_bias_names, detach_at(model, cut):
        names = (
            ["hook_embed.post"]
            + [o + ".error.post" for o in outs]
            + [o + ".sae.hook_feature_acts.pre" for o in outs]
            + [o + ".sae.hook_feature_acts.post" for o in outs]
            + [rm.cfg.hook_point_out + sfx for rm in lorsas for sfx in (".sae.hook_attn_score", ".sae.hook_q_post_rot", ".sae.hook_k_post_rot")]
            + ln_detach_hooks(model)
            + list(model_bias_names)
            + list(sae_bias_names)
        )
        logits, cache = model.run_with_ref_cache(tokens, names_filter=names)
    return logits, cache


def _coerce_feature_dim(features: "list[tuple[str, int, int]] | NodeDimension", device) -> NodeDimension:
    if isinstance(features, NodeDimension):
        if len(features) == 0:
            raise ValueError("target_type='features' requires a non-empty NodeDimension")
        return features
    if len(features) == 0:
        raise ValueError("target_type='features' requires a non-empty features list")
    by_key: dict[str, list[tuple[int, int]]] = {}
    for key, pos, f in features:
        by_key.setdefault(key, []).append((int(pos), int(f)))
    return NodeDimension.from_node_infos([NodeInfo(k, torch.tensor(v, device=device, dtype=torch.long)) for k, v in by_key.items()], device=device)


def _bias_source_entries(model: HookedTransformer, replacement_modules, cache, seq_indices):
    keys = [f"blocks.{i}.{kind}" for i in range(len(model.blocks)) for kind in ("attn.hook_b_O", "mlp.hook_b_out")]
    keys += [rm.cfg.hook_point_out + sfx for rm in replacement_modules for sfx in (".sae.hook_b_Q", ".sae.hook_b_K", ".sae.hook_b_D")]
    return [(k, seq_indices, cache[k]) for k in keys if k in cache]


def _lorsa_tables(replacement_modules):
    lorsas = [rm for rm in replacement_modules if isinstance(rm, LowRankSparseAttention)]
    return {rm.cfg.hook_point_out: rm.cfg.ov_group_size for rm in lorsas}, {rm.cfg.hook_point_out: rm.attn_scale for rm in lorsas}


def _per_feature(result: QKTracingResult, slot_to_unique: list[int], features: NodeDimension) -> QKTracingResult:
    pick = lambda ni: NodeIndexed([ni.value[u] for u in slot_to_unique], (features,))  # noqa: E731
    return QKTracingResult(pick(result.q_marginal), pick(result.k_marginal), pick(result.pairs))


@timer.time("attribute")
def attribute(model: HookedTransformer, inputs: "torch.Tensor | str", replacement_modules: list[SparseDictionary],
              target_type: Literal["logits", "features"] = "logits", features: "list[tuple[str, int, int]] | NodeDimension" = (),
              max_n_logits: int = 10, desired_logit_prob: float = 0.95, batch_size: int = 512, max_features: int | None = None,
              enable_qk_tracing: bool = False, qk_top_fraction: float = 0.6, qk_topk: int = 10) -> AttributionResult:  # fmt: skip
    """Attribution graph of one prompt.

    Targets are either the top output logits at the last position (the smallest prefix of the ``max_n_logits`` most
    likely tokens whose probabilities reach ``desired_logit_prob``; each logit is taken relative to the mean logit) or
    given feature nodes ``(hook key, position, feature)``. Sources are token embeddings and the dictionaries' error
    terms at every position; active features are intermediates, of which the ``max_features`` most influential are
    collected greedily. ``batch_size`` is the number of prompt replicas = Jacobian rows per backward pass.
    """
    assert not enable_qk_tracing or batch_size >= qk_topk, f"attribute(batch_size={batch_size}) must be >= qk_topk={qk_topk} when enable_qk_tracing=True"
    dev = next(model.parameters()).device
    tokens = ensure_tokenized(inputs, model.tokenizer, device=dev)
    batch_logits, cache = collect_cache(model, tokens[None].expand(batch_size, -1), replacement_modules, with_bias_leaves=enable_qk_tracing)
    seq_len = cache["hook_embed.post"].shape[1]
    top_idx = top_p = None
    if target_type == "features":
        feat_dim = _coerce_feature_dim(features, dev)
        targets = NodeRefs.from_nodes_and_refs([(ni.key, ni.indices, cache[ni.key + ".pre"]) for ni in feat_dim.node_infos])
        reduction_weight = torch.ones(len(feat_dim), device=dev, dtype=targets.dtype)
    elif target_type == "logits":
        with torch.no_grad():
            probs = torch.softmax(batch_logits[0, -1].float(), dim=-1)
            top_p, top_idx = torch.topk(probs, min(max_n_logits, probs.numel()))
            cutoff = int(torch.searchsorted(torch.cumsum(top_p, 0), torch.tensor(desired_logit_prob, device=dev))) + 1
            top_p, top_idx = top_p[:cutoff], top_idx[:cutoff]
        last = batch_logits[:, -1, :]
        targets = NodeRefs.from_nodes_and_refs([("logits", top_idx[:, None], last - last.mean(dim=-1, keepdim=True))])
        reduction_weight = top_p.to(targets.dtype)
    else:
        raise ValueError(f"invalid target_type={target_type!r}")

    seq_indices = torch.arange(seq_len, device=dev)[:, None]
    outs = [rm.cfg.hook_point_out for rm in replacement_modules]
    sources = NodeRefs.from_nodes_and_refs(
        [("hook_embed", seq_indices, cache["hook_embed.post"])] + [(o + ".error", seq_indices, cache[o + ".error.post"]) for o in outs]
    )
    inter = [(o + ".sae.hook_feature_acts", torch.nonzero(cache[o + ".sae.hook_feature_acts.pre"][0]),
              cache[o + ".sae.hook_feature_acts.pre"], cache[o + ".sae.hook_feature_acts.post"]) for o in outs]  # fmt: skip
    intermediates = IntermediateRefs(
        upstream=NodeRefs.from_nodes_and_refs([(k, i, pre) for k, i, pre, _ in inter]),
        downstream=NodeRefs.from_nodes_and_refs([(k, i, post) for k, i, _, post in inter]),
    )
    max_intermediates = max_features if max_features is not None else len(intermediates.downstream.dimension)
    max_iter = len(replacement_modules) + 10
    attribution, collected = greedily_collect_attribution(targets, sources, intermediates, max_intermediates, reduction_weight, max_iter)
    attribution = attribution[None, sources.dimension + collected]

    with torch.no_grad():
        target_vals = [v[0] for v in targets.values]
        inter_vals = [v[0] for v in intermediates.upstream[collected].values] if len(collected) else []
        src_vals = [torch.ones(len(idx), device=dev, dtype=sources.dtype) for _, idx, _ in sources]
        activations = torch.cat([t.detach().to(sources.dtype) for t in target_vals + inter_vals + src_vals])
    activations_vec = NodeIndexedVector.from_data(activations, (targets.dimension + collected + sources.dimension,))

    qk = None
    if enable_qk_tracing:
        lorsa_keys = {rm.cfg.hook_point_out + ".sae.hook_feature_acts" for rm in replacement_modules if isinstance(rm, LowRankSparseAttention)}
        lorsa_features = collected.filter_keys(lambda k: k in lorsa_keys)
        if len(lorsa_features) > 0:
            total = compute_intermediates_attribution(attribution, targets.dimension, collected, max_iter)
            infl = NodeIndexedVector.from_data(reduction_weight, (targets.dimension,)) @ total[None, lorsa_features]
            _, top_lorsa = infl.topk(k=max(1, int(len(lorsa_features) * qk_top_fraction)))
            groups, scales = _lorsa_tables(replacement_modules)
            q_t, k_t, slot_to_unique = _retrieve_qk_vector_targets(top_lorsa, cache, groups, scales)
            qk_sources = sources + NodeRefs.from_nodes_and_refs(
                [(o + ".sae.hook_feature_acts", torch.nonzero(cache[o + ".sae.hook_feature_acts.post"][0]), cache[o + ".sae.hook_feature_acts.post"]) for o in outs]
                + _bias_source_entries(model, replacement_modules, cache, seq_indices)
            )
            qk = _per_feature(compute_qk_tracing(q_t, k_t, qk_sources, topk=qk_topk), slot_to_unique, top_lorsa)

    tok = model.tokenizer
    decode = (lambda i: tok.decode([i])) if tok is not None else str
    prompt_ids = tokens.detach().cpu().tolist()
    logit_ids = top_idx.detach().cpu().tolist() if top_idx is not None and top_idx.numel() > 0 else None
    return AttributionResult(
        activations=activations_vec,
        attribution=attribution,
        targets=targets.dimension,
        logits=batch_logits[:, -1, top_idx].detach() if logit_ids is not None else None,
        probs=top_p if target_type == "logits" else None,
        prompt_token_ids=prompt_ids,
        prompt_tokens=[decode(i) for i in prompt_ids],
        logit_token_ids=logit_ids,
        logit_tokens=[decode(i) for i in logit_ids] if logit_ids is not None else None,
        qk_trace_results=qk,
    )


def _retrieve_qk_vector_targets(features: NodeDimension, cache: dict[str, torch.Tensor], ov_group_sizes: dict[str, int],
                                attn_scales: dict[str, float]) -> tuple[NodeRefs, NodeRefs, list[int]]:  # fmt: skip
    """For attention features ``(q position, OV head)``: the query vector at the q position and the key vector at the
    most-attended position of the feature's QK head (both scaled by ``attn_scale ** -0.5`` so that their dot product
    IS the attention score). OV heads sharing a QK head give the same pair; pairs are deduplicated and
    ``slot_to_unique`` maps each feature to its pair."""
    triples = []
    for node in features:
        path = node.key.replace(".sae.hook_feature_acts", "")
        q_pos, ov_head = node.indices[0].tolist()
        head = ov_head // ov_group_sizes[path]
        k_pos = int(cache[f"{path}.sae.hook_attn_score"][0, head, q_pos].argmax())
        triples.append((path, int(head), int(q_pos), k_pos))
    unique: dict[tuple, int] = {}
    slot_to_unique = [unique.setdefault(t, len(unique)) for t in triples]

    @functools.cache
    def scaled(path: str):
        c = attn_scales[path] ** -0.5
        return cache[f"{path}.sae.hook_q_post_rot"] * c, cache[f"{path}.sae.hook_k_post_rot"] * c

    q_entries, k_entries = [], []
    for path, head, q_pos, k_pos in unique:
        q_ref, k_ref = scaled(path)
        q_entries.append((f"{path}.sae.hook_q_post_rot", torch.tensor([[q_pos, head]], device=q_ref.device), q_ref))
        k_entries.append((f"{path}.sae.hook_k_post_rot", torch.tensor([[k_pos, head]], device=k_ref.device), k_ref))
    return NodeRefs.from_nodes_and_refs(q_entries), NodeRefs.from_nodes_and_refs(k_entries), slot_to_unique


def qk_trace(model: HookedTransformer, inputs: "torch.Tensor | str", replacement_modules: list[SparseDictionary],
             lorsa_features: NodeDimension, topk: int = 10, batch_size: int = 1) -> QKTracingResult:  # fmt: skip
    """QK tracing of given attention features without building the whole attribution graph."""
    dev = next(model.parameters()).device
    tokens = ensure_tokenized(inputs, model.tokenizer, device=dev)
    _, cache = collect_cache(model, tokens[None].expand(batch_size * topk, -1), replacement_modules, with_bias_leaves=True)
    seq_indices = torch.arange(cache["hook_embed.post"].shape[1], device=dev)[:, None]
    entries = [("hook_embed", seq_indices, cache["hook_embed.post"])]
    for rm in replacement_modules:
        o = rm.cfg.hook_point_out
        entries.append((o + ".error", seq_indices, cache[o + ".error.post"]))
        entries.append((o + ".sae.hook_feature_acts", torch.nonzero(cache[o + ".sae.hook_feature_acts.post"][0]), cache[o + ".sae.hook_feature_acts.post"]))
    entries += _bias_source_entries(model, replacement_modules, cache, seq_indices)
    groups, scales = _lorsa_tables(replacement_modules)
    q_t, k_t, slot_to_unique = _retrieve_qk_vector_targets(lorsa_features, cache, groups, scales)
    return _per_feature(compute_qk_tracing(q_t, k_t, NodeRefs.from_nodes_and_refs(entries), topk=topk), slot_to_unique, lorsa_features)


def _slot_rows(stacked: torch.Tensor, topk: int) -> torch.Tensor:
    """Slot ``s`` owns forward rows ``s*topk .. (s+1)*topk``: ``[n_slots, topk, ...]``."""
    return torch.stack([stacked[s * topk : (s + 1) * topk, s] for s in range(stacked.shape[1])], dim=0)


def compute_hessian_matrix(targets: NodeRefs, sources: NodeRefs, topk: int) -> "NodeIndexed[list[NodeIndexed[torch.Tensor]]]":
    """Second-order attributions: per target its ``topk`` first-order sources and, for each of them, the source with
    the largest second-order (input x gradient of the first-order score) interaction. Each target uses ``topk``
    forward rows, one per first-order source followed up."""
    per_batch = sources.batch_size // topk
    results: list[NodeIndexed[torch.Tensor]] = []
    for tb in targets.iter_batches(per_batch):
        stacked = torch.cat(tb.values, dim=1)
        n = stacked.shape[1]
        first_root = _slot_rows(stacked, topk)
        g1 = torch.autograd.grad(first_root.sum(), sources.refs(), create_graph=True, retain_graph=True, allow_unused=True)
        a1 = attribution_scores(g1, sources)
        picks = torch.stack([a1[s * topk].topk(topk).indices for s in range(n)])  # [n, topk]
        rows = torch.arange(n, device=a1.device)[:, None] * topk + torch.arange(topk, device=a1.device)[None]
        g2 = torch.autograd.grad(a1[rows, picks].sum(), sources.refs(), retain_graph=True, materialize_grads=True)
        a2 = attribution_scores(g2, sources).detach()
        for s in range(n):
            vals, idx = a2[s * topk : (s + 1) * topk].max(dim=-1)
            order = torch.argsort(vals, descending=True)
            order = order[vals[order] != 0]
            results.append(NodeIndexed(vals[order], (sources.dimension.offsets_to_nodes(picks[s][order]), sources.dimension.offsets_to_nodes(idx[order]))))
    return NodeIndexed(results, (targets.dimension,))


def _extract_topk_pairwise_attributions(q_side: NodeIndexedMatrix, k_side: NodeIndexedMatrix, topk: int) -> "NodeIndexed[torch.Tensor]":
    """Merge the strongest entries of the (q pick x source) and (k pick x source) second-order blocks into at most
    ``topk`` non-zero (q-role node, k-role node) pairs; pairs already counted from the q side are dropped on the k side."""
    if len(k_side.dimensions[0]) > 0 and len(q_side.dimensions[0]) > 0:
        k_side = k_side.clone()
        present = k_side.dimensions[1].nodes_to_offsets(q_side.dimensions[0])
        k_side.data[:, present[present >= 0]] = 0
    q_top, k_top = q_side.flat_topk(topk), k_side.flat_topk(topk)
    values = torch.cat([q_top.value, k_top.value])
    q_role = q_top.dimensions[0] + k_top.dimensions[1]
    k_role = q_top.dimensions[1] + k_top.dimensions[0]
    n = min(topk, int((values != 0).sum()))
    # the strongest NON-ZERO entries: an entry zeroed by the de-duplication above (or absent from the graph) must not
    # outrank a negative one and come back labelled with a pair whose true term is not zero
    top_v, top_i = torch.topk(values.masked_fill(values == 0, float("-inf")), n)
    return NodeIndexed(top_v, (q_role.offsets_to_nodes(top_i), k_role.offsets_to_nodes(top_i)))


@timer.time("compute_qk_tracing")
def compute_qk_tracing(q_targets: NodeRefs, k_targets: NodeRefs, sources: NodeRefs, topk: int) -> QKTracingResult:
    """Attribute attention scores ``q . k``. First order: the vector-Jacobian product of ``q`` with cotangent ``k``
    gives each source's contribution through the query side (``a_Q``), and vice versa (``a_K``). Second order: for the
    ``topk`` strongest first-order entries of a slot, back-propagate that entry (one forward row each) to get its
    partner sources on the other side; merged into (q source, k source) pairs."""
    assert len(q_targets.dimension) == len(k_targets.dimension)
    per_batch = max(1, sources.batch_size // topk)

    def vjp(outputs: torch.Tensor, cotangent: torch.Tensor) -> torch.Tensor:
        grads = torch.autograd.grad(outputs, sources.refs(), grad_outputs=cotangent, create_graph=True, retain_graph=True, allow_unused=True)
        return attribution_scores(grads, sources)

    def top_nonzero(scores: torch.Tensor) -> NodeIndexed[torch.Tensor]:
        v, i = scores.detach().topk(min(topk, scores.numel()))
        keep = v != 0
        return NodeIndexed(v[keep], (sources.dimension.offsets_to_nodes(i[keep]),))

    q_marg, k_marg, pairs = [], [], []
    for q_sub, k_sub in zip(q_targets.iter_batches(per_batch), k_targets.iter_batches(per_batch)):
        q_vecs = _slot_rows(torch.cat(q_sub.values, dim=1), topk)  # [n_slots, topk, d_qk]
        k_vecs = _slot_rows(torch.cat(k_sub.values, dim=1), topk)
        n = q_vecs.shape[0]
        a_q, a_k = vjp(q_vecs, k_vecs), vjp(k_vecs, q_vecs)
        n_src = a_q.shape[1]
        first = torch.arange(n, device=a_q.device) * topk
        rows = first[:, None] + torch.arange(topk, device=a_q.device)[None]
        _, pick = torch.cat([a_q[first].detach(), a_k[first].detach()], dim=-1).topk(topk, dim=-1)
        is_q = pick < n_src
        src = torch.where(is_q, pick, pick - n_src)
        second_root = torch.where(is_q, a_q[rows, src], a_k[rows, src]).sum()
        g2 = torch.autograd.grad(second_root, sources.refs(), retain_graph=True, materialize_grads=True)
        a2 = attribution_scores(g2, sources).detach()
        a_q, a_k = a_q.detach(), a_k.detach()
        for s in range(n):
            q_marg.append(top_nonzero(a_q[s * topk]))
            k_marg.append(top_nonzero(a_k[s * topk]))
            block = a2[s * topk : (s + 1) * topk]
            qm = is_q[s]
            q_side = NodeIndexedMatrix.from_data(block[qm], (sources.dimension.offsets_to_nodes(src[s][qm]), sources.dimension))
            k_side = NodeIndexedMatrix.from_data(block[~qm], (sources.dimension.offsets_to_nodes(src[s][~qm]), sources.dimension))
            pairs.append(_extract_topk_pairwise_attributions(q_side, k_side, topk))
    outer = (q_targets.dimension,)
    return QKTracingResult(NodeIndexed(q_marg, outer), NodeIndexed(k_marg, outer), NodeIndexed(pairs, outer))
