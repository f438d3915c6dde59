"""Attribution result -> JSON graph for the circuit viewer (the ``load_circuit_graph`` part of
server/routers/circuits.py:136-393 of the reference project; same node / link schema).

Node ids: embeddings ``E_<token id>_<pos>``, features and logits ``<layer>_<index>_<pos>``, errors
``<layer>_error_<pos>``; rows of the viewer are ``2 * block`` for attention dictionaries, ``2 * block + 1`` for MLP
ones, ``2 * n_layers`` for logits, ``-1`` for embeddings.
"""

from __future__ import annotations

import re
from typing import Any

import torch

from ..circuits import AttributionResult, NodeDimension, prune_attribution


def _block_of(hook: str) -> int:
    m = re.search(r"blocks\.(\d+)\.", hook)
    return int(m.group(1)) if m else 0


def build_graph(ar: AttributionResult, prompt: str, sae_metadata: dict[str, dict[str, Any]], node_threshold: float = 0.6,
                edge_threshold: float = 0.8) -> dict[str, Any]:  # fmt: skip
    """``sae_metadata``: hook_point_out -> {"sae_name", "is_lorsa", "layer_idx"}."""
    dev = ar.attribution.data.device
    weight = ar.probs if ar.probs is not None else torch.ones(len(ar.targets), device=dev, dtype=ar.attribution.data.dtype)
    pruned = prune_attribution(ar.attribution, weight.to(ar.attribution.data.dtype), node_threshold, edge_threshold, targets=ar.targets)
    edge_w, (targets, sources) = pruned.nonzero()
    ov_nodes = (sources + targets).unique()
    qk = ar.qk_trace_results
    qk_nodes = NodeDimension.empty(dev)
    if qk is not None:
        for res, _ in qk.pairs:
            qk_nodes = qk_nodes + res.dimensions[0] + res.dimensions[1]
        for res, _ in list(qk.q_marginal) + list(qk.k_marginal):
            qk_nodes = qk_nodes + res.dimensions[0]
        qk_nodes = (qk_nodes.unique() - ov_nodes) if len(qk_nodes) else qk_nodes
    nodes = ov_nodes + qk_nodes
    acts = torch.zeros(len(nodes), dtype=torch.float32, device=dev)
    off = ar.activations.dimensions[0].nodes_to_offsets(ov_nodes)
    acts[: len(ov_nodes)] = torch.where(off >= 0, ar.activations.data[off.clamp(min=0)].float(), torch.zeros((), device=dev))
    token_of = dict(zip(ar.logit_token_ids or [], ar.logit_tokens or []))
    prob_of = dict(zip(ar.logit_token_ids or [], (ar.probs.tolist() if ar.probs is not None else [])))
    logit_rows = ar.targets.node_mappings.get("logits") if ar.targets is not None else None
    target_vocab = int(logit_rows.indices[0, 0]) if logit_rows is not None and len(logit_rows) else -1
    n_layers = max((int(m["layer_idx"]) for m in sae_metadata.values()), default=-1) + 1

    def layer_of(hook_out: str) -> tuple[int, bool, dict | None]:
        meta = sae_metadata.get(hook_out)
        lorsa = bool(meta["is_lorsa"]) if meta else False
        base = int(meta["layer_idx"]) if meta else _block_of(hook_out)
        return 2 * base + int(not lorsa), lorsa, meta

    def make_node(key: str, idx: list[int], activation: float, from_qk: bool) -> dict[str, Any]:
        common = {"is_target_logit": False, "is_from_qk_tracing": from_qk}
        if key == "hook_embed":
            pos = idx[0]
            tid = int(ar.prompt_token_ids[pos]) if pos < len(ar.prompt_token_ids) else -1
            return {"feature_type": "embedding", "node_id": f"E_{tid}_{pos}", "layer": -1, "ctx_idx": pos,
                    "token": ar.prompt_tokens[pos] if pos < len(ar.prompt_tokens) else "", **common}  # fmt: skip
        if key == "logits":
            v, ctx, layer = idx[0], max(len(ar.prompt_token_ids) - 1, 0), 2 * n_layers
            return {"feature_type": "logit", "node_id": f"{layer}_{v}_{ctx}", "layer": layer, "ctx_idx": ctx, "token_prob": prob_of.get(v),
                    "token": token_of.get(v), **common, "is_target_logit": v == target_vocab}  # fmt: skip
        if key.endswith(".error"):
            layer, lorsa, _ = layer_of(key.removesuffix(".error"))
            return {"feature_type": "lorsa error" if lorsa else "mlp reconstruction error", "node_id": f"{layer}_error_{idx[0]}",
                    "layer": layer, "ctx_idx": idx[0], **common}  # fmt: skip
        if key.endswith(".sae.hook_feature_acts"):
            layer, lorsa, meta = layer_of(key.removesuffix(".sae.hook_feature_acts"))
            pos, f = (idx + [0, 0])[:2]
            return {"feature_type": "lorsa" if lorsa else "cross layer transcoder", "node_id": f"{layer}_{f}_{pos}", "layer": layer,
                    "ctx_idx": pos, "feature": f, "sae_name": meta["sae_name"] if meta else None, "activation": activation,
                    "qk_tracing_results": None, **common}  # fmt: skip
        return {"feature_type": "bias", "node_id": f"{key}:{'_'.join(map(str, idx))}", "layer": 0, "ctx_idx": idx[0] if idx else 0, **common}

    key_ids, index_rows, act_list = nodes.key_ids.tolist(), nodes.indices.tolist(), acts.tolist()
    entries = [make_node(str(nodes.keys[k]), row[: nodes.ranks[k]], a, i >= len(ov_nodes))
               for i, (k, row, a) in enumerate(zip(key_ids, index_rows, act_list))]  # fmt: skip
    ids = [e["node_id"] for e in entries]
    t_off, s_off = nodes.nodes_to_offsets(targets).tolist(), nodes.nodes_to_offsets(sources).tolist()
    links = [{"source": ids[s], "target": ids[t], "weight": float(w)} for w, s, t in zip(edge_w.tolist(), s_off, t_off)]
    if qk is not None:
        lookup = lambda dim: [ids[o] if o >= 0 else None for o in nodes.nodes_to_offsets(dim).tolist()]  # noqa: E731
        for o, (pair, _), (qm, _), (km, _) in zip(nodes.nodes_to_offsets(qk.pairs.dimensions[0]).tolist(), qk.pairs, qk.q_marginal, qk.k_marginal):
            if o < 0:
                continue  # the traced feature itself was pruned away
            entries[o]["qk_tracing_results"] = {
                "pair_wise_contributors": [(q, k, float(v)) for q, k, v in zip(lookup(pair.dimensions[0]), lookup(pair.dimensions[1]), pair.value.tolist())],
                "top_q_marginal_contributors": [(n, float(v)) for n, v in zip(lookup(qm.dimensions[0]), qm.value.tolist())],
                "top_k_marginal_contributors": [(n, float(v)) for n, v in zip(lookup(km.dimensions[0]), km.value.tolist())],
            }
    return {"metadata": {"prompt_tokens": ar.prompt_tokens, "prompt": prompt, "schema_version": 1}, "nodes": entries, "links": links}
