"""Circuit endpoints: prompt preview, dictionary sets, background attribution jobs, pruned graphs, QK details
(server/routers/circuits.py of the reference project; same paths and payloads)."""

from __future__ import annotations

import functools
import re
import threading
import traceback
from datetime import datetime, timezone
from typing import Any, Optional

import torch
from fastapi import APIRouter, BackgroundTasks, Response
from pydantic import BaseModel

from ...backend.hooked_transformer import HookedTransformer
from ...circuits import attribute
from ...database import CircuitConfig, CircuitInput, CircuitStatus
from ...models.lorsa import LorsaConfig
from ...parallel.mesh import is_primary_rank
from ...utils.logging import get_distributed_logger
from .. import config as C
from ..common import make_serializable, synchronized
from ..graph import build_graph
from ..loaders import get_model, get_sae, get_sae_cfg
from ..samples import list_feature_data
from ..workers import distributed

logger = get_distributed_logger("server.circuits")
router = APIRouter(tags=["circuits"])
_generation_lock = threading.Lock()


def _render_prompt(model, inp: CircuitInput) -> str:
    if inp.input_type == "plain_text":
        return inp.text
    if inp.input_type == "chat_template":
        return model.tokenizer.apply_chat_template(inp.messages, tokenize=False, add_generation_prompt=False, continue_final_message=True)
    raise ValueError(f"Invalid input type: {inp.input_type}")


def _model_of_set(sae_set, device_mesh=None):
    name = C.client.get_sae_model_name(sae_set.sae_names[0], sae_set.sae_series)
    return get_model(name=name, device_mesh=device_mesh)


class PreviewRequest(BaseModel):
    input: CircuitInput
    sae_set_name: str


@router.post("/preview")
@distributed
def preview(request: PreviewRequest, device_mesh=None):
    """The rendered prompt and the five most likely next tokens."""
    sae_set = C.client.get_sae_set(name=request.sae_set_name)
    assert sae_set is not None, f"SAE set {request.sae_set_name} not found"
    model = _model_of_set(sae_set, device_mesh)
    assert isinstance(model, HookedTransformer), f"Preview needs the hooked-transformer backend, got {type(model).__name__}"
    assert model.tokenizer is not None, "Preview requires a tokenizer"
    prompt = _render_prompt(model, request.input)
    with torch.no_grad():
        probs = torch.softmax(model(model.to_tokens(prompt))[0, -1].float(), dim=-1)
        top = torch.topk(probs, min(5, probs.numel()))
    return {"prompt": prompt, "next_tokens": [{"token": model.tokenizer.decode([i]), "prob": p} for i, p in zip(top.indices.tolist(), top.values.tolist())]}


class CreateSaeSetRequest(BaseModel):
    name: str
    sae_names: list[str]


@router.get("/sae-sets")
def list_sae_sets():
    return [s.name for s in C.client.list_sae_sets() if s.sae_series == C.sae_series]


@router.post("/sae-sets")
def create_sae_set(request: CreateSaeSetRequest):
    if C.client.get_sae_set(request.name) is not None:
        return Response(content=f"SAE set with name '{request.name}' already exists", status_code=409)
    C.client.add_sae_set(name=request.name, sae_series=C.sae_series, sae_names=request.sae_names)
    return {"message": f"SAE set '{request.name}' created successfully"}


class GenerateCircuitRequest(BaseModel):
    """``list_of_features``: ``(layer, feature index, position, is_lorsa)`` targets; logits are the targets without it."""

    input: CircuitInput
    name: Optional[str] = None
    group: Optional[str] = None
    desired_logit_prob: float = 0.98
    max_feature_nodes: int = 256
    qk_tracing_topk: int = 10
    max_n_logits: int = 1
    list_of_features: Optional[list[tuple[int, int, int, bool]]] = None
    parent_id: Optional[str] = None


def _sae_metadata(sae_names: list[str]) -> dict[str, dict[str, Any]]:
    meta = {}
    for name in sae_names:
        cfg = get_sae_cfg(name=name)
        m = re.search(r"blocks\.(\d+)\.", cfg.hook_point_out)
        meta[cfg.hook_point_out] = {"sae_name": name, "is_lorsa": isinstance(cfg, LorsaConfig), "layer_idx": int(m.group(1)) if m else 0}
    return meta


@synchronized
@functools.lru_cache(maxsize=C.LRU_CACHE_SIZE_CIRCUITS)
def load_circuit_graph(*, circuit_id: str, node_threshold: float, edge_threshold: float) -> dict[str, Any]:
    """Load the stored attribution, prune it with the given thresholds and attach the feature records."""
    circuit = C.client.get_circuit(circuit_id)
    if circuit is None:
        raise ValueError(f"Circuit {circuit_id} not found")
    if circuit.status != CircuitStatus.COMPLETED:
        raise ValueError(f"Circuit {circuit_id} is not completed (status: {circuit.status})")
    ar = C.client.load_attribution(circuit_id, device=C.device)
    if ar is None:
        raise ValueError(f"Attribution data not found for circuit {circuit_id}")
    sae_set = C.client.get_sae_set(name=circuit.sae_set_name)
    if sae_set is None:
        raise ValueError(f"SAE set {circuit.sae_set_name} not found")
    graph = build_graph(ar, circuit.prompt, _sae_metadata(sae_set.sae_names), node_threshold, edge_threshold)
    by_sae: dict[str, list[int]] = {}
    for node in graph["nodes"]:
        if node.get("sae_name") is not None:
            by_sae.setdefault(node["sae_name"], []).append(node["feature"])
    records: dict[tuple[str, int], dict[str, Any]] = {}
    for name, idx in by_sae.items():
        records |= list_feature_data(sae_name=name, indices=sorted(set(idx)), with_samplings=False)
    for node in graph["nodes"]:
        if node.get("sae_name") is not None:
            node["feature"] = records.get((node["sae_name"], node["feature"]), {"feature_index": node["feature"], "dictionary_name": node["sae_name"]})
    return graph


@distributed
def run_circuit_attribution(circuit_id: str, sae_set_name: str, prompt: str, request: GenerateCircuitRequest, device_mesh=None):
    """Background job: run the attribution and store it; progress and failures are written to the circuit record."""
    primary = is_primary_rank(device_mesh)
    try:
        with _generation_lock:
            if primary:
                C.client.update_circuit_status(circuit_id, CircuitStatus.RUNNING)
                C.client.update_circuit_progress(circuit_id, 0.0, "Loading sparse dictionaries...")
            sae_set = C.client.get_sae_set(name=sae_set_name)
            assert sae_set is not None, f"SAE set {sae_set_name} not found"
            saes = {n: get_sae(name=n, device_mesh=device_mesh) for n in sae_set.sae_names}
            model = _model_of_set(sae_set, device_mesh)
            assert isinstance(model, HookedTransformer), "Circuit tracing needs the hooked-transformer backend"
            if primary:
                C.client.update_circuit_progress(circuit_id, 15.0, "Computing attribution...")
            targets: list[tuple[str, int, int]] = []
            if request.list_of_features:
                key_of = {}
                for sae in saes.values():
                    m = re.search(r"blocks\.(\d+)\.", sae.cfg.hook_point_out)
                    if m:
                        key_of[(int(m.group(1)), isinstance(sae.cfg, LorsaConfig))] = sae.cfg.hook_point_out + ".sae.hook_feature_acts"
                missing = [(l, a) for l, _, _, a in request.list_of_features if (l, a) not in key_of]
                assert not missing, f"No SAE in set {sae_set_name} covers (layer, is_lorsa)={missing}"
                targets = [(key_of[(l, a)], pos, f) for l, f, pos, a in request.list_of_features]
            result = attribute(model, prompt, list(saes.values()), target_type="features" if targets else "logits", features=targets,
                               max_n_logits=request.max_n_logits, desired_logit_prob=request.desired_logit_prob, batch_size=10,
                               max_features=request.max_feature_nodes, enable_qk_tracing=request.qk_tracing_topk > 0,
                               qk_topk=max(1, min(request.qk_tracing_topk, 10)))  # fmt: skip
            if primary:
                C.client.update_circuit_progress(circuit_id, 90.0, "Storing attribution data...")
                C.client.store_attribution(circuit_id, result.to("cpu"))
                C.client.update_circuit_progress(circuit_id, 100.0, "Completed")
                C.client.update_circuit_status(circuit_id, CircuitStatus.COMPLETED)
    except Exception as e:  # noqa: BLE001 - the failure is the job's result
        logger.error(f"Circuit {circuit_id} attribution failed: {e}\n{traceback.format_exc()}")
        if primary:
            C.client.update_circuit_status(circuit_id, CircuitStatus.FAILED, error_message=str(e))


@router.post("/circuits")
def create_circuit(sae_set_name: str, request: GenerateCircuitRequest, background_tasks: BackgroundTasks):
    """Start a job and return at once (status ``pending``); poll ``/circuits/{id}/status``."""
    sae_set = C.client.get_sae_set(name=sae_set_name)
    if sae_set is None:
        return Response(content=f"SAE set {sae_set_name} not found", status_code=404)
    model = _model_of_set(sae_set)
    if getattr(model, "tokenizer", None) is None:
        return Response(content="Circuit generation requires a tokenizer", status_code=400)
    try:
        prompt = _render_prompt(model, request.input)
    except ValueError as e:
        return Response(content=str(e), status_code=400)
    cfg = CircuitConfig(desired_logit_prob=request.desired_logit_prob, max_feature_nodes=request.max_feature_nodes,
                        qk_tracing_topk=request.qk_tracing_topk, max_n_logits=request.max_n_logits, list_of_features=request.list_of_features)  # fmt: skip
    circuit_id = C.client.create_circuit(sae_set_name=sae_set_name, sae_series=C.sae_series, prompt=prompt, input=request.input, config=cfg,
                                         name=request.name, group=request.group, parent_id=request.parent_id)  # fmt: skip
    background_tasks.add_task(run_circuit_attribution, circuit_id=circuit_id, sae_set_name=sae_set_name, prompt=prompt, request=request, timeout=3600.0)
    return {"circuit_id": circuit_id, "status": CircuitStatus.PENDING, "name": request.name, "group": request.group, "sae_set_name": sae_set_name,
            "prompt": prompt, "config": cfg.model_dump(), "input": request.input.model_dump(),
            "created_at": datetime.now(timezone.utc).replace(tzinfo=None).isoformat() + "Z", "parent_id": request.parent_id}  # fmt: skip


@router.get("/circuits")
def list_circuits(limit: int = 100, skip: int = 0, group: Optional[str] = None):
    rows = []
    for c in C.client.list_circuits(sae_series=C.sae_series, limit=limit, skip=skip, group=group):
        d = c.model_dump()
        d["created_at"] = c.created_at.isoformat() + "Z"
        rows.append(d)
    return make_serializable(rows)


@router.get("/circuits/{circuit_id}/status")
def get_circuit_status(circuit_id: str):
    status = C.client.get_circuit_status(circuit_id)
    if status is None:
        return Response(content=f"Circuit {circuit_id} not found", status_code=404)
    return status


def _ready_graph(circuit_id: str, node_threshold: float, edge_threshold: float):
    circuit = C.client.get_circuit(circuit_id)
    if circuit is None:
        return None, Response(content=f"Circuit {circuit_id} not found", status_code=404)
    if circuit.status != CircuitStatus.COMPLETED:
        return None, Response(content=f"Circuit {circuit_id} is not ready (status: {circuit.status})", status_code=202,
                              headers={"X-Circuit-Status": str(circuit.status)})  # fmt: skip
    try:
        return (circuit, load_circuit_graph(circuit_id=circuit_id, node_threshold=node_threshold, edge_threshold=edge_threshold)), None
    except ValueError as e:
        return None, Response(content=str(e), status_code=404)


@router.get("/circuits/{circuit_id}")
def get_circuit(circuit_id: str, node_threshold: float = 0.6, edge_threshold: float = 0.8):
    """The graph pruned on the fly: nodes / edges holding these fractions of the total influence are kept."""
    ok, err = _ready_graph(circuit_id, node_threshold, edge_threshold)
    if err is not None:
        return err
    circuit, graph = ok
    return make_serializable({
        "circuit_id": circuit.id, "name": circuit.name, "group": circuit.group, "input": circuit.input.model_dump(),
        "sae_set_name": circuit.sae_set_name, "prompt": circuit.prompt, "config": circuit.config.model_dump(), "graph_data": graph,
        "created_at": circuit.created_at.isoformat() + "Z", "parent_id": circuit.parent_id, "status": circuit.status,
        "node_threshold": node_threshold, "edge_threshold": edge_threshold,
    })  # fmt: skip


@router.get("/circuits/{circuit_id}/qk/{node_id}")
def get_circuit_qk_node(circuit_id: str, node_id: str, node_threshold: float = 0.6, edge_threshold: float = 0.8):
    """QK tracing of one attention-feature node with the nodes it references."""
    ok, err = _ready_graph(circuit_id, node_threshold, edge_threshold)
    if err is not None:
        return err
    by_id = {n["node_id"]: n for n in ok[1]["nodes"]}
    node = by_id.get(node_id)
    if node is None:
        return Response(content=f"Node {node_id} not found in circuit {circuit_id}", status_code=404)
    qk = node.get("qk_tracing_results")
    if qk is None:
        return Response(content=f"Node {node_id} has no QK tracing results", status_code=404)
    refs = {r for r, _ in qk.get("top_q_marginal_contributors", [])} | {r for r, _ in qk.get("top_k_marginal_contributors", [])}
    for q, k, _ in qk.get("pair_wise_contributors", []):
        refs |= {q, k}
    refs.discard(node_id)
    return make_serializable({"target_node": node, "referenced_nodes": [by_id[r] for r in refs if r in by_id]})


@router.delete("/circuits/{circuit_id}")
def delete_circuit(circuit_id: str):
    if C.client.delete_circuit(circuit_id):
        load_circuit_graph.cache_clear()
        return {"message": "Circuit deleted successfully"}
    return Response(content=f"Circuit {circuit_id} not found", status_code=404)
