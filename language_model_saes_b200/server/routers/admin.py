"""``/admin``: manage dictionaries, dictionary sets and circuits (server/routers/admin.py of the reference project).
Works through the store abstraction, so it serves the local file store as well as MongoDB."""

from __future__ import annotations

import re
from typing import Any, Optional

from fastapi import APIRouter, Response
from pydantic import BaseModel

from .. import config as C
from ..common import make_serializable, natural_sort_key
from ..loaders import get_sae

router = APIRouter(prefix="/admin", tags=["admin"])


@router.get("/saes")
def admin_list_saes(limit: int = 100, skip: int = 0, search: Optional[str] = None):
    st = C.client.store
    saes = st.find("saes", {"series": C.sae_series})
    if search:
        pat = re.compile(search, re.IGNORECASE)
        saes = [s for s in saes if pat.search(s["name"])]
    saes.sort(key=lambda s: s["name"])
    rows = []
    for s in saes[skip : skip + limit]:
        q = {"sae_name": s["name"], "sae_series": C.sae_series}
        rows.append({"name": s["name"], "series": s["series"], "path": s.get("path"), "model_name": s.get("model_name"),
                     "analysis_count": st.count("analyses", q), "feature_count": st.count("features", q), "cfg": s.get("cfg")})  # fmt: skip
    return make_serializable({"saes": rows, "total_count": len(saes)})


class UpdateSaeRequest(BaseModel):
    new_name: Optional[str] = None
    path: Optional[str] = None
    model_name: Optional[str] = None


@router.put("/saes/{name}")
def admin_update_sae(name: str, request: UpdateSaeRequest):
    st = C.client.store
    if st.find_one("saes", {"name": name, "series": C.sae_series}) is None:
        return Response(content=f"SAE {name} not found", status_code=404)
    upd: dict[str, Any] = {k: v for k, v in (("path", request.path), ("model_name", request.model_name)) if v is not None}
    if request.new_name is not None and request.new_name != name:
        if st.find_one("saes", {"name": request.new_name, "series": C.sae_series}):
            return Response(content=f"SAE with name '{request.new_name}' already exists", status_code=409)
        upd["name"] = request.new_name
        get_sae.cache_clear()
    if not upd:
        return {"message": "No updates provided"}
    C.client.update_sae(name, C.sae_series, upd)
    return {"message": f"SAE '{request.new_name or name}' updated successfully"}


@router.delete("/saes/{name}")
def admin_delete_sae(name: str):
    if C.client.store.find_one("saes", {"name": name, "series": C.sae_series}) is None:
        return Response(content=f"SAE {name} not found", status_code=404)
    C.client.remove_sae(sae_name=name, sae_series=C.sae_series)
    get_sae.cache_clear()
    return {"message": f"SAE '{name}' and all associated data deleted successfully"}


@router.get("/sae-sets")
def admin_list_sae_sets():
    rows = [{"name": s.name, "sae_series": s.sae_series, "sae_names": s.sae_names} for s in C.client.list_sae_sets() if s.sae_series == C.sae_series]
    return sorted(rows, key=lambda r: natural_sort_key(r["name"]))


class UpdateSaeSetRequest(BaseModel):
    new_name: Optional[str] = None
    sae_names: Optional[list[str]] = None


@router.put("/sae-sets/{name}")
def admin_update_sae_set(name: str, request: UpdateSaeSetRequest):
    if C.client.get_sae_set(name) is None:
        return Response(content=f"SAE set {name} not found", status_code=404)
    upd: dict[str, Any] = {}
    if request.sae_names is not None:
        upd["sae_names"] = request.sae_names
    if request.new_name is not None and request.new_name != name:
        if C.client.get_sae_set(request.new_name) is not None:
            return Response(content=f"SAE set with name '{request.new_name}' already exists", status_code=409)
        upd["name"] = request.new_name
    if not upd:
        return {"message": "No updates provided"}
    C.client.update_sae_set(name, upd)
    return {"message": f"SAE set '{request.new_name or name}' updated successfully"}


@router.delete("/sae-sets/{name}")
def admin_delete_sae_set(name: str):
    if C.client.store.delete_many("sae_sets", {"name": name}) == 0:
        return Response(content=f"SAE set {name} not found", status_code=404)
    return {"message": f"SAE set '{name}' deleted successfully"}


def _circuit_row(c) -> dict[str, Any]:
    d = c.model_dump()
    d["created_at"] = c.created_at.isoformat() + "Z"
    return d


@router.get("/circuits")
def admin_list_circuits(limit: int = 100, skip: int = 0):
    rows = [_circuit_row(c) for c in C.client.list_circuits(sae_series=C.sae_series, limit=limit, skip=skip)]
    return make_serializable({"circuits": rows, "total_count": C.client.store.count("circuits", {"sae_series": C.sae_series})})


class UpdateCircuitRequest(BaseModel):
    name: Optional[str] = None
    group: Optional[str] = None


@router.put("/circuits/{circuit_id}")
def admin_update_circuit(circuit_id: str, request: UpdateCircuitRequest):
    upd = {k: v for k, v in (("name", request.name), ("group", request.group)) if v is not None}
    if not upd:
        return {"message": "No updates provided"}
    if not C.client.update_circuit(circuit_id, upd):
        return Response(content=f"Circuit {circuit_id} not found", status_code=404)
    return {"message": "Circuit updated successfully"}


class BulkGroupRequest(BaseModel):
    circuit_ids: list[str]
    group: Optional[str] = None


@router.post("/circuits/bulk-group")
def admin_bulk_group_circuits(request: BulkGroupRequest):
    return {"message": f"Updated {C.client.update_circuits_group(request.circuit_ids, request.group)} circuits"}


@router.get("/stats")
def admin_get_stats():
    st, ser = C.client.store, C.sae_series
    return {"sae_count": st.count("saes", {"series": ser}), "sae_set_count": st.count("sae_sets", {"sae_series": ser}),
            "circuit_count": st.count("circuits", {"sae_series": ser}), "bookmark_count": st.count("bookmarks", {"sae_series": ser}),
            "sae_series": ser}  # fmt: skip
