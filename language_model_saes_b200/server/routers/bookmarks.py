"""``/bookmarks``: list bookmarked features, optionally with their feature records
(server/routers/bookmarks.py of the reference project)."""

from typing import Optional

from fastapi import APIRouter, Response

from .. import config as C
from ..common import make_serializable
from ..samples import list_feature_data

router = APIRouter(prefix="/bookmarks", tags=["bookmarks"])


@router.get("")
def list_bookmarks(sae_name: Optional[str] = None, limit: int = 100, skip: int = 0, include_features: bool = False):
    marks = C.client.list_bookmarks(sae_name=sae_name, sae_series=C.sae_series, limit=limit, skip=skip)
    features = {}
    if include_features:
        by_sae: dict[str, list[int]] = {}
        for b in marks:
            by_sae.setdefault(b.sae_name, []).append(b.feature_index)
        for name, idx in by_sae.items():
            features |= list_feature_data(sae_name=name, indices=idx)
    rows = []
    for b in marks:
        d = b.model_dump()
        d["created_at"] = b.created_at.isoformat() + "Z"
        if include_features:
            if (b.sae_name, b.feature_index) not in features:
                return Response(content=f"Feature {b.feature_index} not found in SAE {b.sae_name}", status_code=404)
            d["feature"] = features[(b.sae_name, b.feature_index)]
        rows.append(d)
    return make_serializable({"bookmarks": rows, "total_count": C.client.get_bookmark_count(sae_name=sae_name, sae_series=C.sae_series)})
