"""Metadata store for dictionaries, per-feature analyses, bookmarks, dictionary sets and circuits.

Collections, record models and the client's methods follow database.py of the reference project
(:30-183 records, :185-1071 ``MongoClient``): collections ``features, saes, analyses, datasets, models,
bookmarks, sae_sets, circuits`` and a blob store for numpy arrays (GridFS there).

Two interchangeable document stores sit under the same client: MongoDB through ``pymongo`` (+ GridFS) when the
package is installed and the URI is a ``mongodb://`` one, and an embedded file store (one JSON file per
document, ``.npy`` blobs) for ``file://<dir>`` URIs or machines without pymongo, so that analysis, the CLI and the
server work offline with the same code.
"""

from __future__ import annotations

import io
import json
import os
import threading
import time
import uuid
from datetime import datetime, timezone
from pathlib import Path
from typing import Annotated, Any, Iterable, Literal, Optional, Union

import numpy as np
import torch
from pydantic import BaseModel, Field, field_validator

from .backend.language_model import LanguageModelConfig
from .config import DatasetConfig
from .models.sparse_dictionary import SAE_TYPE_TO_CONFIG_CLASS, SparseDictionaryConfig


class MongoDBConfig(BaseModel):
    mongo_uri: str = Field(default_factory=lambda: os.environ.get("MONGO_URI", "mongodb://localhost:27017/"))
    mongo_db: str = Field(default_factory=lambda: os.environ.get("MONGO_DB", "mechinterp"))


class DatasetRecord(BaseModel):
    name: str
    cfg: DatasetConfig


class FeatureAnalysisSampling(BaseModel):
    model_config = {"arbitrary_types_allowed": True}
    name: str
    feature_acts_indices: np.ndarray
    feature_acts_values: np.ndarray
    z_pattern_indices: np.ndarray | None = None
    z_pattern_values: np.ndarray | None = None
    dataset_name: list[str]
    shard_idx: np.ndarray | None = None
    n_shards: np.ndarray | None = None
    context_idx: np.ndarray
    model_name: list[str]


class FeatureAnalysis(BaseModel):
    name: str
    act_times: int
    max_feature_acts: float
    decoder_norms: Optional[list[float]] = None
    decoder_similarity_matrices: Optional[list[list[float]]] = None
    decoder_inner_product_matrices: Optional[list[list[float]]] = None
    n_analyzed_tokens: Optional[int] = None
    act_times_modalities: Optional[dict[str, float]] = None
    max_feature_acts_modalities: Optional[dict[str, float]] = None
    samplings: list[FeatureAnalysisSampling] = []


class FeatureRecord(BaseModel):
    sae_name: str
    sae_series: str
    index: int
    analyses: list[FeatureAnalysis] = []
    logits: Optional[dict[str, list[dict[str, Any]]]] = None
    interpretation: Optional[dict[str, Any]] = None
    metric: Optional[dict[str, float]] = None


class AnalysisRecord(BaseModel):
    name: str
    sae_name: str
    sae_series: str


class ModelRecord(BaseModel):
    name: str
    cfg: LanguageModelConfig


def _load_model_modules() -> None:
    from importlib import import_module

    for m in ("sae", "crosscoder", "clt", "lorsa", "molt"):
        import_module(f"{__package__}.models.{m}")


class SAERecord(BaseModel):
    name: str
    series: str
    path: str
    cfg: SparseDictionaryConfig
    model_name: Optional[str] = None

    @field_validator("cfg", mode="before")
    @classmethod
    def _resolve_concrete_sae_cfg(cls, value: Any) -> Any:
        """A stored config dict is validated with the config class registered for its ``sae_type``."""
        if not isinstance(value, dict) or not isinstance(value.get("sae_type"), str):
            return value
        if value["sae_type"] not in SAE_TYPE_TO_CONFIG_CLASS:
            _load_model_modules()
        cfg_cls = SAE_TYPE_TO_CONFIG_CLASS.get(value["sae_type"])
        if cfg_cls is None:
            raise ValueError(f"Unknown sae_type '{value['sae_type']}' in SAE config")
        return cfg_cls.model_validate(value)


class SAESetRecord(BaseModel):
    name: str
    sae_series: str
    sae_names: list[str]


class BookmarkRecord(BaseModel):
    sae_name: str
    sae_series: str
    feature_index: int
    created_at: datetime
    tags: list[str] = []
    notes: Optional[str] = None


class CircuitStatus(str):
    PENDING = "pending"
    RUNNING = "running"
    COMPLETED = "completed"
    FAILED = "failed"


class CircuitConfig(BaseModel):
    desired_logit_prob: float = 0.98
    max_feature_nodes: int = 256
    qk_tracing_topk: int = 10
    max_n_logits: int = 1
    list_of_features: Optional[list[tuple[int, int, int, bool]]] = None


class CircuitTextInput(BaseModel):
    input_type: Literal["plain_text"] = "plain_text"
    text: str


class CircuitChatTemplateInput(BaseModel):
    input_type: Literal["chat_template"] = "chat_template"
    messages: list[dict[str, str]]


CircuitInput = Annotated[Union[CircuitTextInput, CircuitChatTemplateInput], Field(discriminator="input_type")]


class CircuitRecord(BaseModel):
    id: str
    name: Optional[str] = None
    group: Optional[str] = None
    sae_set_name: str
    sae_series: str
    prompt: str
    input: CircuitInput
    config: CircuitConfig
    created_at: datetime
    parent_id: Optional[str] = None
    status: str = CircuitStatus.PENDING
    progress: float = 0.0
    progress_phase: Optional[str] = None
    error_message: Optional[str] = None


# --------------------------------------------------------------------------------------------------
# document stores
# --------------------------------------------------------------------------------------------------
def _matches(doc: dict, query: dict) -> bool:
    """Equality on (dotted) keys plus the operators the client uses: $in, $exists, $gt, $gte, $lt, $lte, $ne."""
    for key, want in query.items():
        cur: Any = doc
        found = True
        for part in key.split("."):
            if isinstance(cur, dict) and part in cur:
                cur = cur[part]
            else:
                found = False
                break
        if isinstance(want, dict) and any(k.startswith("$") for k in want):
            for op, arg in want.items():
                ok = {
                    "$in": lambda: found and cur in arg,
                    "$exists": lambda: found == bool(arg),
                    "$gt": lambda: found and cur is not None and cur > arg,
                    "$gte": lambda: found and cur is not None and cur >= arg,
                    "$lt": lambda: found and cur is not None and cur < arg,
                    "$lte": lambda: found and cur is not None and cur <= arg,
                    "$ne": lambda: (cur if found else None) != arg,
                }[op]()
                if not ok:
                    return False
        elif not found or cur != want:
            return False
    return True


def _set_dotted(doc: dict, key: str, value: Any) -> None:
    parts = key.split(".")
    for p in parts[:-1]:
        doc = doc.setdefault(p, {})
    doc[parts[-1]] = value


class LocalStore:
    """Embedded document store: ``<root>/<collection>/<id>.json`` and ``<root>/blobs/<id>.npy``."""

    def __init__(self, root: str | Path):
        self.root = Path(root)
        self.root.mkdir(parents=True, exist_ok=True)
        (self.root / "blobs").mkdir(exist_ok=True)
        self._lock = threading.RLock()
        self._cache: dict[str, dict[str, dict]] = {}
        self._stamps: dict[str, int] = {}
        self._own: dict[str, int] = {}

    def _coll(self, name: str) -> dict[str, dict]:
        """Documents of a collection, cached in memory. Files are replaced atomically (write + rename), which bumps the
        directory's modification time; a cache older than the directory is re-read, so that several processes (a job
        and the command line, say) see each other's writes."""
        with self._lock:
            d = self.root / name
            d.mkdir(exist_ok=True)
            stamp = d.stat().st_mtime_ns
            # File-system timestamps tick coarsely (a few ms): an equal stamp only proves "unchanged" once it is older
            # than a tick, or when it is the stamp of this object's own last write.
            settled = time.time_ns() - stamp > 20_000_000 or self._own.get(name) == stamp
            if name not in self._cache or self._stamps.get(name) != stamp or not settled:
                self._cache[name] = {p.stem: json.loads(p.read_text()) for p in d.glob("*.json")}
                self._stamps[name] = stamp
            return self._cache[name]

    def _touch(self, coll: str) -> None:
        self._stamps[coll] = self._own[coll] = (self.root / coll).stat().st_mtime_ns

    def _write(self, coll: str, _id: str, doc: dict) -> None:
        tmp = self.root / coll / f".{_id}.tmp"
        tmp.write_text(json.dumps(doc, default=str))
        os.replace(tmp, self.root / coll / f"{_id}.json")
        self._touch(coll)

    def find(self, coll: str, query: dict) -> list[dict]:
        with self._lock:
            return [dict(d) for d in self._coll(coll).values() if _matches(d, query)]

    def find_one(self, coll: str, query: dict) -> dict | None:
        for d in self._coll(coll).values():
            if _matches(d, query):
                return dict(d)
        return None

    def count(self, coll: str, query: dict) -> int:
        return sum(1 for d in self._coll(coll).values() if _matches(d, query))

    def insert_one(self, coll: str, doc: dict) -> str:
        with self._lock:
            _id = str(doc.get("_id") or uuid.uuid4().hex)
            doc = {**doc, "_id": _id}
            self._coll(coll)[_id] = doc
            self._write(coll, _id, doc)
            return _id

    def update_one(self, coll: str, query: dict, set_fields: dict, upsert: bool = False, push: dict | None = None) -> bool:
        with self._lock:
            target = next((d for d in self._coll(coll).values() if _matches(d, query)), None)
            if target is None:
                if not upsert:
                    return False
                target = {k: v for k, v in query.items() if not isinstance(v, dict)}
                target["_id"] = uuid.uuid4().hex
                self._coll(coll)[target["_id"]] = target
            for k, v in set_fields.items():
                _set_dotted(target, k, v)
            for k, v in (push or {}).items():
                target.setdefault(k, []).append(v)
            self._write(coll, target["_id"], target)
            return True

    def delete_many(self, coll: str, query: dict) -> int:
        with self._lock:
            docs = self._coll(coll)
            ids = [i for i, d in docs.items() if _matches(d, query)]
            for i in ids:
                del docs[i]
                (self.root / coll / f"{i}.json").unlink(missing_ok=True)
            self._touch(coll)
            return len(ids)

    def put_blob(self, data: bytes) -> str:
        bid = uuid.uuid4().hex
        (self.root / "blobs" / bid).write_bytes(data)
        return bid

    def get_blob(self, bid: str) -> bytes:
        return (self.root / "blobs" / bid).read_bytes()

    def delete_blob(self, bid: str) -> None:
        (self.root / "blobs" / bid).unlink(missing_ok=True)


class PyMongoStore:
    """The same operations on a MongoDB database (blobs in GridFS)."""

    def __init__(self, uri: str, db: str):
        import gridfs
        import pymongo

        self.client = pymongo.MongoClient(uri)
        self.db = self.client[db]
        self.fs = gridfs.GridFS(self.db)
        self.db["features"].create_index([("sae_name", 1), ("sae_series", 1), ("index", 1)], unique=True)
        self.db["saes"].create_index([("name", 1), ("series", 1)], unique=True)
        self.db["bookmarks"].create_index([("sae_name", 1), ("sae_series", 1), ("feature_index", 1)], unique=True)

    def find(self, coll, query):
        return list(self.db[coll].find(query))

    def find_one(self, coll, query):
        return self.db[coll].find_one(query)

    def count(self, coll, query):
        return self.db[coll].count_documents(query)

    def insert_one(self, coll, doc):
        return str(self.db[coll].insert_one(doc).inserted_id)

    def update_one(self, coll, query, set_fields, upsert=False, push=None):
        upd: dict[str, Any] = {}
        if set_fields:
            upd["$set"] = set_fields
        if push:
            upd["$push"] = push
        r = self.db[coll].update_one(query, upd, upsert=upsert)
        return r.matched_count > 0 or r.upserted_id is not None

    def delete_many(self, coll, query):
        return self.db[coll].delete_many(query).deleted_count

    def put_blob(self, data: bytes) -> str:
        return str(self.fs.put(data))

    def get_blob(self, bid: str) -> bytes:
        from bson import ObjectId

        return self.fs.get(ObjectId(bid)).read()

    def delete_blob(self, bid: str) -> None:
        from bson import ObjectId

        self.fs.delete(ObjectId(bid))


def _open_store(cfg: MongoDBConfig):
    uri = cfg.mongo_uri
    if uri.startswith("file://"):
        return LocalStore(Path(uri[len("file://") :]) / cfg.mongo_db)
    try:
        import pymongo  # noqa: F401
    except ImportError:
        root = Path(os.environ.get("LMSAE_LOCAL_DB", Path.home() / ".lmsae_db"))
        return LocalStore(root / cfg.mongo_db)
    return PyMongoStore(uri, cfg.mongo_db)


# --------------------------------------------------------------------------------------------------
# client
# --------------------------------------------------------------------------------------------------
class MongoClient:
    def __init__(self, cfg: MongoDBConfig):
        self.cfg = cfg
        self.store = _open_store(cfg)
        self._use_blobs = True

    # ---- numpy blobs -------------------------------------------------------------------------
    def enable_gridfs(self) -> None:
        self._use_blobs = True

    def disable_gridfs(self) -> None:
        self._use_blobs = False

    def is_gridfs_enabled(self) -> bool:
        return self._use_blobs

    def _to_gridfs(self, data: Any) -> Any:
        """Replace every numpy array / tensor inside ``data`` by a reference to a stored blob."""
        if isinstance(data, torch.Tensor):
            data = data.detach().cpu().numpy()
        if isinstance(data, np.ndarray):
            if not self._use_blobs:
                return data.tolist()
            buf = io.BytesIO()
            np.save(buf, data, allow_pickle=False)
            return {"__blob__": self.store.put_blob(buf.getvalue())}
        if isinstance(data, dict):
            return {k: self._to_gridfs(v) for k, v in data.items()}
        if isinstance(data, (list, tuple)):
            return [self._to_gridfs(v) for v in data]
        if isinstance(data, np.generic):
            return data.item()
        return data

    def _from_gridfs(self, data: Any) -> Any:
        if isinstance(data, dict):
            if set(data) == {"__blob__"}:
                return np.load(io.BytesIO(self.store.get_blob(data["__blob__"])), allow_pickle=False)
            return {k: self._from_gridfs(v) for k, v in data.items()}
        if isinstance(data, list):
            return [self._from_gridfs(v) for v in data]
        return data

    def _remove_gridfs_objs(self, data: Any) -> None:
        if isinstance(data, dict):
            if set(data) == {"__blob__"}:
                self.store.delete_blob(data["__blob__"])
            else:
                for v in data.values():
                    self._remove_gridfs_objs(v)
        elif isinstance(data, list):
            for v in data:
                self._remove_gridfs_objs(v)

    # ---- dictionaries --------------------------------------------------------------------------
    def create_sae(self, name: str, series: str, path: str, cfg: SparseDictionaryConfig, model_name: str | None = None):
        """Register a dictionary and one (empty) feature record per latent."""
        self.store.update_one("saes", {"name": name, "series": series},
                              {"path": path, "cfg": cfg.model_dump(), "model_name": model_name}, upsert=True)  # fmt: skip
        if self.store.count("features", {"sae_name": name, "sae_series": series}) == 0:
            for i in range(cfg.d_sae):
                self.store.insert_one("features", {"sae_name": name, "sae_series": series, "index": i, "analyses": []})

    def create_analysis(self, name: str, sae_name: str, sae_series: str):
        self.store.update_one("analyses", {"name": name, "sae_name": sae_name, "sae_series": sae_series}, {}, upsert=True)

    def update_sae(self, name: str, series: str, update_data: dict[str, Any]):
        """Update a dictionary record; renaming (``name`` / ``series`` in the update) cascades to its features,
        analyses, bookmarks and sets."""
        new_name, new_series = update_data.get("name", name), update_data.get("series", series)
        self.store.update_one("saes", {"name": name, "series": series}, update_data)
        if (new_name, new_series) != (name, series):
            for coll, q in (("features", {"sae_name": name, "sae_series": series}),
                            ("analyses", {"sae_name": name, "sae_series": series}),
                            ("bookmarks", {"sae_name": name, "sae_series": series})):  # fmt: skip
                while self.store.update_one(coll, q, {"sae_name": new_name, "sae_series": new_series}):
                    pass
            for s in self.store.find("sae_sets", {"sae_series": series}):
                if name in s["sae_names"]:
                    names = [new_name if n == name else n for n in s["sae_names"]]
                    self.store.update_one("sae_sets", {"name": s["name"]}, {"sae_names": names})

    def update_sae_set(self, name: str, update_data: dict[str, Any]):
        self.store.update_one("sae_sets", {"name": name}, update_data)

    def remove_sae(self, sae_name: str, sae_series: str | None = None):
        q = {"name": sae_name} | ({"series": sae_series} if sae_series is not None else {})
        fq = {"sae_name": sae_name} | ({"sae_series": sae_series} if sae_series is not None else {})
        for f in self.store.find("features", fq):
            self._remove_gridfs_objs(f.get("analyses"))
        self.store.delete_many("features", fq)
        self.store.delete_many("analyses", fq)
        self.store.delete_many("saes", q)

    def list_analyses(self, sae_name: str, sae_series: str | None = None) -> list[str]:
        q = {"sae_name": sae_name} | ({"sae_series": sae_series} if sae_series is not None else {})
        return [a["name"] for a in self.store.find("analyses", q)]

    def list_saes(self, sae_series: str | None = None, has_analyses: bool = False) -> list[str]:
        q = {"series": sae_series} if sae_series is not None else {}
        names = [s["name"] for s in self.store.find("saes", q)]
        if has_analyses:
            aq = {"sae_series": sae_series} if sae_series is not None else {}
            with_a = {a["sae_name"] for a in self.store.find("analyses", aq)}
            names = [n for n in names if n in with_a]
        return names

    def get_sae(self, sae_name: str, sae_series: str) -> Optional[SAERecord]:
        d = self.store.find_one("saes", {"name": sae_name, "series": sae_series})
        return SAERecord.model_validate(d) if d else None

    def get_sae_path(self, sae_name: str, sae_series: str):
        d = self.store.find_one("saes", {"name": sae_name, "series": sae_series})
        return d["path"] if d else None

    def get_sae_model_name(self, sae_name: str, sae_series: str) -> Optional[str]:
        d = self.store.find_one("saes", {"name": sae_name, "series": sae_series})
        return d.get("model_name") if d else None

    # ---- datasets / models -----------------------------------------------------------------------
    def add_dataset(self, name: str, cfg: DatasetConfig):
        self.store.update_one("datasets", {"name": name}, {"cfg": cfg.model_dump()}, upsert=True)

    def get_dataset(self, name: str) -> Optional[DatasetRecord]:
        d = self.store.find_one("datasets", {"name": name})
        return DatasetRecord.model_validate(d) if d else None

    def get_dataset_cfg(self, name: str) -> Optional[DatasetConfig]:
        d = self.get_dataset(name)
        return d.cfg if d else None

    def add_model(self, name: str, cfg: LanguageModelConfig):
        self.store.update_one("models", {"name": name}, {"cfg": cfg.model_dump()}, upsert=True)

    def get_model_cfg(self, name: str) -> Optional[LanguageModelConfig]:
        d = self.store.find_one("models", {"name": name})
        return LanguageModelConfig.model_validate(d["cfg"]) if d else None

    # ---- features ----------------------------------------------------------------------------
    def _feature_record(self, d: dict | None) -> Optional[FeatureRecord]:
        return FeatureRecord.model_validate(self._from_gridfs(d)) if d else None

    def get_feature(self, sae_name: str, sae_series: str | None, index: int) -> Optional[FeatureRecord]:
        q = {"sae_name": sae_name, "index": index} | ({"sae_series": sae_series} if sae_series is not None else {})
        return self._feature_record(self.store.find_one("features", q))

    def list_features(self, sae_name: str, sae_series: str | None = None, indices: Iterable[int] | None = None) -> list[FeatureRecord]:
        q: dict[str, Any] = {"sae_name": sae_name} | ({"sae_series": sae_series} if sae_series is not None else {})
        if indices is not None:
            q["index"] = {"$in": list(indices)}
        recs = [self._feature_record(d) for d in self.store.find("features", q)]
        return sorted([r for r in recs if r is not None], key=lambda r: r.index)

    def get_analysis(self, name: str, sae_name: str, sae_series: str) -> Optional[AnalysisRecord]:
        d = self.store.find_one("analyses", {"name": name, "sae_name": sae_name, "sae_series": sae_series})
        return AnalysisRecord.model_validate(d) if d else None

    def _analysis_field(self, sae_name: str, sae_series: str, name: str, field: str) -> dict[int, Any] | None:
        out = {}
        for f in self.store.find("features", {"sae_name": sae_name, "sae_series": sae_series}):
            for a in f.get("analyses", []):
                if a.get("name") == name:
                    out[f["index"]] = a.get(field)
        return out or None

    def get_max_feature_acts(self, sae_name: str, sae_series: str, name: str = "default") -> dict[int, int] | None:
        return self._analysis_field(sae_name, sae_series, name, "max_feature_acts")

    def get_feature_act_times(self, sae_name: str, sae_series: str, name: str = "default"):
        return self._analysis_field(sae_name, sae_series, name, "act_times")

    def get_alive_feature_count(self, sae_name: str, sae_series: str, name: str = "default"):
        times = self.get_feature_act_times(sae_name, sae_series, name)
        return None if times is None else sum(1 for v in times.values() if v and v > 0)

    def get_random_alive_feature(self, sae_name: str, sae_series: str, name: str = "default",
                                 metric_filters: dict[str, dict[str, float]] | None = None) -> Optional[FeatureRecord]:  # fmt: skip
        import random

        times = self.get_feature_act_times(sae_name, sae_series, name) or {}
        alive = [i for i, v in times.items() if v and v > 0]
        random.shuffle(alive)
        for i in alive:
            rec = self.get_feature(sae_name, sae_series, i)
            if rec is None:
                continue
            if metric_filters and not all(
                rec.metric is not None and m in rec.metric
                and rec.metric[m] >= b.get("$gte", float("-inf")) and rec.metric[m] <= b.get("$lte", float("inf"))
                for m, b in metric_filters.items()
            ):  # fmt: skip
                continue
            return rec
        return None

    def add_feature_analysis(self, name: str, sae_name: str, sae_series: str, analysis: list[dict], start_idx: int = 0):
        """Append one analysis per feature, for features ``start_idx .. start_idx + len(analysis)``."""
        for i, a in enumerate(analysis):
            payload = self._to_gridfs({**a, "name": name})
            payload.pop("feature_idx", None)
            q = {"sae_name": sae_name, "sae_series": sae_series, "index": start_idx + i}
            if not self.store.update_one("features", q, {}, push={"analyses": payload}):
                self.store.insert_one("features", {**q, "analyses": [payload]})
        self.create_analysis(name, sae_name, sae_series)

    def remove_feature_analysis(self, name: str, sae_name: str, sae_series: str):
        for f in self.store.find("features", {"sae_name": sae_name, "sae_series": sae_series}):
            keep = [a for a in f.get("analyses", []) if a.get("name") != name]
            for a in f.get("analyses", []):
                if a.get("name") == name:
                    self._remove_gridfs_objs(a)
            self.store.update_one("features", {"sae_name": sae_name, "sae_series": sae_series, "index": f["index"]}, {"analyses": keep})
        self.store.delete_many("analyses", {"name": name, "sae_name": sae_name, "sae_series": sae_series})

    def remove_sae_analysis(self, sae_name: str, sae_series: str):
        for n in self.list_analyses(sae_name, sae_series):
            self.remove_feature_analysis(n, sae_name, sae_series)

    def update_feature(self, sae_name: str, feature_index: int, update_data: dict, sae_series: str | None = None):
        q = {"sae_name": sae_name, "index": feature_index} | ({"sae_series": sae_series} if sae_series is not None else {})
        if not self.store.update_one("features", q, self._to_gridfs(update_data)):
            raise ValueError(f"Feature {feature_index} not found for SAE {sae_name}/{sae_series}")

    def update_features(self, sae_name: str, sae_series: str, update_data: list[dict], start_idx: int = 0):
        for i, d in enumerate(update_data):
            self.update_feature(sae_name, start_idx + i, d, sae_series)

    def get_available_metrics(self, sae_name: str, sae_series: str) -> list[str]:
        names: set[str] = set()
        for f in self.store.find("features", {"sae_name": sae_name, "sae_series": sae_series, "metric": {"$exists": True}}):
            names.update((f.get("metric") or {}).keys())
        return sorted(names)

    def count_features_with_filters(self, sae_name: str, sae_series: str, name: str | None = None,
                                    metric_filters: dict[str, dict[str, float]] | None = None) -> int:  # fmt: skip
        """Features that fired at least once in the analysis ``name`` (any analysis when None) and pass the metric
        filters (``{"metric": {"$gte": a, "$lte": b}}``)."""
        q: dict[str, Any] = {"sae_name": sae_name, "sae_series": sae_series}
        for m, bounds in (metric_filters or {}).items():
            q[f"metric.{m}"] = bounds
        alive = lambda a: (name is None or a.get("name") == name) and (a.get("max_feature_acts") or 0) > 0  # noqa: E731
        return sum(1 for f in self.store.find("features", q) if any(alive(a) for a in f.get("analyses", [])))

    # ---- bookmarks ---------------------------------------------------------------------------
    def add_bookmark(self, sae_name: str, sae_series: str, feature_index: int, tags: list[str] | None = None, notes: str | None = None) -> bool:
        q = {"sae_name": sae_name, "sae_series": sae_series, "feature_index": feature_index}
        if self.store.find_one("bookmarks", q) is not None:
            return False
        if self.get_feature(sae_name, sae_series, feature_index) is None:
            raise ValueError(f"Feature {feature_index} not found for SAE {sae_name}/{sae_series}")
        self.store.insert_one("bookmarks", {**q, "created_at": datetime.now(timezone.utc).isoformat(), "tags": tags or [], "notes": notes})
        return True

    def remove_bookmark(self, sae_name: str, sae_series: str, feature_index: int) -> bool:
        return self.store.delete_many("bookmarks", {"sae_name": sae_name, "sae_series": sae_series, "feature_index": feature_index}) > 0

    def is_bookmarked(self, sae_name: str, sae_series: str, feature_index: int) -> bool:
        return self.store.find_one("bookmarks", {"sae_name": sae_name, "sae_series": sae_series, "feature_index": feature_index}) is not None

    def get_bookmark(self, sae_name: str, sae_series: str, feature_index: int) -> Optional[BookmarkRecord]:
        d = self.store.find_one("bookmarks", {"sae_name": sae_name, "sae_series": sae_series, "feature_index": feature_index})
        return BookmarkRecord.model_validate(d) if d else None

    def list_bookmarks(self, sae_name: str | None = None, sae_series: str | None = None, tags: list[str] | None = None,
                       limit: int | None = None, skip: int = 0) -> list[BookmarkRecord]:  # fmt: skip
        q = ({"sae_name": sae_name} if sae_name else {}) | ({"sae_series": sae_series} if sae_series else {})
        recs = [BookmarkRecord.model_validate(d) for d in self.store.find("bookmarks", q)]
        if tags:
            recs = [r for r in recs if set(tags) & set(r.tags)]
        recs.sort(key=lambda r: r.created_at, reverse=True)
        return recs[skip : (skip + limit) if limit is not None else None]

    def update_bookmark(self, sae_name: str, sae_series: str, feature_index: int, tags: list[str] | None = None, notes: str | None = None) -> bool:
        upd = ({"tags": tags} if tags is not None else {}) | ({"notes": notes} if notes is not None else {})
        if not upd:
            return False
        return self.store.update_one("bookmarks", {"sae_name": sae_name, "sae_series": sae_series, "feature_index": feature_index}, upd)

    def get_bookmark_count(self, sae_name: Optional[str] = None, sae_series: Optional[str] = None) -> int:
        return self.store.count("bookmarks", ({"sae_name": sae_name} if sae_name else {}) | ({"sae_series": sae_series} if sae_series else {}))

    # ---- dictionary sets -----------------------------------------------------------------------
    def add_sae_set(self, name: str, sae_series: str, sae_names: list[str]):
        self.store.update_one("sae_sets", {"name": name}, {"sae_series": sae_series, "sae_names": sae_names}, upsert=True)

    def get_sae_set(self, name: str) -> Optional[SAESetRecord]:
        d = self.store.find_one("sae_sets", {"name": name})
        return SAESetRecord.model_validate(d) if d else None

    def list_sae_sets(self) -> list[SAESetRecord]:
        return [SAESetRecord.model_validate(d) for d in self.store.find("sae_sets", {})]

    def remove_sae_set(self, name: str, sae_series: str):
        self.store.delete_many("sae_sets", {"name": name, "sae_series": sae_series})

    # ---- circuits ----------------------------------------------------------------------------
    def create_circuit(self, sae_set_name: str, sae_series: str, prompt: str, input: Any, config: CircuitConfig,
                       name: str | None = None, group: str | None = None, parent_id: str | None = None) -> str:  # fmt: skip
        cid = uuid.uuid4().hex
        inp = input.model_dump() if isinstance(input, BaseModel) else input
        self.store.insert_one("circuits", {
            "id": cid, "name": name, "group": group, "sae_set_name": sae_set_name, "sae_series": sae_series, "prompt": prompt,
            "input": inp, "config": config.model_dump(), "created_at": datetime.now(timezone.utc).isoformat(),
            "parent_id": parent_id, "status": CircuitStatus.PENDING, "progress": 0.0, "progress_phase": None,
            "error_message": None,
        })  # fmt: skip
        return cid

    def get_circuit(self, circuit_id: str) -> Optional[CircuitRecord]:
        d = self.store.find_one("circuits", {"id": circuit_id})
        return CircuitRecord.model_validate({k: v for k, v in d.items() if k not in ("_id", "attribution")}) if d else None

    def list_circuits(self, sae_series: str | None = None, group: str | None = None, limit: int | None = None, skip: int = 0) -> list[CircuitRecord]:
        q = ({"sae_series": sae_series} if sae_series else {}) | ({"group": group} if group else {})
        recs = [CircuitRecord.model_validate({k: v for k, v in d.items() if k not in ("_id", "attribution")}) for d in self.store.find("circuits", q)]
        recs.sort(key=lambda r: r.created_at, reverse=True)
        return recs[skip : (skip + limit) if limit is not None else None]

    def update_circuits_group(self, circuit_ids: list[str], group: Optional[str]) -> int:
        return sum(1 for cid in circuit_ids if self.store.update_one("circuits", {"id": cid}, {"group": group}))

    def update_circuit(self, circuit_id: str, update_data: dict[str, Any]) -> bool:
        return self.store.update_one("circuits", {"id": circuit_id}, update_data)

    def delete_circuit(self, circuit_id: str) -> bool:
        d = self.store.find_one("circuits", {"id": circuit_id})
        if d is None:
            return False
        self._remove_gridfs_objs(d.get("attribution"))
        return self.store.delete_many("circuits", {"id": circuit_id}) > 0

    def update_circuit_progress(self, circuit_id: str, progress: float, progress_phase: str | None = None) -> bool:
        return self.update_circuit(circuit_id, {"progress": progress, "progress_phase": progress_phase})

    def update_circuit_status(self, circuit_id: str, status: str, error_message: str | None = None) -> bool:
        upd: dict[str, Any] = {"status": status, "error_message": error_message}
        if status == CircuitStatus.COMPLETED:
            upd["progress"] = 100.0
        return self.update_circuit(circuit_id, upd)

    def store_attribution(self, circuit_id: str, attribution: Any) -> bool:
        """Serialise an ``AttributionResult`` with the versioned serializer and attach it to the circuit."""
        from .core.serialize import dumps

        blob = self.store.put_blob(dumps(attribution))
        return self.update_circuit(circuit_id, {"attribution": {"__blob__": blob}})

    def load_attribution(self, circuit_id: str, device: torch.device | str = "cpu"):
        from .circuits.attribution import AttributionResult
        from .core.serialize import loads

        d = self.store.find_one("circuits", {"id": circuit_id})
        if d is None or not d.get("attribution"):
            return None
        return loads(self.store.get_blob(d["attribution"]["__blob__"]), AttributionResult, device=device)

    def get_circuit_status(self, circuit_id: str) -> Optional[dict[str, Any]]:
        d = self.store.find_one("circuits", {"id": circuit_id})
        if d is None:
            return None
        return {k: d.get(k) for k in ("status", "progress", "progress_phase", "error_message")}
