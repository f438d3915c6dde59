"""The HTTP server against the local file store with a tiny model: feature browsing, inference, bookmarks, admin and a
complete circuit job (create -> background attribution -> pruned graph -> QK node)."""

import importlib
import json
import sys

import msgpack
import numpy as np
import pytest
import torch
from conftest import tiny_lm_config

from language_model_saes_b200.models.lorsa import LorsaConfig, LowRankSparseAttention
from language_model_saes_b200.models.sae import SAEConfig, SparseAutoEncoder


@pytest.fixture(scope="module")
def server(tiny_lm_workspace, tmp_path_factory):
    from fastapi.testclient import TestClient

    root = tmp_path_factory.mktemp("server")
    mp = pytest.MonkeyPatch()
    mp.setenv("MONGO_URI", f"file://{root / 'db'}")
    mp.setenv("MONGO_DB", "srv")
    mp.setenv("SAE_SERIES", "ser")
    mp.setenv("NUM_WORKERS", "0")
    for name in [m for m in sys.modules if m.startswith("language_model_saes_b200.server")]:
        del sys.modules[name]
    app_mod = importlib.import_module("language_model_saes_b200.server.app")
    C = importlib.import_module("language_model_saes_b200.server.config")
    client = C.client
    from language_model_saes_b200.config import DatasetConfig

    client.add_dataset("toy", DatasetConfig(dataset_name_or_path=str(tiny_lm_workspace / "data"), is_dataset_on_disk=True))
    client.add_model("tiny", tiny_lm_config(tiny_lm_workspace))
    torch.manual_seed(0)
    names = []
    for layer in range(2):
        tc = SparseAutoEncoder(SAEConfig(hook_point_in=f"blocks.{layer}.ln2.hook_normalized", hook_point_out=f"blocks.{layer}.hook_mlp_out",
                                         d_model=16, expansion_factor=2, act_fn="topk", top_k=4, norm_activation="inference"))  # fmt: skip
        tc.init_parameters(encoder_uniform_bound=0.5, decoder_uniform_bound=0.5)
        lo = LowRankSparseAttention(LorsaConfig(hook_point_in=f"blocks.{layer}.ln1.hook_normalized", hook_point_out=f"blocks.{layer}.hook_attn_out",
                                                d_model=16, expansion_factor=2, n_qk_heads=4, d_qk_head=8, rotary_dim=8, n_ctx=32, act_fn="topk",
                                                top_k=4, norm_activation="inference"))  # fmt: skip
        lo.init_parameters(encoder_uniform_bound=0.5, decoder_uniform_bound=0.5)
        for kind, m in (("tc", tc), ("lorsa", lo)):
            path = root / f"{kind}{layer}"
            m.save_pretrained(path)
            m.cfg.save_hyperparameters(path)
            client.create_sae(f"{kind}-L{layer}", "ser", str(path), m.cfg, model_name="tiny")
            names.append(f"{kind}-L{layer}")
    acts = np.zeros((2, 16), dtype=np.float32)
    acts[0, 3], acts[0, 4], acts[1, 7] = 2.0, 0.5, 1.0
    r, c = np.nonzero(acts)
    rec = {"act_times": 3, "n_analyzed_tokens": 100, "max_feature_acts": 2.0, "samplings": [{
        "name": "top_activations", "feature_acts_indices": np.stack([r, c]).astype(np.float32), "feature_acts_values": acts[r, c],
        "context_idx": np.array([5, 9]), "dataset_name": ["toy", "toy"], "model_name": ["tiny", "tiny"]}]}  # fmt: skip
    for n in names:
        client.add_feature_analysis("default", n, "ser", [rec, {**rec, "act_times": 0, "max_feature_acts": 0.0}], start_idx=0)
    with TestClient(app_mod.app) as http:
        yield http, client, names
    mp.undo()


def _unpack(resp):
    assert resp.status_code == 200, resp.text
    return msgpack.unpackb(resp.content, raw=False)


def test_dictionary_and_feature_endpoints(server):
    http, client, names = server
    assert http.get("/dictionaries").json() == sorted(names, key=lambda n: (n.split("-")[0], int(n[-1])))
    d = _unpack(http.get("/dictionaries/tc-L0"))
    assert d["alive_feature_count"] == 1 and d["feature_activation_times_histogram"][0]["type"] == "bar"
    f = _unpack(http.get("/dictionaries/tc-L0/features/0"))
    assert f["feature_index"] == 0 and f["act_times"] == 3 and f["is_bookmarked"] is False
    sample = f["sample_groups"][0]["samples"][0]
    assert sample["feature_acts_indices"] == [3, 4] and sample["feature_acts_values"] == [2.0, 0.5] and "text" in sample and len(sample["origins"]) > 4
    assert _unpack(http.get("/dictionaries/tc-L0/features/random"))["feature_index"] == 0
    assert http.get("/dictionaries/tc-L0/features/abc").status_code == 400
    assert http.get("/dictionaries/tc-L0/features/999").status_code == 404
    lst = http.get("/dictionaries/tc-L0/features", params={"start": 0, "end": 2, "visible_range": 2}).json()
    assert len(lst) == 2 and lst[0]["samples"][0]["token_offset"] == 1 and len(lst[0]["samples"][0]["origins"]) <= 4
    assert http.get("/dictionaries/tc-L0/features/0/samplings").json() == [{"name": "top_activations", "length": 2}]
    part = _unpack(http.get("/dictionaries/tc-L0/features/0/sampling/top_activations", params={"start": 1, "length": 1}))
    assert len(part) == 1 and part[0]["feature_acts_indices"] == [7]
    assert http.get("/dictionaries/tc-L0/analyses").json() == ["default"]
    assert http.get("/dictionaries/tc-L0/features/count").json() == {"count": 1}
    assert http.get("/dictionaries/tc-L0/features/count", params={"metric_filters": "{bad"}).status_code == 400


def test_inference_interpretation_bookmarks_admin(server):
    http, client, names = server
    inf = _unpack(http.post("/dictionaries/tc-L0/features/0/infer", params={"text": "the cat sat on a mat"}))
    assert inf["text"] == "the cat sat on a mat" and len(inf["origins"]) == 7 and len(inf["feature_acts_indices"]) == len(inf["feature_acts_values"])
    top = _unpack(http.post("/dictionaries/tc-L0/inference", params={"text": "the cat sat on a mat", "max_features": 3}))
    assert all("inference" in t and "feature_index" in t for t in top)
    r = http.put("/dictionaries/tc-L0/features/0/interpretation", json={"text": "cats"})
    assert r.status_code == 200 and client.get_feature("tc-L0", "ser", 0).interpretation == {"text": "cats"}
    assert http.post("/dictionaries/tc-L0/features/0/bookmark").status_code == 200
    assert http.post("/dictionaries/tc-L0/features/0/bookmark").status_code == 409
    assert http.get("/dictionaries/tc-L0/features/0/bookmark").json() == {"is_bookmarked": True}
    marks = http.get("/bookmarks", params={"include_features": True}).json()
    assert marks["total_count"] == 1 and marks["bookmarks"][0]["feature"]["interpretation"] == {"text": "cats"}
    assert http.delete("/dictionaries/tc-L0/features/0/bookmark").status_code == 200
    assert http.delete("/dictionaries/tc-L0/features/0/bookmark").status_code == 404
    stats = http.get("/admin/stats").json()
    assert stats["sae_count"] == 4 and stats["sae_series"] == "ser"
    saes = http.get("/admin/saes", params={"search": "lorsa"}).json()
    assert saes["total_count"] == 2 and saes["saes"][0]["feature_count"] == 32
    assert http.put("/admin/saes/nope", json={"path": "x"}).status_code == 404


def test_circuit_job_roundtrip(server):
    http, client, names = server
    assert http.post("/sae-sets", json={"name": "all", "sae_names": names}).status_code == 200
    assert http.post("/sae-sets", json={"name": "all", "sae_names": names}).status_code == 409
    assert http.get("/sae-sets").json() == ["all"]
    prev = http.post("/preview", json={"input": {"input_type": "plain_text", "text": "the cat sat"}, "sae_set_name": "all"}).json()
    assert prev["prompt"] == "the cat sat" and len(prev["next_tokens"]) == 5
    req = {"input": {"input_type": "plain_text", "text": "the cat sat on a"}, "name": "c1", "max_feature_nodes": 24, "qk_tracing_topk": 3,
           "max_n_logits": 2, "desired_logit_prob": 0.5}  # fmt: skip
    made = http.post("/circuits", params={"sae_set_name": "all"}, json=req).json()
    cid = made["circuit_id"]
    status = http.get(f"/circuits/{cid}/status").json()
    assert status["status"] == "completed", status
    got = http.get(f"/circuits/{cid}", params={"node_threshold": 0.8, "edge_threshold": 0.95}).json()
    graph = got["graph_data"]
    kinds = {n["feature_type"] for n in graph["nodes"]}
    assert "logit" in kinds and "embedding" in kinds and ({"lorsa", "cross layer transcoder"} & kinds)
    ids = {n["node_id"] for n in graph["nodes"]}
    assert len(ids) == len(graph["nodes"]) and all(l["source"] in ids and l["target"] in ids for l in graph["links"])
    assert graph["metadata"]["prompt_tokens"] == ["the", "cat", "sat", "on", "a"]
    feat = next(n for n in graph["nodes"] if n["feature_type"] in ("lorsa", "cross layer transcoder"))
    assert feat["feature"]["dictionary_name"] == feat["sae_name"]
    traced = [n for n in graph["nodes"] if n.get("qk_tracing_results")]
    if traced:
        qk = http.get(f"/circuits/{cid}/qk/{traced[0]['node_id']}", params={"node_threshold": 0.8, "edge_threshold": 0.95}).json()
        assert qk["target_node"]["node_id"] == traced[0]["node_id"]
    assert http.get(f"/circuits/{cid}/qk/nope").status_code == 404
    assert [c["name"] for c in http.get("/circuits").json()] == ["c1"]
    assert http.put(f"/admin/circuits/{cid}", json={"group": "g"}).status_code == 200
    assert http.get("/admin/circuits").json()["circuits"][0]["group"] == "g"
    assert http.delete(f"/circuits/{cid}").status_code == 200
    assert http.get(f"/circuits/{cid}").status_code == 404


def test_ui_pages_are_served_and_call_existing_routes(server):
    """The browser pages are static files next to the server; every API path they name is a route of the app."""
    import re

    http, _, names = server
    page = http.get("/ui/index.html")
    assert page.status_code == 200 and 'src="pages.js"' in page.text
    scripts = [http.get(f"/ui/{name}") for name in re.findall(r'<script src="([^"]+)">', page.text)]
    assert len(scripts) >= 5 and all(s.status_code == 200 for s in scripts)
    routes = {(m, r.path) for r in http.app.routes for m in getattr(r, "methods", ())}
    as_route = lambda p: re.sub(r"\$\{[^}]*\}", "{}", p.split("?")[0])  # noqa: E731
    known = {(m, re.sub(r"\{[^}]*\}", "{}", p)) for m, p in routes}
    called = set()
    for text in [s.text for s in scripts]:
        for m in re.finditer(r"api\((`|\")(/[^`\"]*)\1(?:\s*\+\s*query\(\{[^}]*\}\))?(?:,\s*(?:jsonOpts\(\"(\w+)\"|\{\s*method:\s*(?:\"(\w+)\"|[^}]*\?\s*\"(\w+)\"\s*:\s*\"(\w+)\")))?", text):
            methods = [g for g in m.groups()[2:] if g] or ["GET"]
            called |= {(meth, as_route(m.group(2))) for meth in methods}
    assert len(called) > 20
    called = {(m, p.replace("/features/random", "/features/{}")) for m, p in called}  # "random" stands for a feature index
    missing = sorted(c for c in called if c not in known)
    assert not missing, missing
    # the pages' data sources answer for the fixtures of this module
    assert http.get("/admin/stats").json()["sae_count"] == len(names)
    assert http.get(f"/dictionaries/{names[0]}/features", params={"start": 0, "end": 2, "sample_length": 1}).status_code == 200


def test_management_routes_rename_filter_and_delete(server):
    """Runs last: it renames and deletes what the other tests read. Feature metrics and their filters, bookmark notes, renaming
    a dictionary (its features, analyses, bookmarks and sets follow), renaming and deleting a set, grouping circuits."""
    http, client, names = server
    # metrics stored on features, and the filters of count / random
    client.update_feature("tc-L1", 0, {"metric": {"score": 0.9, "depth": 2.0}}, sae_series="ser")
    client.update_feature("tc-L1", 1, {"metric": {"score": 0.1}}, sae_series="ser")
    assert http.get("/dictionaries/tc-L1/metrics").json() == {"metrics": ["depth", "score"]}
    count = lambda f: http.get("/dictionaries/tc-L1/features/count", params={"metric_filters": json.dumps(f)}).json()["count"]  # noqa: E731
    assert count({"score": {"$gte": 0.5}}) == 1
    assert count({"score": {"$gte": 0.95}}) == 0
    assert count({"score": {"$lte": 0.5}}) == 0  # feature 1 passes the filter but never fired
    hit = http.get("/dictionaries/tc-L1/features/random", params={"metric_filters": json.dumps({"score": {"$gte": 0.5}})})
    assert _unpack(hit)["feature_index"] == 0
    miss = http.get("/dictionaries/tc-L1/features/random", params={"metric_filters": json.dumps({"score": {"$gte": 0.95}})})
    assert miss.status_code == 404
    # bookmark notes and tags
    assert http.put("/dictionaries/tc-L1/features/0/bookmark", params={"notes": "n"}).status_code == 404
    assert http.post("/dictionaries/tc-L1/features/0/bookmark").status_code == 200
    # the tag list is the JSON body, the notes a query parameter
    assert http.put("/dictionaries/tc-L1/features/0/bookmark", params={"notes": "look again"}, json=["a", "b"]).status_code == 200
    mark = http.get("/bookmarks", params={"sae_name": "tc-L1"}).json()["bookmarks"][0]
    assert mark["notes"] == "look again" and mark["tags"] == ["a", "b"]
    # sets: create, edit, rename, clash, delete
    if "all" not in http.get("/sae-sets").json():
        assert http.post("/sae-sets", json={"name": "all", "sae_names": names}).status_code == 200
    assert http.post("/sae-sets", json={"name": "mlp", "sae_names": ["tc-L0", "tc-L1"]}).status_code == 200
    assert [s["name"] for s in http.get("/admin/sae-sets").json()] == ["all", "mlp"]
    assert http.put("/admin/sae-sets/mlp", json={"new_name": "all"}).status_code == 409
    assert http.put("/admin/sae-sets/mlp", json={}).json() == {"message": "No updates provided"}
    assert http.put("/admin/sae-sets/nope", json={"new_name": "x"}).status_code == 404
    assert http.put("/admin/sae-sets/mlp", json={"new_name": "transcoders", "sae_names": ["tc-L1"]}).status_code == 200
    sets = {s["name"]: s["sae_names"] for s in http.get("/admin/sae-sets").json()}
    assert sets["transcoders"] == ["tc-L1"] and "mlp" not in sets
    # renaming a dictionary carries its records along
    assert http.put("/admin/saes/tc-L1", json={"new_name": "tc-L0"}).status_code == 409
    assert http.put("/admin/saes/tc-L1", json={"new_name": "mlp-L1", "model_name": "tiny"}).status_code == 200
    assert "mlp-L1" in http.get("/dictionaries").json() and "tc-L1" not in http.get("/dictionaries").json()
    assert _unpack(http.get("/dictionaries/mlp-L1/features/0"))["is_bookmarked"] is True
    assert http.get("/dictionaries/mlp-L1/analyses").json() == ["default"]
    sets = {s["name"]: s["sae_names"] for s in http.get("/admin/sae-sets").json()}
    assert sets["transcoders"] == ["mlp-L1"] and "mlp-L1" in sets["all"] and "tc-L1" not in sets["all"]
    assert _unpack(http.post("/dictionaries/mlp-L1/features/0/infer", params={"text": "the cat"}))["text"] == "the cat"
    # deleting it removes its features and analyses
    assert http.delete("/admin/saes/mlp-L1").status_code == 200
    assert http.delete("/admin/saes/mlp-L1").status_code == 404
    assert http.get("/dictionaries/mlp-L1/features/0").status_code == 404
    assert http.get("/admin/stats").json()["sae_count"] == 3
    assert http.delete("/admin/sae-sets/transcoders").status_code == 200
    assert http.delete("/admin/sae-sets/transcoders").status_code == 404
    # circuits in a group
    left = [n for n in names if n != "tc-L1"]
    assert http.put("/admin/sae-sets/all", json={"sae_names": left}).status_code == 200
    req = {"input": {"input_type": "plain_text", "text": "a cat"}, "name": "c2", "max_feature_nodes": 8, "max_n_logits": 1, "desired_logit_prob": 0.3}
    ids = [http.post("/circuits", params={"sae_set_name": "all"}, json={**req, "name": f"c{i}"}).json()["circuit_id"] for i in (2, 3)]
    assert http.post("/admin/circuits/bulk-group", json={"circuit_ids": ids + ["missing"], "group": "batch"}).json() == {"message": "Updated 2 circuits"}
    rows = http.get("/admin/circuits").json()
    assert rows["total_count"] == 2 and {c["group"] for c in rows["circuits"]} == {"batch"}
    assert http.put(f"/admin/circuits/{ids[0]}", json={"name": "renamed"}).status_code == 200
    assert http.put("/admin/circuits/missing", json={"name": "x"}).status_code == 404
    assert "renamed" in [c["name"] for c in http.get("/circuits").json()]
