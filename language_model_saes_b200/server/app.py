"""FastAPI application (server/app.py of the reference project). Environment: ``NUM_WORKERS`` (0 = run model work in
this process), ``PRELOAD_MODELS`` / ``PRELOAD_SAES`` (comma-separated names), ``PRELOAD_CIRCUITS``
(``id[:node_threshold[:edge_threshold]],...``), ``SAE_SERIES``, ``MONGO_URI``, ``MONGO_DB``.

Run with ``uvicorn language_model_saes_b200.server.app:app``.
"""

from __future__ import annotations

import asyncio
import os
from contextlib import asynccontextmanager

import torch
from fastapi import FastAPI, Response
from fastapi.middleware.cors import CORSMiddleware
from fastapi.middleware.gzip import GZipMiddleware

from .loaders import get_dataset, get_model, get_sae
from .routers import admin, bookmarks, circuits, dictionaries
from .routers.circuits import load_circuit_graph
from .workers import DistributedWorkerRegistry, distributed


@distributed
def workers_on_mount(preload_models: list[str], preload_saes: list[str], device_mesh=None):
    for m in preload_models:
        get_model(name=m, device_mesh=device_mesh)
    for s in preload_saes:
        get_sae(name=s, device_mesh=device_mesh)


@distributed
def workers_on_unmount(device_mesh=None):
    for cache in (get_model, get_dataset, get_sae, load_circuit_graph):
        cache.cache_clear()


def _names(var: str) -> list[str]:
    return [n for n in os.environ.get(var, "").strip().split(",") if n]


@asynccontextmanager
async def lifespan(app: FastAPI):
    DistributedWorkerRegistry.initialize(num_workers=int(os.environ.get("NUM_WORKERS", "0")))
    models = _names("PRELOAD_MODELS")
    task = asyncio.create_task(workers_on_mount(models, _names("PRELOAD_SAES"), timeout=3600.0))
    for m in models:
        get_model(name=m, device_mesh=None)
    for entry in _names("PRELOAD_CIRCUITS"):
        parts = entry.split(":")
        load_circuit_graph(circuit_id=parts[0], node_threshold=float(parts[1]) if len(parts) > 1 else 0.6,
                           edge_threshold=float(parts[2]) if len(parts) > 2 else 0.8)  # fmt: skip
    await task
    yield
    await workers_on_unmount()
    DistributedWorkerRegistry.shutdown()


def create_app() -> FastAPI:
    app = FastAPI(lifespan=lifespan, title="language-model-saes-b200")
    app.add_middleware(GZipMiddleware, minimum_size=1000)
    app.add_middleware(CORSMiddleware, allow_origins=["*"], allow_credentials=True, allow_methods=["*"], allow_headers=["*"])

    @app.exception_handler(AssertionError)
    async def assertion_error_handler(request, exc):
        return Response(content=str(exc), status_code=400)

    @app.exception_handler(torch.cuda.OutOfMemoryError)
    async def oom_error_handler(request, exc):
        for cache in (get_model, get_dataset, get_sae):
            cache.cache_clear()
        return Response(content="CUDA Out of memory", status_code=500)

    for r in (admin.router, dictionaries.router, circuits.router, bookmarks.router):
        app.include_router(r)
    ui_dir = os.path.join(os.path.dirname(__file__), "ui")
    if os.path.isdir(ui_dir):
        from fastapi.staticfiles import StaticFiles

        app.mount("/ui", StaticFiles(directory=ui_dir, html=True), name="ui")
    return app


app = create_app()
