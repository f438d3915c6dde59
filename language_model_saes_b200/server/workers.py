"""Run model work either in this process or on a pool of worker processes, one per GPU
(server/logic/workers.py of the reference project).

``@distributed`` turns ``fn(..., device_mesh=None)`` into ``async fn(...)``. With ``NUM_WORKERS=0`` the call runs on a
thread of the HTTP process. Otherwise the call is sent to EVERY worker (they form one ``("model",)`` mesh and execute
the same function on their shards) and rank 0's return value is the result. Results are matched to callers by task
id through per-task futures filled by one reader thread, instead of polling a shared queue.
"""

from __future__ import annotations

import asyncio
import importlib
import inspect
import os
import threading
import uuid
from functools import wraps
from typing import Any, Callable, Optional


class DistributedWorkerRegistry:
    _workers: list = []
    _task_queues: list = []
    _result_queue: Any = None
    _num_workers: int = 0
    _initialized: bool = False
    _functions: dict[tuple[str, str], Callable] = {}
    _pending: dict[str, "asyncio.Future"] = {}
    _reader: Optional[threading.Thread] = None

    @classmethod
    def initialize(cls, num_workers: int, master_port: int = 29500):
        if cls._initialized:
            return
        if os.environ.get("IS_WORKER") is not None:
            raise RuntimeError("Cannot initialize worker registry from a worker process")
        cls._num_workers = num_workers
        if num_workers > 0:
            import torch.multiprocessing as mp

            ctx = mp.get_context("spawn")
            cls._result_queue = ctx.Queue()
            cls._task_queues = [ctx.Queue() for _ in range(num_workers)]
            for rank in range(num_workers):
                p = ctx.Process(target=cls._worker_loop, args=(rank, num_workers, cls._task_queues[rank], cls._result_queue, master_port), daemon=False)
                p.start()
                cls._workers.append(p)
            cls._reader = threading.Thread(target=cls._read_results, daemon=True)
            cls._reader.start()
        cls._initialized = True

    @classmethod
    def _read_results(cls):
        while True:
            item = cls._result_queue.get()
            if item is None:
                return
            task_id, result = item
            fut = cls._pending.pop(task_id, None)
            if fut is not None and not fut.done():
                loop = fut.get_loop()
                if isinstance(result, Exception):
                    loop.call_soon_threadsafe(fut.set_exception, result)
                else:
                    loop.call_soon_threadsafe(fut.set_result, result)

    @classmethod
    def _worker_loop(cls, rank: int, world_size: int, task_queue, result_queue, master_port: int):
        import torch
        import torch.distributed as dist

        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(master_port), RANK=str(rank), LOCAL_RANK=str(rank),
                          WORLD_SIZE=str(world_size), IS_WORKER="1")  # fmt: skip
        cuda = torch.cuda.is_available()
        if cuda:
            torch.cuda.set_device(rank)
        mesh = None
        if world_size > 1:
            from ..parallel.mesh import build_mesh

            dist.init_process_group(backend="nccl" if cuda else "gloo")
            mesh = build_mesh("cuda" if cuda else "cpu", (world_size,), ("model",))
        while True:
            task = task_queue.get()
            if task is None:
                break
            task_id, module, name, args, kwargs = task
            try:
                if (module, name) not in cls._functions:
                    importlib.import_module(module)
                fn = cls._functions.get((module, name))
                if fn is None:
                    raise ValueError(f"Function {name} not registered (module: {module})")
                if "device_mesh" in inspect.signature(fn).parameters:
                    kwargs = {**kwargs, "device_mesh": mesh}
                result = fn(*args, **kwargs)
                if rank == 0:
                    result_queue.put((task_id, result))
            except Exception as e:  # noqa: BLE001 - reported to the caller
                if rank == 0:
                    result_queue.put((task_id, RuntimeError(f"{type(e).__name__}: {e}")))
        if world_size > 1:
            dist.destroy_process_group()

    @classmethod
    def register_function(cls, module: str, name: str, fn: Callable):
        cls._functions[(module, name)] = fn

    @classmethod
    def submit_to_all_workers(cls, module: str, name: str, *args, **kwargs) -> "asyncio.Future":
        task_id = uuid.uuid4().hex
        fut = asyncio.get_running_loop().create_future()
        cls._pending[task_id] = fut
        for q in cls._task_queues:
            q.put((task_id, module, name, args, kwargs))
        return fut

    @classmethod
    def shutdown(cls):
        if cls._num_workers > 0:
            for q in cls._task_queues:
                q.put(None)
            for w in cls._workers:
                w.join(timeout=5)
                if w.is_alive():
                    w.terminate()
            if cls._result_queue is not None:
                cls._result_queue.put(None)
            cls._workers, cls._task_queues, cls._result_queue, cls._reader = [], [], None, None
        cls._pending.clear()
        cls._initialized = False
        cls._num_workers = 0


def distributed(fn: Callable) -> Callable:
    DistributedWorkerRegistry.register_function(fn.__module__, fn.__name__, fn)
    sig = inspect.signature(fn)
    takes_mesh = "device_mesh" in sig.parameters

    @wraps(fn)
    async def call(*args, timeout: float = 120.0, **kwargs):
        reg = DistributedWorkerRegistry
        if not reg._initialized:
            raise RuntimeError("Workers not initialized. Call DistributedWorkerRegistry.initialize(num_workers) first.")
        if reg._num_workers == 0:
            kw = {**kwargs, "device_mesh": None} if takes_mesh else kwargs
            if asyncio.iscoroutinefunction(fn):
                return await fn(*args, **kw)
            return await asyncio.to_thread(fn, *args, **kw)  # long torch work must not block the event loop
        return await asyncio.wait_for(reg.submit_to_all_workers(fn.__module__, fn.__name__, *args, **kwargs), timeout)

    if takes_mesh:
        call.__signature__ = sig.replace(parameters=[p for p in sig.parameters.values() if p.name != "device_mesh"])  # type: ignore[attr-defined]
    call.__wrapped_sync__ = fn  # type: ignore[attr-defined]
    return call
