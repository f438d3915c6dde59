"""Run a test function on several ranks without a cluster.

``@distributed_test(nproc_per_node=N, backend="gloo")``: when the decorated test is called by pytest (no
``RANK`` in the environment) it spawns N child processes, each of which sets the rendezvous environment
(127.0.0.1), initialises the process group, re-imports the test module by path and calls the same function;
the parent fails if any child fails. Same idea as testing/distributed.py:11-84 of the reference project.
"""

from __future__ import annotations

import functools
import importlib.util
import inspect
import os
import socket
import sys
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _child(rank: int, world: int, port: int, backend: str, module_path: str, func_name: str, args, kwargs, errq):
    os.environ.update(
        MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank)
    )
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
        else:
            # one thread per rank: CPU reductions then add in the same order whatever the load of the machine, so a
            # comparison between a sharded and an unsharded run does not depend on how many cores were free
            torch.set_num_threads(1)
        dist.init_process_group(backend, rank=rank, world_size=world)
        spec = importlib.util.spec_from_file_location("_dist_test_module", module_path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules["_dist_test_module"] = mod
        spec.loader.exec_module(mod)
        fn = getattr(mod, func_name)
        getattr(fn, "__wrapped_test__", fn)(*args, **kwargs)
        dist.barrier()
    except Exception:  # noqa: BLE001
        errq.put((rank, traceback.format_exc()))
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def distributed_test(nproc_per_node: int = 2, backend: str = "gloo"):
    def decorator(func):
        module_path = os.path.abspath(inspect.getfile(func))

        @functools.wraps(func)
        def wrapper(*args, **kwargs):
            if "RANK" in os.environ:  # already inside a spawned rank
                return func(*args, **kwargs)
            ctx = mp.get_context("spawn")
            errq = ctx.Queue()
            port = _free_port()
            procs = [
                ctx.Process(target=_child, args=(r, nproc_per_node, port, backend, module_path, func.__name__, args, kwargs, errq))
                for r in range(nproc_per_node)
            ]
            for p in procs:
                p.start()
            for p in procs:
                p.join(timeout=600)
            failed = [p for p in procs if p.exitcode != 0]
            for p in procs:
                if p.is_alive():
                    p.kill()
            if failed:
                msgs = []
                while not errq.empty():
                    msgs.append("rank %d:\n%s" % errq.get())
                raise AssertionError("distributed test failed\n" + "\n".join(msgs))

        wrapper.__wrapped_test__ = func
        return wrapper

    return decorator
