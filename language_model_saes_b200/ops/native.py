"""Build and load the sm_100a extension that holds every hand-written kernel of this package.

The shared object is built in-tree (``ops/_native_build/_lmsae_native.so``) so that a checkout which was
built once can be copied to a GPU machine and used without a compiler run. ``load()`` returns the
extension module; on a machine with a CUDA device a missing or unloadable extension is an error (the ops
never fall back silently to eager PyTorch there), on a CPU-only machine it returns ``None`` and the ops use
their plain PyTorch definitions, which are also the numerical oracles in the tests.
"""

from __future__ import annotations

import importlib.util
import os
import sys
import threading
from pathlib import Path
from types import ModuleType

import torch

_NAME = "_lmsae_native"
_CSRC = Path(__file__).resolve().parent / "csrc"
# LMSAE_NATIVE_CHECKED=1 selects the bounds-checked debug build (compiled with -DLMSAE_BOUNDS_CHECK into a directory of its
# own): data-dependent indices of the gather kernels are compared with their limits, violations are recorded (see
# ``bounds_report`` of the extension) and clamped instead of read out of bounds.
_CHECKED = os.environ.get("LMSAE_NATIVE_CHECKED", "0") == "1"
_BUILD_DIR = Path(__file__).resolve().parent / ("_native_build_checked" if _CHECKED else "_native_build")
_SOURCES = ["binding.cpp", "encoder_gemm.cu", "topk_merge.cu", "sparse_ops.cu", "comm_ops.cu", "no_alloc.cu", "jumprelu.cu", "clt_ops.cu", "select_ops.cu", "attention.cu", "rotary.cu"]
_CUDA_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-U__CUDA_NO_HALF_OPERATORS__",
    "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__",
]

_lock = threading.Lock()
_module: ModuleType | None = None
_load_error: Exception | None = None


def sources() -> list[str]:
    return [str(_CSRC / s) for s in _SOURCES if (_CSRC / s).exists()]


def so_path() -> Path:
    return _BUILD_DIR / f"{_NAME}.so"


def _source_hash() -> str:
    import hashlib

    h = hashlib.sha256()
    deps = sorted(list(_CSRC.glob("*.cu")) + list(_CSRC.glob("*.cuh")) + list(_CSRC.glob("*.h")) + list(_CSRC.glob("*.cpp")))
    for p in deps:
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(_CUDA_FLAGS + (["-DLMSAE_BOUNDS_CHECK"] if _CHECKED else [])).encode())
    return h.hexdigest()


def _hash_path() -> Path:
    return _BUILD_DIR / f"{_NAME}.sha256"


def _is_stale() -> bool:
    """The .so is current when the recorded hash of the sources it was built from matches (file times are
    not reliable after a checkout has been copied to another machine)."""
    if not so_path().exists() or not _hash_path().exists():
        return True
    return _hash_path().read_text().strip() != _source_hash()


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile the extension for sm_100a with nvcc (works without a GPU) and return the .so path."""
    from torch.utils import cpp_extension

    _BUILD_DIR.mkdir(parents=True, exist_ok=True)
    if not force and not _is_stale():
        return so_path()
    os.environ.setdefault("MAX_JOBS", str(min(8, os.cpu_count() or 4)))
    # The -gencode flag above is what selects the architecture; this only silences torch's own probing
    # on machines without a GPU.
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    cpp_extension.load(
        name=_NAME,
        sources=sources(),
        extra_cflags=["-O3", "-std=c++17"] + (["-DLMSAE_BOUNDS_CHECK"] if _CHECKED else []),
        extra_cuda_cflags=_CUDA_FLAGS + (["-DLMSAE_BOUNDS_CHECK"] if _CHECKED else []),
        extra_ldflags=["-lcuda"],
        build_directory=str(_BUILD_DIR),
        with_cuda=True,
        verbose=verbose,
        is_python_module=False,
    )
    assert so_path().exists(), f"build finished but {so_path()} is missing"
    _hash_path().write_text(_source_hash())
    return so_path()


def _import_so(path: Path) -> ModuleType:
    spec = importlib.util.spec_from_file_location(_NAME, str(path))
    assert spec is not None and spec.loader is not None
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[_NAME] = mod
    return mod


def load(required: bool | None = None) -> ModuleType | None:
    """Return the extension module, building it when needed.

    ``required`` defaults to ``torch.cuda.is_available()``: with a GPU present the extension must load.
    """
    global _module, _load_error
    if required is None:
        required = torch.cuda.is_available()
    with _lock:
        if _module is not None:
            return _module
        if _load_error is not None and not required:
            return None
        try:
            if _is_stale():
                if not required and os.environ.get("LMSAE_BUILD_ON_IMPORT", "0") != "1":
                    raise FileNotFoundError(f"{so_path()} is not built (run __graft_entry__.build())")
                build()
            _module = _import_so(so_path())
            return _module
        except Exception as e:  # noqa: BLE001
            _load_error = e
            if required:
                raise RuntimeError(
                    "the sm_100a extension of language_model_saes_b200 could not be built or loaded; "
                    "the CUDA ops have no eager fallback on a GPU machine"
                ) from e
            return None


def available() -> bool:
    return load(required=False) is not None
