# SPDX-License-Identifier: Apache-2.0
"""Builds and loads the sm_100a CUDA extension that lives in ``arctictraining_b200/csrc``.

The shared object is built *in the source tree* (``csrc/build/atb200_ops.so``) so that it travels with
a copy of the repository; nothing is cached under the user's home directory.  Operators are registered
through ``TORCH_LIBRARY(atb200, ...)`` and called as ``torch.ops.atb200.<name>``.  On a machine with a
GPU the extension is mandatory: if it cannot be loaded, :func:`require` raises instead of silently
falling back to PyTorch code.
"""

from __future__ import annotations

import os
import threading
from pathlib import Path
from typing import List
from typing import Optional

import torch

CSRC = Path(__file__).resolve().parent.parent / "csrc"
BUILD_DIR = CSRC / "build"
LIB_NAME = "atb200_ops"
_lock = threading.Lock()
_loaded: Optional[bool] = None
_load_error: Optional[str] = None

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
    "--expt-relaxed-constexpr",
]


def sources() -> List[str]:
    return sorted(str(p) for p in CSRC.glob("*.cu")) + sorted(str(p) for p in CSRC.glob("*.cpp"))


def lib_path() -> Path:
    return BUILD_DIR / f"{LIB_NAME}.so"


def source_hash() -> str:
    """Content hash of every source and header of the extension (decides whether the library is stale)."""
    import hashlib

    h = hashlib.sha256()
    for p in sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp")) + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _hash_file() -> Path:
    return BUILD_DIR / f"{LIB_NAME}.sha256"


def _stale() -> bool:
    lib = lib_path()
    if not lib.exists():
        return True
    if os.getenv("ATB200_REBUILD") == "1":
        return True
    try:
        return _hash_file().read_text().strip() != source_hash()
    except OSError:
        return True


def _shared_libstdcxx_flags() -> list:
    """Link against the system's shared libstdc++ explicitly.  A toolchain that only ships the static archive would
    otherwise put a second copy of the C++ runtime into the extension, and stream formatting inside error messages then
    runs on facets of the wrong copy (observed as a crash while an exception text was being built)."""
    import glob

    for pattern in ("/usr/lib/x86_64-linux-gnu/libstdc++.so.6", "/usr/lib64/libstdc++.so.6", "/usr/lib/*/libstdc++.so.6"):
        hits = glob.glob(pattern)
        if hits:
            d = os.path.dirname(hits[0])
            return [f"-L{d}", "-l:libstdc++.so.6"]
    return []


def build(verbose: bool = False) -> Path:
    """Compile every ``.cu``/``.cpp`` under ``csrc`` for sm_100a into one shared object."""
    from torch.utils import cpp_extension

    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("MAX_JOBS", str(min(16, os.cpu_count() or 4)))
    cpp_extension.load(
        name=LIB_NAME,
        sources=sources(),
        extra_cflags=["-O3", "-std=c++17"],
        extra_cuda_cflags=NVCC_FLAGS,
        extra_ldflags=_shared_libstdcxx_flags(),
        extra_include_paths=[str(CSRC)],
        build_directory=str(BUILD_DIR),
        is_python_module=False,
        verbose=verbose,
    )
    _hash_file().write_text(source_hash())
    global _loaded
    _loaded = True
    return lib_path()


def load() -> bool:
    """Load the prebuilt library (building it when missing and a compiler is present)."""
    global _loaded, _load_error
    with _lock:
        if _loaded is not None:
            return _loaded
        try:
            if _stale():
                build()
            else:
                torch.ops.load_library(str(lib_path()))
                _loaded = True
        except Exception as exc:  # noqa: BLE001
            _load_error = f"{type(exc).__name__}: {exc}"
            _loaded = False
        return bool(_loaded)


def available() -> bool:
    """True when the CUDA kernels can be used: a GPU is visible and the library is loaded."""
    if not torch.cuda.is_available():
        return False
    if os.getenv("ATB200_DISABLE_KERNELS") == "1":
        return False
    return require()


def require() -> bool:
    """On a GPU machine the native library must load; raise loudly when it does not."""
    if load():
        return True
    raise RuntimeError(
        "arctictraining_b200: the sm_100a CUDA extension could not be loaded on a machine with a GPU "
        f"({_load_error}). Build it with `python -c 'import __graft_entry__ as g; g.build()'`."
    )


def ops():
    return torch.ops.atb200
