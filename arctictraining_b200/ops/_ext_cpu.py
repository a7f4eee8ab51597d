# SPDX-License-Identifier: Apache-2.0
"""Builds and loads the host-side C++ extension (``csrc_cpu``: multi-threaded, vectorised AdamW for optimizer states kept
in host memory).  Built in the source tree like the CUDA library; optional: without a compiler the PyTorch fallback is used.
"""

from __future__ import annotations

import os
import threading
from pathlib import Path
from typing import Optional

import torch

CSRC = Path(__file__).resolve().parent.parent / "csrc_cpu"
BUILD_DIR = CSRC / "build"
LIB_NAME = "atb200_cpu_ops"
_lock = threading.Lock()
_loaded: Optional[bool] = None


def lib_path() -> Path:
    return BUILD_DIR / f"{LIB_NAME}.so"


def build(verbose: bool = False) -> Path:
    from torch.utils import cpp_extension

    from ._ext import _shared_libstdcxx_flags

    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    cpp_extension.load(
        name=LIB_NAME,
        sources=sorted(str(p) for p in CSRC.glob("*.cpp")),
        extra_cflags=["-O3", "-std=c++17", "-fopenmp-simd", "-ffp-contract=off"],
        extra_ldflags=_shared_libstdcxx_flags(),
        build_directory=str(BUILD_DIR),
        is_python_module=False,
        with_cuda=False,
        verbose=verbose,
    )
    global _loaded
    _loaded = True
    return lib_path()


def available() -> bool:
    """Load the prebuilt library, building it once when a compiler is present; ``False`` when neither works."""
    global _loaded
    with _lock:
        if _loaded is not None:
            return _loaded
        try:
            fresh = lib_path().exists() and os.getenv("ATB200_REBUILD") != "1"
            if fresh and lib_path().stat().st_mtime >= max(p.stat().st_mtime for p in CSRC.glob("*.cpp")):
                torch.ops.load_library(str(lib_path()))
                _loaded = True
            else:
                build()
        except Exception:  # noqa: BLE001 - optional acceleration
            _loaded = False
        return _loaded


def ops():
    return torch.ops.atb200_cpu
