"""TileXR-B200: tile-level asynchronous communication runtime for NVIDIA B200.

The package is a thin Python layer over two in-tree native libraries built by
``tilexr_b200._build`` (``lib/libtilexr.so`` with the C API and CUDA kernels, ``_C.so`` with the
PyTorch binding).  There is no Python fallback for any kernel: importing the package without the
native libraries fails with instructions to build them.
"""
from __future__ import annotations

import importlib
import os
from pathlib import Path

__version__ = "0.1.0"

_PKG = Path(__file__).resolve().parent


def _load_native():
    so = _PKG / "_C.so"
    lib = _PKG / "lib" / "libtilexr.so"
    if not so.exists() or not lib.exists():
        if os.environ.get("TILEXR_AUTO_BUILD", "1") != "0":
            from . import _build

            _build.build_all(verbose=False)
        else:
            raise ImportError(
                "tilexr_b200 native libraries are missing; run `python -m tilexr_b200._build` in the repository root"
            )
    import torch  # noqa: F401  (the binding links against libtorch)

    return importlib.import_module("tilexr_b200._C")


_C = _load_native()

from .parallel.comm import (  # noqa: E402
    Comm,
    World,
    group,
    init_emulated_world,
    init_from_torch_distributed,
    init_host_memory,
    init_process,
)
from .ops import collectives, ep, gemm, nvls, quant  # noqa: E402
from .ops.collectives import (  # noqa: E402
    ReduceOp,
    all_gather,
    all_reduce,
    all_to_all,
    broadcast,
    profile_probe,
    reduce_scatter,
)

LIB_PATH = str(_PKG / "lib" / "libtilexr.so")


def launch_count() -> int:
    """Kernels launched by the native library since the process started."""
    return int(_C.launch_count())
