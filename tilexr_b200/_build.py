"""In-tree build of the native libraries.

Two shared objects are produced next to this file:

* ``lib/libtilexr.so`` -- the C API: core runtime, collectives, expert-parallel kernels, GEMM
  fusions, MoonEP stages, host-memory simulator, protocol checker.  C++17 sources go through
  g++, ``.cu`` sources through ``nvcc -gencode arch=compute_100a,code=sm_100a``.
* ``_C.so`` -- the PyTorch binding (``TORCH_LIBRARY`` ops and pybind classes) linked against
  ``libtilexr.so``.

Objects are cached under ``build/`` keyed by source mtime and flags, so a rebuild after a
one-file change takes seconds.  ``python -m tilexr_b200._build`` runs it from the shell.

Both shared objects are linked under a temporary name and renamed into place together at the
end, so that a reader of the tree (a packaging step, another process importing the package)
never finds a half-written library or a binding that is older than the library beside it.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
PKG = ROOT / "tilexr_b200"
BUILD = ROOT / "build"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")

INCLUDES = [
    CSRC / "include",
    CSRC / "comm",
    CSRC / "collectives",
    CSRC / "ep",
    CSRC / "gemm",
    CSRC / "moonep",
    CSRC / "hostsim",
    CSRC / "checker",
    CUDA_HOME / "include",
]

CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-Wextra", "-Wno-unused-parameter", "-pthread"]
NVCC_FLAGS = [
    "-std=c++17",
    "-O3",
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]

LIB_SUBDIRS = ["comm", "collectives", "ep", "gemm", "moonep", "hostsim", "checker"]


def _sources():
    cpp, cu = [], []
    for sub in LIB_SUBDIRS:
        d = CSRC / sub
        if not d.is_dir():
            continue
        cpp += sorted(d.glob("*.cpp"))
        cu += sorted(d.glob("*.cu"))
    return cpp, cu


def _newest_header_mtime() -> float:
    newest = 0.0
    for pattern in ("*.h", "*.cuh", "*.hpp", "*.inc"):
        for p in CSRC.rglob(pattern):
            newest = max(newest, p.stat().st_mtime)
    return newest


def _staged(out: Path) -> Path:
    """Where a shared object is linked before it is renamed into place."""
    return out.with_name(out.name + ".staged")


def _publish(*outs: Path) -> None:
    for out in outs:
        staged = _staged(out)
        if staged.exists():
            os.replace(staged, out)


def _obj_path(src: Path, flags) -> Path:
    key = hashlib.sha1((str(src) + " ".join(flags)).encode()).hexdigest()[:10]
    return BUILD / "obj" / f"{src.stem}.{key}.o"


def _compile(src: Path, header_mtime: float, verbose: bool):
    inc = [f"-I{p}" for p in INCLUDES]
    if src.suffix == ".cu":
        flags = NVCC_FLAGS
        obj = _obj_path(src, flags)
        cmd = [NVCC, *flags, *inc, "-c", str(src), "-o", str(obj)]
    else:
        flags = CXX_FLAGS
        obj = _obj_path(src, flags)
        cmd = ["g++", *flags, *inc, "-c", str(src), "-o", str(obj)]
    if obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, header_mtime):
        return obj, None
    if verbose:
        print("  cc", src.relative_to(ROOT), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        return obj, f"{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}"
    return obj, None


def build_library(verbose: bool = True) -> Path:
    (BUILD / "obj").mkdir(parents=True, exist_ok=True)
    (PKG / "lib").mkdir(parents=True, exist_ok=True)
    cpp, cu = _sources()
    header_mtime = _newest_header_mtime()
    objs, errors = [], []
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        for obj, err in pool.map(lambda s: _compile(s, header_mtime, verbose), cpp + cu):
            objs.append(obj)
            if err:
                errors.append(err)
    if errors:
        raise RuntimeError("native build failed:\n" + "\n".join(errors))
    out = PKG / "lib" / "libtilexr.so"
    if out.exists() and all(out.stat().st_mtime >= o.stat().st_mtime for o in objs):
        return out
    staged = _staged(out)
    cmd = [
        NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(staged), *map(str, objs),
        "-cudart", "static", "-lpthread", "-lrt", "-ldl", "-Xlinker", "-soname=libtilexr.so",
    ]
    if verbose:
        print("  ld", out.relative_to(ROOT), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"link failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    return staged


def build_binding(verbose: bool = True) -> Path:
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    src = CSRC / "torch" / "binding.cpp"
    out = PKG / "_C.so"
    lib = PKG / "lib" / "libtilexr.so"
    if _staged(lib).exists():
        lib = _staged(lib)            # link against the library that is about to be published
    header_mtime = _newest_header_mtime()
    if out.exists() and out.stat().st_mtime >= max(src.stat().st_mtime, header_mtime, lib.stat().st_mtime):
        return out
    inc = [f"-I{p}" for p in INCLUDES] + [f"-I{p}" for p in cpp_extension.include_paths()]
    inc.append(f"-I{sysconfig.get_paths()['include']}")
    torch_lib = Path(torch.__file__).parent / "lib"
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    cmd = [
        "g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-Wall", "-Wno-unused-parameter",
        f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
        *inc, str(src), "-o", str(_staged(out)),
        str(lib), f"-L{torch_lib}", "-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python",
        "-Wl,-rpath,$ORIGIN/lib", f"-Wl,-rpath,{torch_lib}",
    ]
    if verbose:
        print("  cc+ld", out.relative_to(ROOT), "(torch binding, about a minute)", flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"binding build failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    return _staged(out)


def build_checker_cli(verbose: bool = True) -> Path:
    """The stand-alone protocol checker (no CUDA, no torch)."""
    (PKG / "bin").mkdir(parents=True, exist_ok=True)
    out = PKG / "bin" / "tilexr_checker"
    srcs = [CSRC / "checker" / "checker.cpp", CSRC / "checker" / "cli" / "checker_cli.cpp"]
    newest = max([p.stat().st_mtime for p in srcs] + [(CSRC / "checker" / "checker.h").stat().st_mtime])
    if out.exists() and out.stat().st_mtime >= newest:
        return out
    cmd = ["g++", "-std=c++17", "-O2", "-Wall", f"-I{CSRC / 'checker'}", *map(str, srcs), "-o", str(out)]
    if verbose:
        print("  cc+ld", out.relative_to(ROOT), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"checker build failed: {proc.stdout}\n{proc.stderr}")
    return out


def build_all(verbose: bool = True):
    build_library(verbose)
    build_binding(verbose)
    lib, ext = PKG / "lib" / "libtilexr.so", PKG / "_C.so"
    _publish(lib, ext)
    build_checker_cli(verbose)
    return lib, ext


if __name__ == "__main__":
    paths = build_all(verbose=True)
    print("built:", *[p.relative_to(ROOT) for p in paths])
    sys.exit(0)
