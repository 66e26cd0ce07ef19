"""Build ``libsupergnn_b200.so`` (the C-ABI library) in-tree with nvcc for sm_100a.

``python -m super_gnn_b200.build`` compiles every ``csrc/*.cu`` and links one
shared library next to this file.  nvcc cross-compiles without a GPU.  Objects are
rebuilt only when their source or a header they include (transitively) changed; the
GEMM files instantiate CUTLASS templates and take about a minute each.

The dense GEMM is built from the CUTLASS 3.x sm100 collectives.  The header tree is
looked up in ``$CUTLASS_HOME/include`` first, then in the copies that ship inside the
``flashinfer`` and ``tilelang`` wheels; the build fails if none has the sm100
emulated-fp32 mainloop.
"""
from __future__ import annotations

import glob
import importlib.util
import os
import re
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libsupergnn_b200.so")
OBJ_DIR = os.path.join(HERE, "build")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-O2",
    "--expt-relaxed-constexpr",
    "-diag-suppress", "20012",  # CUTLASS: __host__ __device__ on defaulted constructors
]

_CUTLASS_PROBE = os.path.join("cutlass", "gemm", "collective", "sm100_mma_warpspecialized_emulated.hpp")


def cutlass_include() -> str:
    """Directory holding ``cutlass/`` and ``cute/`` with the sm100 emulated-fp32 mainloop."""
    cands = []
    if os.environ.get("CUTLASS_HOME"):
        cands.append(os.path.join(os.environ["CUTLASS_HOME"], "include"))
    for pkg, rel in (("flashinfer", ("data", "cutlass", "include")), ("tilelang", ("3rdparty", "cutlass", "include"))):
        spec = importlib.util.find_spec(pkg)  # locates the wheel without importing it
        for base in (spec.submodule_search_locations or []) if spec else []:
            cands.append(os.path.join(base, *rel))
    for c in cands:
        if os.path.exists(os.path.join(c, _CUTLASS_PROBE)):
            return c
    raise RuntimeError("no CUTLASS header tree with " + _CUTLASS_PROBE + " found (looked in: " + ", ".join(cands) +
                       "); set CUTLASS_HOME")


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found: supergnn_b200 has no prebuilt fallback and no CPU path")
    return found


def sources() -> list:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps() -> list:
    return sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(HERE, "..", "include", "supergnn_b200.h")]


def is_current() -> bool:
    if not os.path.exists(LIB):
        return False
    t = os.path.getmtime(LIB)
    return all(os.path.getmtime(d) <= t for d in _deps() if os.path.exists(d))


_INCLUDE = re.compile(r'^\s*#\s*include\s+"([^"]+)"', re.M)


def _local_headers(path: str, seen: set) -> set:
    """Quoted includes of ``path`` that resolve next to it, transitively."""
    with open(path) as f:
        text = f.read()
    for inc in _INCLUDE.findall(text):
        cand = os.path.normpath(os.path.join(os.path.dirname(path), inc))
        if os.path.exists(cand) and cand not in seen:
            seen.add(cand)
            _local_headers(cand, seen)
    return seen


def _object_is_current(src: str, obj: str) -> bool:
    if not os.path.exists(obj):
        return False
    t = os.path.getmtime(obj)
    return all(os.path.getmtime(d) <= t for d in [src, os.path.abspath(__file__)] + sorted(_local_headers(src, set())))


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and is_current():
        return LIB
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    cutlass_flags = ["-I", cutlass_include()]

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        if not force and _object_is_current(src, obj):
            return obj
        with open(src) as f:
            uses_cutlass = "gemm_bf16x9.cuh" in f.read()
        cmd = [nvcc] + NVCC_FLAGS + (cutlass_flags if uses_cutlass else []) + ["-c", src, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, sources()))
    cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
