"""Compile the reference's own CPU ops, in place, into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  The shared object built here is the unmodified
reference implementation (super_gnn/ops/csrc/{utils,spmm,ops,vertex_cover,
quantization_x86}.cpp) of the ops on the GraphSAGE hot path.  It is used to
(1) pin the C restatement in ``oracle/sgnn_oracle.c``, (2) generate the golden
vectors under ``tests/golden/`` and (3) serve as the timed CPU baseline.  It is
never loaded by the product package.

No reference source is copied: g++ reads the files where they lie and only the
object/shared files land in ``oracle/_ref/`` (git-ignored).  The reference's
own ``setup.py`` is not executed; the flags below restate the x86 branch of
super_gnn/ops/setup.py:7-35 (``-O3 -fopenmp -mavx512{f,cd,bw,dq,vl,ifma,vbmi}``).

Usage: ``python oracle/build_ref.py [--reference DIR]``.  Without the argument the
reference tree is looked for in ``$SUPERGNN_REFERENCE_DIR`` and then in a directory
named ``reference`` beside the repository.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
MODULE = "supergnn_ops"
SOURCES = ["utils.cpp", "spmm.cpp", "ops.cpp", "vertex_cover.cpp", "quantization_x86.cpp"]
ISA_FLAGS = ["-mavx512f", "-mavx512cd", "-mavx512bw", "-mavx512dq", "-mavx512vl",
             "-mavx512ifma", "-mavx512vbmi"]


def default_reference_dir() -> str:
    """``$SUPERGNN_REFERENCE_DIR``, else ``<parent of the repository>/reference``."""
    env = os.environ.get("SUPERGNN_REFERENCE_DIR")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def so_path() -> str:
    return os.path.join(OUT_DIR, MODULE + sysconfig.get_config_var("EXT_SUFFIX"))


def host_can_run_ref() -> bool:
    """True when this host's CPU has every ISA extension the build enables."""
    try:
        with open("/proc/cpuinfo") as f:
            txt = f.read()
    except OSError:
        return False
    flags = set()
    for line in txt.splitlines():
        if line.startswith("flags"):
            flags = set(line.split(":", 1)[1].split())
            break
    need = {"avx512f", "avx512cd", "avx512bw", "avx512dq", "avx512vl", "avx512ifma", "fma"}
    return need.issubset(flags) and bool({"avx512vbmi", "avx512_vbmi"} & flags)


def build(reference: str | None = None, verbose: bool = False) -> str | None:
    """Build ``oracle/_ref/supergnn_ops*.so``; returns its path or None when the
    reference tree is absent (the prebuilt file, if any, is then used as is)."""
    reference = reference or default_reference_dir()
    csrc = os.path.join(reference, "super_gnn", "ops", "csrc")
    target = so_path()
    if not os.path.isdir(csrc):
        return target if os.path.exists(target) else None
    srcs = [os.path.join(csrc, s) for s in SOURCES]
    if os.path.exists(target) and all(os.path.getmtime(target) >= os.path.getmtime(s) for s in srcs):
        return target
    from torch.utils import cpp_extension  # heavy import, only when building

    os.makedirs(OUT_DIR, exist_ok=True)
    cxx = "/usr/bin/g++" if os.path.exists("/usr/bin/g++") else "g++"
    inc = ["-I" + p for p in cpp_extension.include_paths()]
    inc += ["-I" + sysconfig.get_paths()["include"], "-I" + csrc]
    common = ["-O3", "-fopenmp", "-fPIC", "-std=c++17", "-DTORCH_EXTENSION_NAME=" + MODULE,
              "-DTORCH_API_INCLUDE_EXTENSION_H", "-w"] + ISA_FLAGS
    objs = []
    for s in srcs:
        o = os.path.join(OUT_DIR, os.path.basename(s)[:-4] + ".o")
        cmd = [cxx] + common + inc + ["-c", s, "-o", o]
        if verbose:
            print(" ".join(cmd))
        subprocess.check_call(cmd)
        objs.append(o)
    libdirs = cpp_extension.library_paths()
    link = [cxx, "-shared", "-fopenmp"] + objs + ["-L" + p for p in libdirs]
    link += ["-Wl,-rpath," + p for p in libdirs]
    link += ["-lc10", "-ltorch", "-ltorch_cpu", "-ltorch_python", "-o", target]
    if verbose:
        print(" ".join(link))
    subprocess.check_call(link)
    for o in objs:
        os.remove(o)
    return target


def load():
    """Import the built reference module (torch must be imported first)."""
    import importlib.util

    import torch  # noqa: F401  (libtorch symbols)

    path = so_path()
    if not os.path.exists(path):
        raise FileNotFoundError(path + " (run python oracle/build_ref.py where the reference tree is mounted)")
    if not host_can_run_ref():
        raise RuntimeError("host CPU lacks the AVX-512 extensions the reference x86 build enables")
    spec = importlib.util.spec_from_file_location(MODULE, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None, help="reference tree (default: see the module docstring)")
    a = ap.parse_args()
    p = build(a.reference, verbose=True)
    print("built:" if p else "reference tree absent, nothing built", p)
    sys.exit(0)
