"""In-tree build of the native library (``siirl_b200/lib/libsiirl_b200.so``).

Every ``.cu`` under ``csrc/`` is compiled for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``),
every ``.cpp`` with g++ through nvcc, and all objects are linked into one shared library that has no
dependency on torch or Python (it shares ``libcudart.so.12`` with torch, so the current device and
context that torch sets on a thread — autograd worker threads included — are the ones it sees): its ``extern "C"`` entry points are called through ``ctypes`` (see
``siirl_b200/ops/lib.py``).  nvcc cross-compiles without a GPU, so this runs on a CPU-only box.

Usage: ``python -m siirl_b200.build_ext [--force] [--verbose]``.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
SRC_DIR = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "build"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libsiirl_b200.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]


def _sources() -> list[Path]:
    return sorted(list(SRC_DIR.rglob("*.cu")) + list(SRC_DIR.rglob("*.cpp")))


def _headers_mtime() -> float:
    hs = list(SRC_DIR.rglob("*.h")) + list(SRC_DIR.rglob("*.cuh")) + [Path(__file__)]
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _obj_for(src: Path) -> Path:
    rel = src.relative_to(SRC_DIR)
    return OBJ_DIR / (str(rel).replace(os.sep, "__") + ".o")


def _compile(src: Path, verbose: bool) -> tuple[Path, str]:
    obj = _obj_for(src)
    cmd = [NVCC, *ARCH_FLAGS, *COMMON_FLAGS, "-I", str(SRC_DIR)]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return obj, proc.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile stale objects and link the shared library; returns its path."""
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    hdr_m = _headers_mtime()
    srcs = _sources()
    stale = []
    for s in srcs:
        o = _obj_for(s)
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hdr_m):
            stale.append(s)
    logs = []
    if stale:
        with cf.ThreadPoolExecutor(max_workers=min(len(stale), os.cpu_count() or 4)) as ex:
            for obj, log in ex.map(lambda s: _compile(s, verbose), stale):
                logs.append((obj, log))
    objs = [_obj_for(s) for s in srcs]
    need_link = bool(stale) or not LIB_PATH.exists() or any(
        o.stat().st_mtime > LIB_PATH.stat().st_mtime for o in objs)
    if need_link:
        cmd = [NVCC, *ARCH_FLAGS, "-shared", "--cudart", "shared", "-o", str(LIB_PATH), *map(str, objs), "-lpthread"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        for obj, log in logs:
            print(f"== {obj.name}\n{log}")
    return LIB_PATH


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(p)
