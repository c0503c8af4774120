"""In-tree build of the native library (``siirl_b200/lib/libsiirl_b200.so``).

Every ``.cu`` under ``csrc/`` is compiled for sm_100a only (``-gencode arch=compute_100a,code=sm_100a``),
every ``.cpp`` with g++ through nvcc, and all objects are linked into one shared library that has no
dependency on torch or Python (it shares ``libcudart.so.12`` with torch, so the current device and
context that torch sets on a thread — autograd worker threads included — are the ones it sees): its ``extern "C"`` entry points are called through ``ctypes`` (see
``siirl_b200/ops/lib.py``).  nvcc cross-compiles without a GPU, so this runs on a CPU-only box.

Usage: ``python -m siirl_b200.build_ext [--force] [--verbose] [--debug-bounds]``.
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
# debug-bounds variant (-DSB_DEBUG_BOUNDS: data-dependent indices report their first violation, see csrc/common.cuh)
DBG_OBJ_DIR = PKG_DIR / "build_dbg"
DBG_LIB_PATH = LIB_DIR / "libsiirl_b200_dbg.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default"]


def _sources() -> list[Path]:
    return sorted(list(SRC_DIR.rglob("*.cu")) + list(SRC_DIR.rglob("*.cpp")))


def _headers_mtime() -> float:
    hs = list(SRC_DIR.rglob("*.h")) + list(SRC_DIR.rglob("*.cuh")) + [Path(__file__)]
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _obj_for(src: Path, debug_bounds: bool = False) -> Path:
    rel = src.relative_to(SRC_DIR)
    return (DBG_OBJ_DIR if debug_bounds else OBJ_DIR) / (str(rel).replace(os.sep, "__") + ".o")


def _compile(src: Path, verbose: bool, debug_bounds: bool = False) -> tuple[Path, str]:
    obj = _obj_for(src, debug_bounds)
    cmd = [NVCC, *ARCH_FLAGS, *COMMON_FLAGS, "-I", str(SRC_DIR)]
    if debug_bounds:
        cmd += ["-DSB_DEBUG_BOUNDS"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return obj, proc.stderr


def build(force: bool = False, verbose: bool = False, debug_bounds: bool = False) -> Path:
    """Compile stale objects and link the shared library; returns its path."""
    obj_dir, lib_path = (DBG_OBJ_DIR, DBG_LIB_PATH) if debug_bounds else (OBJ_DIR, LIB_PATH)
    obj_dir.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    hdr_m = _headers_mtime()
    srcs = _sources()
    if not force and lib_path.exists() and lib_path.stat().st_mtime >= max([hdr_m] + [x.stat().st_mtime for x in srcs]):
        return lib_path         # a library newer than every source: nothing to do (object files may be absent)
    stale = []
    for s in srcs:
        o = _obj_for(s, debug_bounds)
        if force or not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hdr_m):
            stale.append(s)
    logs = []
    if stale:
        with cf.ThreadPoolExecutor(max_workers=min(len(stale), os.cpu_count() or 4)) as ex:
            for obj, log in ex.map(lambda s: _compile(s, verbose, debug_bounds), stale):
                logs.append((obj, log))
    objs = [_obj_for(s, debug_bounds) for s in srcs]
    need_link = bool(stale) or not lib_path.exists() or any(
        o.stat().st_mtime > lib_path.stat().st_mtime for o in objs)
    if need_link:
        cmd = [NVCC, *ARCH_FLAGS, "-shared", "--cudart", "shared", "-o", str(lib_path), *map(str, objs), "-lpthread"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        for obj, log in logs:
            print(f"== {obj.name}\n{log}")
    return lib_path


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, debug_bounds="--debug-bounds" in sys.argv)
    print(p)
