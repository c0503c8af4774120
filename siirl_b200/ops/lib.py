"""ctypes access to ``libsiirl_b200.so`` (the in-tree sm_100a kernel + host runtime library).

The library is plain C ABI: tensors are passed as raw device pointers plus the current CUDA stream.
On a machine with a GPU the library is mandatory — a missing build raises instead of silently
falling back to PyTorch code.  On a CPU-only machine the host-side entry points (partitioner,
sample index, safetensors reader) still work; the kernel entry points are never called there.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libsiirl_b200.so"
_lib: Optional["_CountingLib"] = None
_status_words: dict[int, torch.Tensor] = {}

# kernels launched by one call of each entry point (for the launch counter of the benchmark)
_KERNELS_PER_CALL = {"sb_rmsnorm_bwd": 2, "sb_grpo_group_adv": 4, "sb_fmha_bwd": 3, "sb_kk_partition": 0,
                     "sb_rmsnorm_bwd_blocks": 0, "sb_gemm_set_pair_kernel": 0}


class _CountingLib:
    """Thin proxy over the ctypes library that counts kernel launches made through it."""

    def __init__(self, cdll: ctypes.CDLL):
        self._cdll = cdll
        self.launches = 0
        self._cache: dict = {}

    def __getattr__(self, name: str):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._cdll, name)
            k = _KERNELS_PER_CALL.get(name, 1)

            def counted(*args, _raw=raw, _k=k):
                self.launches += _k
                return _raw(*args)

            fn = counted
            self._cache[name] = fn
        return fn


def launch_count() -> int:
    """Number of kernels of this library launched so far in this process (graph replays included)."""
    return _lib.launches if _lib is not None else 0


def add_launches(n: int) -> None:
    if _lib is not None:
        _lib.launches += n


class NativeLibraryMissing(ImportError):
    pass


class KernelStatusError(RuntimeError):
    """A kernel reported a non-zero status word (for instance a bounded wait that ran out)."""

    def __init__(self, code: int):
        names = {1: "producer wait timed out", 2: "mma wait timed out", 3: "epilogue wait timed out",
                 4: "flag wait timed out", 5: "bad argument"}
        super().__init__(f"kernel status {code}: {names.get(code, 'unknown')}")
        self.code = code


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def _debug_bounds() -> bool:
    """``SIIRL_DEBUG_BOUNDS=1`` loads the debug-bounds build of the library (built on first use): data-dependent
    indices report their first violation, read with :func:`bounds_violations`."""
    return os.environ.get("SIIRL_DEBUG_BOUNDS", "0") not in ("", "0")


def bounds_violations() -> list:
    """``[(unit, site, index, limit)]`` recorded by the debug-bounds build since the last call (empty in the normal
    build, which carries no records)."""
    out = []
    if not _debug_bounds():
        return out
    L = get_lib()
    for unit in ("elementwise", "kv_cache"):
        try:
            fn = getattr(L._cdll, f"sb_bounds_read_{unit}")
        except AttributeError:
            continue
        buf = (ctypes.c_int * 4)()
        check(fn(buf), f"sb_bounds_read_{unit}")
        if buf[0]:
            out.append((unit, int(buf[1]), int(buf[2]), int(buf[3])))
    return out


def get_lib() -> "_CountingLib":
    global _lib, _LIB_PATH
    if _lib is None:
        if _debug_bounds():
            from .. import build_ext
            _LIB_PATH = build_ext.build(debug_bounds=True)
        if not _LIB_PATH.exists():
            raise NativeLibraryMissing(
                f"{_LIB_PATH} not found: run `python -m siirl_b200.build_ext` (or __graft_entry__.build())")
        import torch  # noqa: F401  (loads libcudart.so.12 into the process first)
        _lib = _CountingLib(ctypes.CDLL(str(_LIB_PATH), mode=os.RTLD_GLOBAL if hasattr(os, "RTLD_GLOBAL")
                                        else ctypes.DEFAULT_MODE))
    return _lib


def use_native(t: torch.Tensor) -> bool:
    """True when ``t`` lives on a GPU, in which case the native kernels MUST be used."""
    if t.is_cuda:
        get_lib()
        return True
    return False


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def status_word(device: Optional[torch.device] = None) -> torch.Tensor:
    """Per-device int32 word that kernels write when a bounded wait expires."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
        _status_words[idx] = w
    return w


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronising read of the status word; raises KernelStatusError when a kernel gave up a wait."""
    w = status_word(device)
    code = int(w.item())
    if code != 0:
        w.zero_()
        raise KernelStatusError(code)


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
