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
_lib: Optional[ctypes.CDLL] = None
_status_words: dict[int, torch.Tensor] = {}


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


def get_lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise NativeLibraryMissing(
                f"{_LIB_PATH} not found: run `python -m siirl_b200.build_ext` (or __graft_entry__.build())")
        import torch  # noqa: F401  (loads libcudart.so.12 into the process first)
        _lib = ctypes.CDLL(str(_LIB_PATH), mode=os.RTLD_GLOBAL if hasattr(os, "RTLD_GLOBAL") else ctypes.DEFAULT_MODE)
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
