"""Device helpers (reference: siirl/utils/extras/device.py switches CUDA / Ascend NPU).  This framework targets one
accelerator family, so the switch is CUDA-or-CPU; the function names are kept for user code written against them."""
from __future__ import annotations

import torch


def is_cuda_available() -> bool:
    return torch.cuda.is_available()


is_npu_available = False


def get_device_name() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


def get_torch_device():
    return torch.cuda if torch.cuda.is_available() else torch.cpu


def get_device_id() -> int:
    return torch.cuda.current_device() if torch.cuda.is_available() else 0


def get_nccl_backend() -> str:
    return "nccl" if torch.cuda.is_available() else "gloo"


def device_synchronize() -> None:
    if torch.cuda.is_available():
        torch.cuda.synchronize()
