"""Image ops of the embodied path: crop + bilinear resize and the synthetic-environment rasteriser.  The numpy
functions are the CPU twins (oracle and timed CPU baseline); CUDA tensors use ``csrc/image_ops.cu``."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import numpy as np
import torch

from . import lib as _lib

_f = ctypes.c_float


def resize_bilinear_reference(img: np.ndarray, out_hw: Tuple[int, int], crop=None) -> np.ndarray:
    """``img [N, H, W, C] uint8``; ``crop = (y0, x0, h, w)`` in source pixels (default: whole image)."""
    N, H, W, C = img.shape
    OH, OW = out_hw
    y0, x0, ch, cw = crop if crop is not None else (0.0, 0.0, float(H), float(W))
    sy = np.clip(y0 + (np.arange(OH) + 0.5) * ch / OH - 0.5, 0, H - 1)
    sx = np.clip(x0 + (np.arange(OW) + 0.5) * cw / OW - 0.5, 0, W - 1)
    yi, xi = np.floor(sy).astype(int), np.floor(sx).astype(int)
    y1, x1 = np.minimum(yi + 1, H - 1), np.minimum(xi + 1, W - 1)
    wy, wx = (sy - yi)[None, :, None, None], (sx - xi)[None, None, :, None]
    f = img.astype(np.float32)
    top = (1 - wx) * f[:, yi][:, :, xi] + wx * f[:, yi][:, :, x1]
    bot = (1 - wx) * f[:, y1][:, :, xi] + wx * f[:, y1][:, :, x1]
    return np.clip((1 - wy) * top + wy * bot + 0.5, 0, 255).astype(np.uint8)


def resize_bilinear(img: torch.Tensor, out_hw: Tuple[int, int], crop=None) -> torch.Tensor:
    N, H, W, C = img.shape
    if not img.is_cuda:
        return torch.from_numpy(resize_bilinear_reference(img.numpy(), out_hw, crop))
    y0, x0, ch, cw = crop if crop is not None else (0.0, 0.0, float(H), float(W))
    out = torch.empty(N, out_hw[0], out_hw[1], C, dtype=torch.uint8, device=img.device)
    L = _lib.get_lib()
    _lib.check(L.sb_resize_bilinear_u8(_lib.ptr(img.contiguous()), _lib.ptr(out), N, H, W, C, out_hw[0], out_hw[1],
                                       _f(y0), _f(x0), _f(ch), _f(cw), _lib.stream()), "sb_resize_bilinear_u8")
    return out


def center_crop_box(H: int, W: int, scale: float = 0.9) -> Tuple[float, float, float, float]:
    """Centre crop with area ``scale`` of the image (the VLA evaluation crop)."""
    s = float(np.sqrt(scale))
    return ((1 - s) / 2 * H, (1 - s) / 2 * W, s * H, s * W)


def raster_synth_env_reference(state: np.ndarray, H: int, W: int) -> np.ndarray:
    N = state.shape[0]
    v, u = np.meshgrid((np.arange(H) + 0.5) / H, (np.arange(W) + 0.5) / W, indexing="ij")
    out = np.zeros((N, H, W, 3), dtype=np.uint8)
    for n in range(N):
        s = state[n].astype(np.float32)
        r = 40.0 + 60.0 * v
        g = 44.0 + 50.0 * u
        b = 52.0 + 30.0 * (1.0 - v)
        dg = np.sqrt((u - s[2]) ** 2 + (v - s[3]) ** 2)
        goal = dg < 0.06
        r, g, b = np.where(goal, 30.0, r), np.where(goal, 200.0, g), np.where(goal, 60.0, b)
        da = np.sqrt((u - s[0]) ** 2 + (v - s[1]) ** 2)
        rad = 0.035 + 0.015 * s[4]
        ag = da < rad
        shade = 1.0 - 0.5 * (da / rad) ** 2
        r, g, b = np.where(ag, 220.0 * shade, r), np.where(ag, 60.0 * shade, g), np.where(ag, 50.0 * shade, b)
        out[n] = np.stack([r, g, b], -1).astype(np.uint8)
    return out


def raster_synth_env(state: torch.Tensor, H: int = 256, W: int = 256, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``state [N, 8]`` fp32 -> ``[N, H, W, 3]`` uint8 observation written into a device buffer."""
    N = state.shape[0]
    if not state.is_cuda:
        return torch.from_numpy(raster_synth_env_reference(state.numpy(), H, W))
    if out is None:
        out = torch.empty(N, H, W, 3, dtype=torch.uint8, device=state.device)
    L = _lib.get_lib()
    _lib.check(L.sb_raster_synth_env(_lib.ptr(state.float().contiguous()), _lib.ptr(out), N, H, W, _lib.stream()),
               "sb_raster_synth_env")
    return out
