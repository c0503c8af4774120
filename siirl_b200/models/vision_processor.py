"""Image preprocessing for the Qwen2.5-VL family (what the reference gets from the HF ``AutoProcessor`` and
siirl/data_coordinator/dataloader/vision_utils.py): resize so that both sides are multiples of ``patch * merge`` and
the area lies in ``[min_pixels, max_pixels]``, normalise, cut into ``patch x patch`` patches duplicated over
``temporal_patch_size`` frames, order them ``(t, h/m, w/m, m, m)`` — the order ``VisionTower`` expects — and expand
every image placeholder of the prompt into ``t * (h/m) * (w/m)`` image tokens."""
from __future__ import annotations

import math
from typing import Any, Dict, List, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from .config import DecoderConfig
from .vision import mrope_positions

_MEAN = (0.48145466, 0.4578275, 0.40821073)
_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(h: int, w: int, factor: int, min_pixels: int, max_pixels: int) -> Tuple[int, int]:
    """Target size: multiples of ``factor``, aspect ratio kept as far as possible, area within the bounds."""
    hb = max(factor, round(h / factor) * factor)
    wb = max(factor, round(w / factor) * factor)
    if hb * wb > max_pixels:
        beta = math.sqrt(h * w / max_pixels)
        hb = max(factor, math.floor(h / beta / factor) * factor)
        wb = max(factor, math.floor(w / beta / factor) * factor)
    elif hb * wb < min_pixels:
        beta = math.sqrt(min_pixels / (h * w))
        hb = math.ceil(h * beta / factor) * factor
        wb = math.ceil(w * beta / factor) * factor
    return hb, wb


def _to_chw_float(img: Any) -> torch.Tensor:
    """PIL image, ``[H, W, 3]`` uint8 array / tensor, ``[3, H, W]`` float tensor or a dict with ``bytes``."""
    if isinstance(img, dict) and "bytes" in img:
        import io

        from PIL import Image  # only needed for encoded images
        img = Image.open(io.BytesIO(img["bytes"])).convert("RGB")
    if hasattr(img, "convert"):
        img = np.asarray(img.convert("RGB"))
    t = torch.as_tensor(np.asarray(img) if not isinstance(img, torch.Tensor) else img)
    if t.dim() == 3 and t.shape[-1] == 3:
        t = t.permute(2, 0, 1)
    t = t.float()
    return t / 255.0 if t.max() > 1.5 else t


class VLProcessor:
    def __init__(self, cfg: DecoderConfig, min_pixels: int = 32 * 32, max_pixels: int = 768 * 768):
        assert cfg.vision is not None
        v = cfg.vision
        self.cfg = cfg
        self.patch, self.merge, self.tpatch = v.patch_size, v.spatial_merge_size, v.temporal_patch_size
        self.min_pixels, self.max_pixels = min_pixels, max_pixels
        self.image_token_id = cfg.image_token_id

    def process_image(self, img: Any) -> Tuple[torch.Tensor, torch.Tensor]:
        """-> (patches ``[gh*gw, 3*T*P*P]`` fp32, grid ``[1, 3]`` = (1, gh, gw))."""
        x = _to_chw_float(img)
        H, W = x.shape[1:]
        h2, w2 = smart_resize(H, W, self.patch * self.merge, self.min_pixels, self.max_pixels)
        if (h2, w2) != (H, W):
            x = F.interpolate(x[None], size=(h2, w2), mode="bilinear", align_corners=False, antialias=True)[0]
        mean = torch.tensor(_MEAN).view(3, 1, 1)
        std = torch.tensor(_STD).view(3, 1, 1)
        x = (x.clamp(0, 1) - mean) / std
        P, m = self.patch, self.merge
        gh, gw = h2 // P, w2 // P
        x = x.reshape(3, gh // m, m, P, gw // m, m, P).permute(1, 4, 2, 5, 0, 3, 6)       # gh/m, gw/m, m, m, C, P, P
        x = x.unsqueeze(5).expand(-1, -1, -1, -1, -1, self.tpatch, -1, -1)
        return x.reshape(gh * gw, 3 * self.tpatch * P * P).contiguous(), torch.tensor([[1, gh, gw]])

    def process_video(self, frames: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """``frames [F, 3, H, W]`` in [0, 1] (sides already multiples of patch * merge, e.g. from
        ``dataloader.vision_utils.process_video``) -> (patches ``[t*gh*gw, 3*T*P*P]``, grid ``[1, 3]`` = (t, gh, gw))
        with ``t = F / temporal_patch_size`` (the last frame is repeated to fill the last temporal patch)."""
        x = frames.float()
        Fn, _, H, W = x.shape
        unit = self.patch * self.merge
        if H % unit or W % unit:
            h2, w2 = smart_resize(H, W, unit, self.min_pixels, self.max_pixels)
            x = F.interpolate(x, size=(h2, w2), mode="bilinear", align_corners=False, antialias=True)
            H, W = h2, w2
        if Fn % self.tpatch:
            x = torch.cat([x, x[-1:].expand(self.tpatch - Fn % self.tpatch, -1, -1, -1)])
        t = x.shape[0] // self.tpatch
        mean = torch.tensor(_MEAN).view(1, 3, 1, 1)
        std = torch.tensor(_STD).view(1, 3, 1, 1)
        x = (x.clamp(0, 1) - mean) / std
        P, m = self.patch, self.merge
        gh, gw = H // P, W // P
        # [t, T, C, gh/m, m, P, gw/m, m, P] -> (t, gh/m, gw/m, m, m, C, T, P, P)
        x = x.reshape(t, self.tpatch, 3, gh // m, m, P, gw // m, m, P).permute(0, 3, 6, 4, 7, 2, 1, 5, 8)
        return x.reshape(t * gh * gw, 3 * self.tpatch * P * P).contiguous(), torch.tensor([[t, gh, gw]])

    def __call__(self, prompt_ids: Sequence[int], images: Sequence[Any], videos: Sequence[Any] = ()) -> Dict[str, Any]:
        """Expands each single placeholder ``image_token_id`` of ``prompt_ids`` to the token count of the next visual
        input.  Videos (frame tensors ``[F, 3, H, W]``) follow the images and use the same placeholder and the same
        vision tower, with a temporal grid dimension > 1."""
        pv, grids = [], []
        for im in images:
            p, g = self.process_image(im)
            pv.append(p)
            grids.append(g)
        for vid in videos:
            p, g = self.process_video(vid)
            pv.append(p)
            grids.append(g)
        grid = torch.cat(grids) if grids else torch.zeros(0, 3, dtype=torch.int64)
        out_ids: List[int] = []
        k = 0
        for t in prompt_ids:
            if t == self.image_token_id and k < len(grids):
                n = int(grid[k].prod()) // (self.merge ** 2)
                out_ids.extend([self.image_token_id] * n)
                k += 1
            else:
                out_ids.append(int(t))
        if k < len(grids):                       # prompts without placeholders: images go in front
            front: List[int] = []
            for j in range(k, len(grids)):
                front.extend([self.image_token_id] * (int(grid[j].prod()) // (self.merge ** 2)))
            out_ids = front + out_ids
        return {"input_ids": out_ids, "pixel_values": torch.cat(pv) if pv else None, "image_grid_thw": grid}

    def rope(self, ids: torch.Tensor, grid: torch.Tensor) -> Tuple[torch.Tensor, int]:
        """3-row rope positions of one sequence and its rope delta (= length - next position)."""
        pos = mrope_positions(ids, self.image_token_id, grid, self.merge)
        return pos, int(ids.numel() - (int(pos.max()) + 1)) if ids.numel() else 0


def make_vl_processor(cfg: DecoderConfig, min_pixels: int = 32 * 32, max_pixels: int = 768 * 768):
    """Image processor matching the model's vision tower: native-resolution patches for Qwen2.5-VL, 448-pixel tiles for
    the InternVL family (``max_pixels`` bounds the tile count there)."""
    if cfg.moonvit is not None:
        from .moonvit import MoonViTProcessor
        return MoonViTProcessor(cfg, min_pixels, max_pixels)
    if cfg.vit is not None:
        from .internvl import InternVLProcessor
        s = cfg.vit.image_size
        return InternVLProcessor(cfg, 1, max(1, min(12, max_pixels // (s * s))))
    if cfg.vision is None:
        raise ValueError("the model has no vision tower")
    return VLProcessor(cfg, min_pixels, max_pixels)
