"""InternVL family: InternViT tower + pixel-shuffle token merge + MLP projector in front of a Llama-style decoder.

The reference trains InternVL through the upstream remote-code classes it vendors
(siirl/models/transformers/internvl_chat/modeling_internvl_chat.py:37-196: ``extract_feature`` = ViT -> drop class
token -> ``pixel_shuffle(0.5)`` -> ``mlp1``; image features written over the ``<IMG_CONTEXT>`` positions) and prepares
its inputs with dynamic 448-pixel tiling (siirl/models/transformers/internvl.py:1070-1116).  Here the tower is the
generic :class:`ViTEncoder` on the packed attention kernel, the language model is :class:`DecoderLM` (InternLM2 and
Qwen2 are the same block with different parameter names), and the processor has the interface of the Qwen2.5-VL one so
that the dataset, the rollout engine and the actor treat both families alike.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .vit import MLPProjector, ViTConfig, ViTEncoder, pixel_shuffle

IMG_START_TOKEN, IMG_END_TOKEN, IMG_CONTEXT_TOKEN = "<img>", "</img>", "<IMG_CONTEXT>"
_MEAN, _STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)


class InternVLVision(nn.Module):
    """``pixel_values [tiles, 3, S, S]`` -> ``[tiles * tokens_per_tile, llm_hidden]``."""

    def __init__(self, vit: ViTConfig, llm_hidden: int, downsample_ratio: float, dtype, device, gen):
        super().__init__()
        self.cfg = vit
        self.downsample_ratio = downsample_ratio
        self.encoder = ViTEncoder(vit, dtype, device, gen)
        merged = int(vit.hidden_size / (downsample_ratio * downsample_ratio))
        self.projector = MLPProjector(merged, llm_hidden, dtype, device, gen, pre_norm=True, hidden=llm_hidden)

    @property
    def tokens_per_tile(self) -> int:
        g = self.cfg.image_size // self.cfg.patch_size
        return int(g * self.downsample_ratio) ** 2

    def forward(self, pixel_values: torch.Tensor, grid_thw=None) -> torch.Tensor:
        f = self.encoder(pixel_values)                                  # [N, g*g, H]
        N, L, H = f.shape
        g = int(math.isqrt(L))
        f = pixel_shuffle(f.reshape(N, g, g, H), self.downsample_ratio)
        f = f.reshape(N * f.shape[1] * f.shape[2], f.shape[3])
        return self.projector(f)


# ---- dynamic tiling -----------------------------------------------------------------------------------------------
def closest_tile_grid(width: int, height: int, min_num: int = 1, max_num: int = 6, image_size: int = 448) -> Tuple[int, int]:
    """(columns, rows) of the tile grid whose aspect ratio is closest to the image's, among all grids of
    ``min_num..max_num`` tiles; on a tie the larger grid wins when the image has more than half its pixels."""
    ratio = width / height
    grids = sorted({(i, j) for n in range(min_num, max_num + 1) for i in range(1, n + 1) for j in range(1, n + 1)
                    if min_num <= i * j <= max_num}, key=lambda g: g[0] * g[1])
    best, best_diff = (1, 1), float("inf")
    for c, r in grids:
        diff = abs(ratio - c / r)
        if diff < best_diff:
            best, best_diff = (c, r), diff
        elif diff == best_diff and width * height > 0.5 * image_size * image_size * c * r:
            best = (c, r)
    return best


def dynamic_tiles(img: torch.Tensor, min_num: int = 1, max_num: int = 6, image_size: int = 448,
                  use_thumbnail: bool = True) -> torch.Tensor:
    """``img [3, H, W]`` in [0, 1] -> ``[tiles, 3, S, S]``: the image resized to the closest tile grid and cut row by
    row, plus a whole-image thumbnail when there is more than one tile."""
    _, H, W = img.shape
    c, r = closest_tile_grid(W, H, min_num, max_num, image_size)
    x = F.interpolate(img[None], size=(r * image_size, c * image_size), mode="bicubic", align_corners=False).clamp(0, 1)[0]
    tiles = x.reshape(3, r, image_size, c, image_size).permute(1, 3, 0, 2, 4).reshape(r * c, 3, image_size, image_size)
    if use_thumbnail and r * c > 1:
        thumb = F.interpolate(img[None], size=(image_size, image_size), mode="bicubic", align_corners=False).clamp(0, 1)
        tiles = torch.cat([tiles, thumb])
    return tiles


class InternVLProcessor:
    """Tiles and normalises images and expands each image placeholder of a prompt to ``tokens_per_tile * tiles``
    context tokens.  Same call interface as the Qwen2.5-VL processor: ``image_grid_thw`` rows are ``(tiles, 1, 1)``
    and rope positions are the plain token index."""

    def __init__(self, cfg, min_tiles: int = 1, max_tiles: int = 6, use_thumbnail: bool = True):
        assert cfg.vit is not None
        self.cfg = cfg
        self.image_size = cfg.vit.image_size
        g = cfg.vit.image_size // cfg.vit.patch_size
        self.tokens_per_tile = int(g * cfg.downsample_ratio) ** 2
        self.min_tiles, self.max_tiles, self.use_thumbnail = min_tiles, max_tiles, use_thumbnail
        self.image_token_id = cfg.image_token_id
        self.merge = 1

    def process_image(self, img: Any) -> Tuple[torch.Tensor, torch.Tensor]:
        from .vision_processor import _to_chw_float
        x = _to_chw_float(img).clamp(0, 1)
        tiles = dynamic_tiles(x, self.min_tiles, self.max_tiles, self.image_size, self.use_thumbnail)
        mean = torch.tensor(_MEAN).view(1, 3, 1, 1)
        std = torch.tensor(_STD).view(1, 3, 1, 1)
        return ((tiles - mean) / std).contiguous(), torch.tensor([[tiles.shape[0], 1, 1]])

    def process_video(self, frames: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Every frame is one tile (InternVL feeds videos as single-tile images)."""
        x = F.interpolate(frames.float().clamp(0, 1), size=(self.image_size, self.image_size), mode="bicubic",
                          align_corners=False).clamp(0, 1)
        mean = torch.tensor(_MEAN).view(1, 3, 1, 1)
        std = torch.tensor(_STD).view(1, 3, 1, 1)
        return ((x - mean) / std).contiguous(), torch.tensor([[x.shape[0], 1, 1]])

    def __call__(self, prompt_ids: Sequence[int], images: Sequence[Any], videos: Sequence[Any] = ()) -> Dict[str, Any]:
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
        counts = [int(g[0, 0]) * self.tokens_per_tile for g in grids]
        out_ids: List[int] = []
        k = 0
        for t in prompt_ids:
            if t == self.image_token_id and k < len(counts):
                out_ids.extend([self.image_token_id] * counts[k])
                k += 1
            else:
                out_ids.append(int(t))
        if k < len(counts):
            front: List[int] = []
            for j in range(k, len(counts)):
                front.extend([self.image_token_id] * counts[j])
            out_ids = front + out_ids
        return {"input_ids": out_ids, "pixel_values": torch.cat(pv) if pv else None, "image_grid_thw": grid}

    def rope(self, ids: torch.Tensor, grid: torch.Tensor) -> Tuple[torch.Tensor, int]:
        n = int(ids.numel())
        return torch.arange(n, dtype=torch.int64)[None].expand(3, n).contiguous(), 0


def expand_image_text(prompt: str, tiles_per_image: Sequence[int], tokens_per_tile: int, placeholder: str = "<image>") -> str:
    """Text-side expansion used with a string tokenizer: every ``<image>`` becomes
    ``<img>`` + ``<IMG_CONTEXT>`` x (tokens_per_tile * tiles) + ``</img>``."""
    for n in tiles_per_image:
        prompt = prompt.replace(placeholder, IMG_START_TOKEN + IMG_CONTEXT_TOKEN * (tokens_per_tile * n) + IMG_END_TOKEN, 1)
    return prompt
