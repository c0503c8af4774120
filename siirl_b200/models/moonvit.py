"""MoonViT vision tower and projector of Kimi-VL on the packed kernels.

The reference trains Kimi-VL through the model's upstream remote code, patched for sequence parallelism
(siirl/models/transformers/kimi_vl.py:27-75 image-feature merge, :120-225 attention).  The tower's public architecture:
a 14 x 14 patch projection, a learnable ``[64, 64, H]`` position table interpolated (bicubic) to each image's patch
grid, pre-LayerNorm blocks whose attention rotates query / key pairs by the patch's (x, y) position, GELU(tanh) MLPs, a
final LayerNorm, a 2 x 2 neighbourhood merge, and the projector LayerNorm -> Linear -> GELU -> Linear into the
language-model width.  Images are the sequences of one packed non-causal attention call.

Rotary layout.  Checkpoints pair channels (2j, 2j+1) of a head and alternate the axes: pair j even turns with x, odd
with y, both at frequency ``theta^(-4 (j // 2) / d)``.  The rope kernel rotates pairs (p, p + d/2) and picks the
position row by contiguous ranges of p, so the q and k rows of ``wqkv`` are held permuted in memory (x pairs first,
then y pairs; real parts in the first half of the head): scores are unchanged because q and k get the same
permutation.  ``rope_permutation`` is applied on load and undone on export.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops.attention import SeqInfo, attention_packed
from .config import MoonViTConfig


def rope_permutation(head_dim: int) -> torch.Tensor:
    """``perm[new] = old`` channel index inside one head (see the module docstring)."""
    quarter, half = head_dim // 4, head_dim // 2
    perm = torch.empty(head_dim, dtype=torch.int64)
    for old in range(head_dim):
        j, comp = old // 2, old % 2
        p = (j // 2) if j % 2 == 0 else quarter + j // 2
        perm[p + comp * half] = old
    return perm


def qk_row_permutation(cfg: MoonViTConfig) -> torch.Tensor:
    """Row permutation of ``wqkv`` (weight rows and bias entries): q and k heads permuted, v untouched."""
    H, nh = cfg.hidden_size, cfg.num_heads
    hd = H // nh
    per_head = rope_permutation(hd)
    rows = []
    for blk in range(3):
        for h in range(nh):
            base = blk * H + h * hd
            rows.append(base + (per_head if blk < 2 else torch.arange(hd)))
    return torch.cat(rows)


class MoonViTBlock(nn.Module):
    def __init__(self, cfg: MoonViTConfig, dtype, device, gen, param):
        super().__init__()
        H, I = cfg.hidden_size, cfg.intermediate_size
        self.norm0_weight = param((H,), dtype, device, -1, gen)
        self.norm0_bias = param((H,), dtype, device, 0, gen)
        self.wqkv_weight = param((3 * H, H), dtype, device, 0.02, gen)      # rows in the permuted rotary layout
        self.wqkv_bias = param((3 * H,), dtype, device, 0, gen)
        self.wo_weight = param((H, H), dtype, device, 0.02, gen)
        self.wo_bias = param((H,), dtype, device, 0, gen)
        self.norm1_weight = param((H,), dtype, device, -1, gen)
        self.norm1_bias = param((H,), dtype, device, 0, gen)
        self.fc0_weight = param((I, H), dtype, device, 0.02, gen)
        self.fc0_bias = param((I,), dtype, device, 0, gen)
        self.fc1_weight = param((H, I), dtype, device, 0.02, gen)
        self.fc1_bias = param((H,), dtype, device, 0, gen)


class MoonViT(nn.Module):
    """``forward(pixel_values [patches, C*P*P], grid_thw [images, 3] = (1, h, w)) -> [patches / merge^2, llm_hidden]``;
    patches of an image in raster order."""

    def __init__(self, cfg: MoonViTConfig, llm_hidden: int, dtype, device, gen):
        super().__init__()
        from .decoder import _param
        self.cfg = cfg
        H = cfg.hidden_size
        self.patch_dim = cfg.in_channels * cfg.patch_size * cfg.patch_size
        self.patch_dim_padded = (self.patch_dim + 7) // 8 * 8
        self.patch_embed_weight = _param((H, self.patch_dim_padded), dtype, device, 0.02, gen)
        if self.patch_dim_padded != self.patch_dim:
            with torch.no_grad():       # columns that only ever meet the zero padding of the input rows
                self.patch_embed_weight[:, self.patch_dim:].zero_()
        self.patch_embed_bias = _param((H,), dtype, device, 0, gen)
        self.pos_emb = _param((cfg.init_pos_emb_height, cfg.init_pos_emb_width, H), dtype, device, 0.02, gen)
        self.blocks = nn.ModuleList([MoonViTBlock(cfg, dtype, device, gen, _param) for _ in range(cfg.depth)])
        self.final_norm_weight = _param((H,), dtype, device, -1, gen)
        self.final_norm_bias = _param((H,), dtype, device, 0, gen)
        m2 = cfg.merge * cfg.merge
        self.pre_norm_weight = _param((H,), dtype, device, -1, gen)
        self.pre_norm_bias = _param((H,), dtype, device, 0, gen)
        self.linear_1_weight = _param((H * m2, H * m2), dtype, device, 0.02, gen)
        self.linear_1_bias = _param((H * m2,), dtype, device, 0, gen)
        self.linear_2_weight = _param((llm_hidden, H * m2), dtype, device, 0.02, gen)
        self.linear_2_bias = _param((llm_hidden,), dtype, device, 0, gen)
        self.head_dim = H // cfg.num_heads
        self.kernel_head_dim = next(d for d in (32, 64, 128) if d >= self.head_dim)
        self._rope = None

    def _rope_tables(self, device, max_pos: int):
        if self._rope is None or self._rope[0].shape[0] < max_pos or self._rope[0].device != torch.device(device):
            quarter = self.head_dim // 4
            inv = 1.0 / (10000.0 ** (torch.arange(0, quarter, dtype=torch.float64) / quarter))
            ang = torch.outer(torch.arange(max_pos, dtype=torch.float64), inv)
            ang = torch.cat([ang, ang], dim=-1)            # columns [0, q): x frequencies, [q, 2q): y frequencies
            self._rope = (ang.cos().float().to(device), ang.sin().float().to(device))
        return self._rope

    def _ln(self, x, w, b, eps=1e-5):
        return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float(), eps).to(x.dtype)

    def position_embedding(self, h: int, w: int) -> torch.Tensor:
        pe = self.pos_emb
        if (h, w) == tuple(pe.shape[:2]):
            return pe.reshape(h * w, -1)
        x = F.interpolate(pe.float().permute(2, 0, 1)[None], size=(h, w), mode="bicubic", align_corners=False)
        return x[0].permute(1, 2, 0).reshape(h * w, -1).to(pe.dtype)

    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        dev, dtype = self.patch_embed_weight.device, self.patch_embed_weight.dtype
        grids = [(int(h), int(w)) for _, h, w in torch.as_tensor(grid_thw).tolist()]
        x = pixel_values.to(dev, dtype)
        if x.shape[1] != self.patch_dim_padded:
            x = F.pad(x, (0, self.patch_dim_padded - x.shape[1]))
        hdn = ops.linear(x, self.patch_embed_weight, self.patch_embed_bias)
        hdn = hdn + torch.cat([self.position_embedding(h, w) for h, w in grids]).to(dev)
        xs = torch.cat([torch.arange(w).repeat(h) for h, w in grids])
        ys = torch.cat([torch.arange(h).repeat_interleave(w) for h, w in grids])
        pos3 = torch.stack([xs, ys, ys]).to(dev, torch.int32)
        rope = self._rope_tables(dev, int(max(max(g) for g in grids)) + 1)
        info = SeqInfo([h * w for h, w in grids], device=dev)
        nh, D, Dk, H = cfg.num_heads, self.head_dim, self.kernel_head_dim, cfg.hidden_size
        quarter = D // 4
        scale = 1.0 / math.sqrt(D)
        for blk in self.blocks:
            y = ops.linear(self._ln(hdn, blk.norm0_weight, blk.norm0_bias), blk.wqkv_weight, blk.wqkv_bias)
            y = ops.rope(y, 2 * nh, D, pos3, rope[0], rope[1], mrope_section=(quarter, quarter, 0))
            if Dk != D:
                y = F.pad(y.reshape(-1, 3 * nh, D), (0, Dk - D)).reshape(-1, 3 * nh * Dk)
            a = attention_packed(y, info, nh, nh, Dk, causal=False, scale=scale)
            if Dk != D:
                a = a.reshape(-1, nh, Dk)[:, :, :D].reshape(-1, H)
            hdn = hdn + ops.linear(a, blk.wo_weight, blk.wo_bias)
            y = ops.linear(self._ln(hdn, blk.norm1_weight, blk.norm1_bias), blk.fc0_weight, blk.fc0_bias)
            hdn = hdn + ops.linear(F.gelu(y.float(), approximate="tanh").to(y.dtype), blk.fc1_weight, blk.fc1_bias)
        hdn = self._ln(hdn, self.final_norm_weight, self.final_norm_bias)
        # 2 x 2 merge per image, then the projector (its LayerNorm acts on the unmerged vectors)
        hdn = self._ln(hdn, self.pre_norm_weight, self.pre_norm_bias)
        m = cfg.merge
        merged, at = [], 0
        for h, w in grids:
            t = hdn[at:at + h * w].reshape(h // m, m, w // m, m, H).permute(0, 2, 1, 3, 4)
            merged.append(t.reshape((h // m) * (w // m), m * m * H))
            at += h * w
        y = torch.cat(merged)
        y = ops.linear(y, self.linear_1_weight, self.linear_1_bias)
        return ops.linear(F.gelu(y.float()).to(y.dtype), self.linear_2_weight, self.linear_2_bias)


class MoonViTProcessor:
    """Native-resolution patches in raster order; each image placeholder expands to ``(h / merge) * (w / merge)``
    tokens.  Same call interface as the Qwen2.5-VL processor; rope positions are the plain token index."""

    def __init__(self, cfg, min_pixels: int = 28 * 28, max_pixels: int = 768 * 768):
        assert cfg.moonvit is not None
        self.cfg = cfg
        self.patch, self.merge = cfg.moonvit.patch_size, cfg.moonvit.merge
        self.min_pixels, self.max_pixels = min_pixels, max_pixels
        self.image_token_id = cfg.image_token_id

    def process_image(self, img: Any) -> Tuple[torch.Tensor, torch.Tensor]:
        from .vision_processor import _to_chw_float, smart_resize
        x = _to_chw_float(img).clamp(0, 1)
        Hh, Ww = x.shape[1:]
        unit = self.patch * self.merge
        h2, w2 = smart_resize(Hh, Ww, unit, self.min_pixels, self.max_pixels)
        if (h2, w2) != (Hh, Ww):
            x = F.interpolate(x[None], size=(h2, w2), mode="bicubic", align_corners=False).clamp(0, 1)[0]
        x = (x - 0.5) / 0.5
        P = self.patch
        gh, gw = h2 // P, w2 // P
        x = x.reshape(3, gh, P, gw, P).permute(1, 3, 0, 2, 4).reshape(gh * gw, 3 * P * P)
        return x.contiguous(), torch.tensor([[1, gh, gw]])

    def __call__(self, prompt_ids: Sequence[int], images: Sequence[Any], videos: Sequence[Any] = ()) -> Dict[str, Any]:
        pv, grids = [], []
        for im in list(images) + [f for v in videos for f in v]:       # video frames enter as images
            p, g = self.process_image(im)
            pv.append(p)
            grids.append(g)
        grid = torch.cat(grids) if grids else torch.zeros(0, 3, dtype=torch.int64)
        counts = [int(g[0, 1] * g[0, 2]) // (self.merge ** 2) for g in grids]
        out_ids: List[int] = []
        k = 0
        for t in prompt_ids:
            if t == self.image_token_id and k < len(counts):
                out_ids.extend([self.image_token_id] * counts[k])
                k += 1
            else:
                out_ids.append(int(t))
        if k < len(counts):
            out_ids = [self.image_token_id] * sum(counts[k:]) + out_ids
        return {"input_ids": out_ids, "pixel_values": torch.cat(pv) if pv else None, "image_grid_thw": grid}

    def rope(self, ids: torch.Tensor, grid: torch.Tensor) -> Tuple[torch.Tensor, int]:
        n = int(ids.numel())
        return torch.arange(n, dtype=torch.int64)[None].expand(3, n).contiguous(), 0
