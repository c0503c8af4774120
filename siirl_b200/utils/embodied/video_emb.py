"""Episode-video embedder for the embodied reward.

The reference embeds the episode video with a V-JEPA ViT (siirl/utils/embodied/video_emb.py:29-170: sample frames,
resize to 384, ViT over 2x16x16 tubelets, mean-pool) and shapes the reward of failed episodes by the distance to
clustered embeddings of successful ones.  This embedder has the same contract — ``[B, T, H, W, 3] uint8`` frames ->
``[B, E]`` fp32 — on the framework's packed ViT (``VisionTower``: tubelet patch GEMM, non-causal packed attention):
frames are sub-sampled to ``num_frames``, resized by the CUDA resize kernel, cut into tubelets of
``temporal_patch_size`` frames and the merged tokens are mean-pooled and L2-normalised.  Weights load from a state
dict when a checkpoint is given, else a fixed-seed random projection (still a consistent metric space for the
distance-based shaping, which is all the reward uses)."""
from __future__ import annotations

from typing import Optional

import torch

from ...models.config import VisionConfig
from ...models.vision import VisionTower
from ...ops.image import resize_bilinear


class VideoEmbedder:
    def __init__(self, img_size: int = 224, num_frames: int = 8, device="cpu", dtype=torch.bfloat16,
                 vision_config: Optional[VisionConfig] = None, checkpoint: Optional[str] = None, seed: int = 1234):
        from ...models.decoder import _Init
        self.cfg = vision_config or VisionConfig(depth=4, hidden_size=256, num_heads=4, intermediate_size=512,
                                                 patch_size=16, window_size=10 ** 6, fullatt_block_indexes=[0, 1, 2, 3],
                                                 out_hidden_size=256)
        unit = self.cfg.patch_size * self.cfg.spatial_merge_size
        self.img_size = max(unit, img_size // unit * unit)
        self.num_frames = max(self.cfg.temporal_patch_size, num_frames // self.cfg.temporal_patch_size
                              * self.cfg.temporal_patch_size)
        self.device, self.dtype = torch.device(device), dtype
        self.tower = VisionTower(self.cfg, dtype, self.device, _Init(seed, self.device))
        for p in self.tower.parameters():
            p.requires_grad_(False)
        if checkpoint:
            self.tower.load_state_dict(torch.load(checkpoint, map_location=self.device), strict=False)

    @torch.no_grad()
    def __call__(self, frames: torch.Tensor, lengths: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``lengths [B]``: number of valid frames per episode (default: all); sampling stays inside them."""
        B, T = frames.shape[:2]
        last = (lengths.reshape(B).cpu().clamp(1, T) - 1).float() if lengths is not None else torch.full((B,), T - 1.0)
        idx = (torch.linspace(0, 1, self.num_frames)[None, :] * last[:, None]).round().long()   # [B, F]
        f = frames[torch.arange(B)[:, None], idx.to(frames.device)].to(self.device)              # [B, F, H, W, 3]
        F_ = self.num_frames
        f = resize_bilinear(f.reshape(B * F_, *f.shape[2:]).contiguous(), (self.img_size, self.img_size))
        x = f.permute(0, 3, 1, 2).float() / 127.5 - 1.0                       # [B*F, 3, S, S]
        P, m, tp = self.cfg.patch_size, self.cfg.spatial_merge_size, self.cfg.temporal_patch_size
        g = self.img_size // P
        t = F_ // tp
        x = x.reshape(B, t, tp, 3, g // m, m, P, g // m, m, P).permute(0, 1, 4, 7, 5, 8, 3, 2, 6, 9)
        x = x.reshape(B * t * g * g, 3 * tp * P * P).to(self.dtype)
        grid = torch.tensor([[t, g, g]] * B, dtype=torch.int64)
        tok = self.tower(x, grid).float()                                     # [B * t*g*g/m^2, E]
        emb = tok.reshape(B, -1, tok.shape[-1]).mean(1)
        return torch.nn.functional.normalize(emb, dim=-1)
