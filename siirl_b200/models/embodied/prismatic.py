"""Prismatic vision backbone and projector of OpenVLA / OpenVLA-OFT on the framework's kernels.

Reference: siirl/models/embodied/openvla_oft/modeling_prismatic.py:67-262 (``PrismaticVisionBackbone``: timm DINOv2 and
SigLIP vision transformers whose second-to-last block outputs are concatenated along the channel axis;
``PrismaticProjector``: Linear -> GELU -> Linear [-> GELU -> Linear]) and :395-500 (patch features enter the
language model's input between the BOS token and the text).  Here both towers are :class:`ViTEncoder` instances (packed
attention + tcgen05 GEMMs), the language model is :class:`DecoderLM`, and the patch features are written over
placeholder tokens that the prompt carries right after BOS, which gives the same sequence.

Pixel layout as in the reference: ``[N, 6 * images, S, S]`` -- per image three channels normalised for the first
tower followed by three normalised for the fused one.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..config import PrismaticConfig
from ..vit import MLPProjector, ViTEncoder

# channel statistics of the two towers' preprocessing (timm data configs of the DINOv2 and SigLIP checkpoints)
DINO_MEAN, DINO_STD = (0.485, 0.456, 0.406), (0.229, 0.224, 0.225)
SIGLIP_MEAN, SIGLIP_STD = (0.5, 0.5, 0.5), (0.5, 0.5, 0.5)


class PrismaticVision(nn.Module):
    def __init__(self, cfg: PrismaticConfig, llm_hidden: int, dtype, device, gen):
        super().__init__()
        self.cfg = cfg
        self.featurizer = ViTEncoder(cfg.featurizer, dtype, device, gen)
        self.fused_featurizer = ViTEncoder(cfg.fused_featurizer, dtype, device, gen) if cfg.fused_featurizer else None
        vd = cfg.vision_dim
        if self.fused_featurizer is not None:
            self.projector = MLPProjector(vd, llm_hidden, dtype, device, gen, pre_norm=False, hidden=4 * vd, layers=3,
                                          hidden_dims=[4 * vd, llm_hidden])
        else:
            self.projector = MLPProjector(vd, llm_hidden, dtype, device, gen, pre_norm=False, hidden=llm_hidden, layers=2)

    @property
    def tokens_per_image(self) -> int:
        return self.cfg.tokens_per_image

    def forward(self, pixel_values: torch.Tensor, grid_thw=None) -> torch.Tensor:
        """``[N, 6 * images, S, S]`` (``[N, 3 * images, S, S]`` without the fused tower) -> ``[N * images * patches,
        llm_hidden]``, images of one sample after each other."""
        per = 6 if self.fused_featurizer is not None else 3
        N, C, S, _ = pixel_values.shape
        k = C // per
        x = pixel_values.reshape(N * k, per, S, S)
        f = self.featurizer(x[:, :3])
        if self.fused_featurizer is not None:
            f = torch.cat([f, self.fused_featurizer(x[:, 3:])], dim=2)
        return self.projector(f.reshape(-1, f.shape[-1]))


def normalize_for_towers(images_u8: torch.Tensor, fused: bool = True) -> torch.Tensor:
    """``[N, S, S, 3] uint8`` -> ``[N, 6, S, S]`` fp32 (``[N, 3, S, S]`` without the fused tower)."""
    x = images_u8.permute(0, 3, 1, 2).float() / 255.0
    dev = x.device

    def norm(mean, std):
        return (x - torch.tensor(mean, device=dev).view(1, 3, 1, 1)) / torch.tensor(std, device=dev).view(1, 3, 1, 1)
    return torch.cat([norm(DINO_MEAN, DINO_STD), norm(SIGLIP_MEAN, SIGLIP_STD)], 1) if fused else norm(DINO_MEAN, DINO_STD)
