"""Generic pre-norm Vision Transformer encoder on the packed attention kernel.

One module covers the image encoders of the vision-language families the reference trains besides Qwen2.5-VL:
InternViT of InternVL (siirl/models/transformers/internvl.py: class token, learned positions, LayerNorm or RMSNorm,
LayerScale ``ls1 / ls2``, GELU MLP), and the timm ViTs inside OpenVLA's Prismatic backbone
(siirl/models/embodied/openvla_oft/modeling_prismatic.py: DINOv2 with class + register tokens and LayerScale, SigLIP
without class token).  Images (or tiles) are the "sequences" of one packed non-causal attention call; projections run
on the tcgen05 GEMM; LayerNorm / GELU are plain PyTorch element-wise statements.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops.attention import SeqInfo, attention_packed
from .config import ViTConfig


class ViTBlock(nn.Module):
    def __init__(self, cfg: ViTConfig, dtype, device, gen, param):
        super().__init__()
        H, I = cfg.hidden_size, cfg.intermediate_size
        self.norm1_weight = param((H,), dtype, device, -1, gen)
        self.norm1_bias = param((H,), dtype, device, 0, gen) if cfg.norm_type == "layer_norm" else None
        self.qkv_weight = param((3 * H, H), dtype, device, 0.02, gen)
        self.qkv_bias = param((3 * H,), dtype, device, 0, gen) if cfg.qkv_bias else None
        self.proj_weight = param((H, H), dtype, device, 0.02, gen)
        self.proj_bias = param((H,), dtype, device, 0, gen)
        self.norm2_weight = param((H,), dtype, device, -1, gen)
        self.norm2_bias = param((H,), dtype, device, 0, gen) if cfg.norm_type == "layer_norm" else None
        self.fc1_weight = param((I, H), dtype, device, 0.02, gen)
        self.fc1_bias = param((I,), dtype, device, 0, gen)
        self.fc2_weight = param((H, I), dtype, device, 0.02, gen)
        self.fc2_bias = param((H,), dtype, device, 0, gen)
        if cfg.layer_scale:
            self.ls1 = param((H,), dtype, device, -1, gen)
            self.ls2 = param((H,), dtype, device, -1, gen)


class ViTEncoder(nn.Module):
    def __init__(self, cfg: ViTConfig, dtype=torch.bfloat16, device="cpu", gen=None):
        super().__init__()
        from .decoder import _Init, _param
        gen = gen if gen is not None else _Init(0, device)
        self.cfg = cfg
        H = cfg.hidden_size
        self.patch_dim = cfg.in_channels * cfg.patch_size * cfg.patch_size
        self.patch_dim_padded = (self.patch_dim + 7) // 8 * 8
        self.patch_embed_weight = _param((H, self.patch_dim_padded), dtype, device, 0.02, gen)
        if self.patch_dim_padded != self.patch_dim:
            with torch.no_grad():       # columns that only ever meet the zero padding of the input rows
                self.patch_embed_weight[:, self.patch_dim:].zero_()
        self.patch_embed_bias = _param((H,), dtype, device, 0, gen)
        n_prefix = cfg.num_prefix_tokens
        self.prefix_tokens = _param((max(n_prefix, 1), H), dtype, device, 0.02, gen) if n_prefix else None
        # learned positions for the class token (when present) and the patches; register tokens carry none (DINOv2)
        self.pos_has_class = cfg.class_token and cfg.class_pos_embed
        self.position_embedding = _param(((1 if self.pos_has_class else 0) + cfg.num_patches, H), dtype, device, 0.02, gen)
        self.blocks = nn.ModuleList([ViTBlock(cfg, dtype, device, gen, _param) for _ in range(cfg.depth)])
        if cfg.final_norm:
            self.norm_weight = _param((H,), dtype, device, -1, gen)
            self.norm_bias = _param((H,), dtype, device, 0, gen) if cfg.norm_type == "layer_norm" else None
        self.head_dim = H // cfg.num_heads
        # the attention kernels take head widths 32 / 64 / 128: other widths (SigLIP-so400m: 72) run zero-padded to
        # the next one, which changes neither the scores nor the kept output columns
        self.kernel_head_dim = next((d for d in (32, 64, 128) if d >= self.head_dim), None)
        assert self.kernel_head_dim is not None, "vision head width above 128"

    def _norm(self, x, w, b):
        if self.cfg.norm_type == "layer_norm":
            return F.layer_norm(x.float(), (x.shape[-1],), w.float(), b.float() if b is not None else None,
                                self.cfg.norm_eps).to(x.dtype)
        return ops.rmsnorm(x, w, self.cfg.norm_eps)[0]

    def patchify(self, images: torch.Tensor) -> torch.Tensor:
        """``[N, C, S, S]`` -> ``[N, patches, C*P*P]`` (row-major patch order, channel-major inside a patch: the
        layout of a stride-P convolution's weight)."""
        N, C, S, _ = images.shape
        P = self.cfg.patch_size
        g = S // P
        x = images.reshape(N, C, g, P, g, P).permute(0, 2, 4, 1, 3, 5)
        return x.reshape(N, g * g, C * P * P)

    def forward(self, images: torch.Tensor, keep_prefix: bool = False) -> torch.Tensor:
        """``images [N, C, S, S]`` (normalised) -> patch features ``[N, patches, H]`` of the selected layer (class /
        register tokens dropped unless ``keep_prefix``)."""
        cfg = self.cfg
        dev, dtype = self.patch_embed_weight.device, self.patch_embed_weight.dtype
        x = self.patchify(images.to(dev, dtype))
        N, L, _ = x.shape
        if x.shape[-1] != self.patch_dim_padded:
            x = F.pad(x, (0, self.patch_dim_padded - x.shape[-1]))
        h = ops.linear(x.reshape(N * L, -1), self.patch_embed_weight, self.patch_embed_bias).reshape(N, L, -1)
        pos = self.position_embedding
        if self.pos_has_class:
            h = h + pos[1:][None]
        else:
            h = h + pos[None]
        n_prefix = cfg.num_prefix_tokens
        if n_prefix:
            pre = self.prefix_tokens[None].expand(N, -1, -1)
            if self.pos_has_class:
                pre = torch.cat([pre[:, :1] + pos[:1][None], pre[:, 1:]], 1)
            h = torch.cat([pre, h], 1)
        S = h.shape[1]
        H, D, Dk = cfg.hidden_size, self.head_dim, self.kernel_head_dim
        nh = cfg.num_heads
        scale = 1.0 / math.sqrt(D)
        info = SeqInfo([S] * N, device=dev)
        h = h.reshape(N * S, H)
        stop = cfg.depth + cfg.select_layer + 1 if cfg.select_layer < 0 else cfg.select_layer
        for blk in self.blocks[:stop]:
            y = ops.linear(self._norm(h, blk.norm1_weight, blk.norm1_bias), blk.qkv_weight, blk.qkv_bias)
            if Dk != D:
                y = F.pad(y.reshape(-1, 3 * nh, D), (0, Dk - D)).reshape(-1, 3 * nh * Dk)
            a = attention_packed(y, info, nh, nh, Dk, causal=False, scale=scale)
            if Dk != D:
                a = a.reshape(-1, nh, Dk)[:, :, :D].reshape(-1, H)
            a = ops.linear(a, blk.proj_weight, blk.proj_bias)
            h = h + (a * blk.ls1 if cfg.layer_scale else a)
            y = ops.linear(self._norm(h, blk.norm2_weight, blk.norm2_bias), blk.fc1_weight, blk.fc1_bias)
            y = ops.linear(F.gelu(y.float(), approximate="tanh" if cfg.act == "gelu_tanh" else "none").to(y.dtype),
                           blk.fc2_weight, blk.fc2_bias)
            h = h + (y * blk.ls2 if cfg.layer_scale else y)
        if cfg.final_norm and stop == cfg.depth:
            h = self._norm(h, self.norm_weight, self.norm_bias)
        h = h.reshape(N, S, H)
        return h if keep_prefix else h[:, n_prefix:]


def pixel_shuffle(x: torch.Tensor, scale: float = 0.5) -> torch.Tensor:
    """InternVL's token merge: ``[N, g, g, C]`` -> ``[N, g*scale, g*scale, C / scale^2]`` (2x2 neighbouring patches
    become one token of four times the width)."""
    n, w, h, c = x.shape
    x = x.reshape(n, w, int(h * scale), int(c / scale))
    x = x.permute(0, 2, 1, 3).contiguous()
    x = x.reshape(n, int(h * scale), int(w * scale), int(c / (scale * scale)))
    return x.permute(0, 2, 1, 3).contiguous()


class MLPProjector(nn.Module):
    """``[LayerNorm] -> Linear -> GELU -> Linear [-> GELU -> Linear]`` from vision width to the language model width."""

    def __init__(self, in_dim: int, out_dim: int, dtype, device, gen, pre_norm: bool = True, hidden: Optional[int] = None,
                 layers: int = 2, hidden_dims=None):
        super().__init__()
        from .decoder import _param
        self.pre_norm = pre_norm
        if pre_norm:
            self.norm_weight = _param((in_dim,), dtype, device, -1, gen)
            self.norm_bias = _param((in_dim,), dtype, device, 0, gen)
        hidden = hidden or out_dim
        dims = [in_dim] + (list(hidden_dims) if hidden_dims is not None else [hidden] * (layers - 1)) + [out_dim]
        self.n = layers
        for i in range(layers):
            setattr(self, f"fc{i}_weight", _param((dims[i + 1], dims[i]), dtype, device, 0.02, gen))
            setattr(self, f"fc{i}_bias", _param((dims[i + 1],), dtype, device, 0, gen))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shp = x.shape
        x = x.reshape(-1, shp[-1])
        if self.pre_norm:
            x = F.layer_norm(x.float(), (x.shape[-1],), self.norm_weight.float(), self.norm_bias.float(), 1e-5).to(x.dtype)
        for i in range(self.n):
            x = ops.linear(x, getattr(self, f"fc{i}_weight"), getattr(self, f"fc{i}_bias"))
            if i + 1 < self.n:
                x = F.gelu(x.float()).to(x.dtype)
        return x.reshape(*shp[:-1], x.shape[-1])
