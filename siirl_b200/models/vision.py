"""Vision tower of the Qwen2.5-VL family on the packed kernels of ``siirl_b200.ops``.

Structure (public architecture; the reference reaches it through HF transformers,
siirl/models/transformers/qwen2_5_vl.py): patch embedding as one GEMM over flattened ``C x T x P x P`` patches, blocks
of RMSNorm -> attention with 2-D rotary positions -> SwiGLU MLP, window attention (``window_size`` pixels) in every
block except ``fullatt_block_indexes``, and a 2x2 spatial merger (RMSNorm -> Linear -> GELU -> Linear) into the
language model width.  Attention is the packed varlen kernel without causal mask: windows (or whole images) are the
"sequences".  Patches are expected in the processor's order: per image ``(t, h/2, w/2, 2, 2)``.
"""
from __future__ import annotations

import math
from typing import List, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops.attention import SeqInfo, attention_packed
from .config import VisionConfig


class VisionBlock(nn.Module):
    def __init__(self, cfg: VisionConfig, dtype, device, gen, param):
        super().__init__()
        H, I = cfg.hidden_size, cfg.intermediate_size
        self.norm1 = param((H,), dtype, device, -1, gen)
        self.qkv_weight = param((3 * H, H), dtype, device, 0.02, gen)
        self.qkv_bias = param((3 * H,), dtype, device, 0, gen)
        self.proj_weight = param((H, H), dtype, device, 0.02, gen)
        self.proj_bias = param((H,), dtype, device, 0, gen)
        self.norm2 = param((H,), dtype, device, -1, gen)
        # The element-wise and GEMM kernels move 16-byte vectors, so the MLP width is rounded up to a multiple of 64
        # (Qwen2.5-VL: 3420 -> 3456).  The extra gate / up rows and down columns are zero and stay zero under
        # training: their activations are silu(0) * 0 and the gradient reaching them is a product with those zeros.
        Ip = self.padded_intermediate = (I + 63) // 64 * 64
        self.gate_up_weight = param((2 * Ip, H), dtype, device, 0.02, gen)
        self.gate_up_bias = param((2 * Ip,), dtype, device, 0, gen)
        self.down_weight = param((H, Ip), dtype, device, 0.02, gen)
        self.down_bias = param((H,), dtype, device, 0, gen)
        if Ip != I:
            with torch.no_grad():
                self.gate_up_weight[I:Ip].zero_()
                self.gate_up_weight[Ip + I:].zero_()
                self.down_weight[:, I:].zero_()


class VisionTower(nn.Module):
    def __init__(self, cfg: VisionConfig, dtype, device, gen):
        super().__init__()
        from .decoder import _param
        self.cfg = cfg
        self.patch_dim = cfg.in_channels * cfg.temporal_patch_size * cfg.patch_size * cfg.patch_size
        self.patch_dim_padded = (self.patch_dim + 7) // 8 * 8
        H = cfg.hidden_size
        self.patch_embed_weight = _param((H, self.patch_dim_padded), dtype, device, 0.02, gen)
        if self.patch_dim_padded != self.patch_dim:
            with torch.no_grad():       # columns that only ever meet the zero padding of the input rows
                self.patch_embed_weight[:, self.patch_dim:].zero_()
        self.blocks = nn.ModuleList([VisionBlock(cfg, dtype, device, gen, _param) for _ in range(cfg.depth)])
        m = cfg.spatial_merge_size ** 2
        self.merger_norm = _param((H,), dtype, device, -1, gen)
        self.merger_fc1_weight = _param((H * m, H * m), dtype, device, 0.02, gen)
        self.merger_fc1_bias = _param((H * m,), dtype, device, 0, gen)
        self.merger_fc2_weight = _param((cfg.out_hidden_size, H * m), dtype, device, 0.02, gen)
        self.merger_fc2_bias = _param((cfg.out_hidden_size,), dtype, device, 0, gen)
        self.head_dim = H // cfg.num_heads
        self._rope = None

    # ---- geometry ---------------------------------------------------------------------------------
    def _positions(self, grid_thw: torch.Tensor) -> torch.Tensor:
        """(h, w) index of every patch in processor order, ``[2, N]``."""
        ms = self.cfg.spatial_merge_size
        hs, ws = [], []
        for t, h, w in grid_thw.tolist():
            hp = torch.arange(h).unsqueeze(1).expand(-1, w)
            wp = torch.arange(w).unsqueeze(0).expand(h, -1)
            hp = hp.reshape(h // ms, ms, w // ms, ms).permute(0, 2, 1, 3).flatten()
            wp = wp.reshape(h // ms, ms, w // ms, ms).permute(0, 2, 1, 3).flatten()
            hs.append(hp.repeat(t))
            ws.append(wp.repeat(t))
        return torch.stack([torch.cat(hs), torch.cat(ws)])

    def _window_order(self, grid_thw: torch.Tensor) -> Tuple[torch.Tensor, List[int]]:
        """Permutation of merge units that groups them by attention window, and the window lengths (in patches)."""
        cfg = self.cfg
        ms = cfg.spatial_merge_size
        win = cfg.window_size // ms // cfg.patch_size      # merge units per window side
        order, lens, base = [], [], 0
        for t, h, w in grid_thw.tolist():
            gh, gw = h // ms, w // ms
            idx = torch.arange(t * gh * gw).reshape(t, gh, gw)
            for ti in range(t):
                for y in range(0, gh, win):
                    for x in range(0, gw, win):
                        blk = idx[ti, y:y + win, x:x + win].flatten() + base
                        order.append(blk)
                        lens.append(blk.numel() * ms * ms)
            base += t * gh * gw
        return torch.cat(order), lens

    def _rope_tables(self, device, max_pos: int):
        if self._rope is None or self._rope[0].shape[0] < max_pos or self._rope[0].device != torch.device(device):
            quarter = self.head_dim // 4
            inv = 1.0 / (10000.0 ** (torch.arange(0, quarter, dtype=torch.float64) / quarter))
            ang = torch.outer(torch.arange(max_pos, dtype=torch.float64), inv)
            ang = torch.cat([ang, ang], dim=-1)            # columns [0,q): h frequencies, [q,2q): w frequencies
            self._rope = (ang.cos().float().to(device), ang.sin().float().to(device))
        return self._rope

    # ---- forward ------------------------------------------------------------------------------------
    def forward(self, pixel_values: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        """``pixel_values [N, C*T*P*P]`` flattened patches, ``grid_thw [n_images, 3]`` -> ``[N / merge^2, out]``."""
        cfg = self.cfg
        dev = self.patch_embed_weight.device
        dtype = self.patch_embed_weight.dtype
        grid_thw = grid_thw.cpu()
        x = pixel_values.to(dev, dtype)
        if x.shape[1] != self.patch_dim_padded:
            x = F.pad(x, (0, self.patch_dim_padded - x.shape[1]))
        h = ops.linear(x, self.patch_embed_weight)
        N = h.shape[0]
        m = cfg.spatial_merge_size ** 2
        unit_order, win_lens = self._window_order(grid_thw)
        patch_order = (unit_order[:, None] * m + torch.arange(m)[None, :]).flatten().to(dev)
        hw = self._positions(grid_thw).to(dev)
        h = h.index_select(0, patch_order)
        hw = hw[:, patch_order]
        pos3 = torch.stack([hw[0], hw[1], hw[1]]).to(torch.int32)
        quarter = self.head_dim // 4
        rope = self._rope_tables(dev, int(hw.max().item()) + 1)
        full_lens = [int(t * hh * ww) for t, hh, ww in grid_thw.tolist()]
        info_win, info_full = SeqInfo(win_lens, device=dev), SeqInfo(full_lens, device=dev)
        nh, hd = cfg.num_heads, self.head_dim
        for i, blk in enumerate(self.blocks):
            info = info_full if i in cfg.fullatt_block_indexes else info_win
            y, _ = ops.rmsnorm(h, blk.norm1, 1e-6)
            qkv = ops.linear(y, blk.qkv_weight, blk.qkv_bias)
            qkv = ops.rope(qkv, 2 * nh, hd, pos3, rope[0], rope[1], mrope_section=(quarter, quarter, 0))
            a = attention_packed(qkv, info, nh, nh, hd, causal=False, scale=1.0 / math.sqrt(hd))
            h = h + ops.linear(a, blk.proj_weight, blk.proj_bias)
            y, _ = ops.rmsnorm(h, blk.norm2, 1e-6)
            h = h + ops.linear(ops.swiglu(ops.linear(y, blk.gate_up_weight, blk.gate_up_bias)), blk.down_weight,
                               blk.down_bias)
        y, _ = ops.rmsnorm(h, self.merger_norm, 1e-6)
        y = y.reshape(N // m, m * cfg.hidden_size)
        y = F.gelu(ops.linear(y, self.merger_fc1_weight, self.merger_fc1_bias))
        y = ops.linear(y, self.merger_fc2_weight, self.merger_fc2_bias)
        inverse = torch.argsort(unit_order).to(dev)
        return y.index_select(0, inverse)


def mrope_positions(input_ids: torch.Tensor, image_token_id: int, grid_thw: torch.Tensor, merge: int) -> torch.Tensor:
    """3-row (t, h, w) rope positions of ONE sequence with image placeholders (Qwen2-VL multimodal rope; the
    reference builds them in the dataset, partitioned_dataset.py:333-442 via ``get_rope_index``).  Text tokens
    advance all three rows together; an image occupies a (t, h/merge, w/merge) grid starting at the current offset;
    the next text token continues after the largest index used."""
    ids = input_ids.tolist()
    out = torch.zeros(3, len(ids), dtype=torch.int64)
    nxt, i, img = 0, 0, 0
    while i < len(ids):
        if ids[i] == image_token_id and img < grid_thw.shape[0]:
            t, h, w = [int(v) for v in grid_thw[img].tolist()]
            gh, gw = h // merge, w // merge
            n = t * gh * gw
            tt = torch.arange(t).repeat_interleave(gh * gw)
            hh = torch.arange(gh).repeat_interleave(gw).repeat(t)
            ww = torch.arange(gw).repeat(gh * t)
            n = min(n, len(ids) - i)
            out[0, i:i + n], out[1, i:i + n], out[2, i:i + n] = tt[:n] + nxt, hh[:n] + nxt, ww[:n] + nxt
            nxt = nxt + max(t, gh, gw)
            i += n
            img += 1
        else:
            out[:, i] = nxt
            nxt += 1
            i += 1
    return out
