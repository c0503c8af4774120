"""Continuous-action modules of OpenVLA-OFT: L1-regression action head, proprioception projector, and the
(un)normalisation of actions / proprioceptive state with dataset statistics.

The reference's OpenVLA-OFT model takes these as outside modules (``action_head`` / ``proprio_projector`` arguments of
siirl/models/embodied/openvla_oft/modeling_prismatic.py:1485-1550 ``_regression_or_discrete_prediction``, :449-459
``_process_proprio_features``, :1378-1397 ``_unnormalize_actions``); its RL path samples the discrete action tokens,
the continuous head serves supervised fine-tuning and evaluation of such checkpoints.  Here they are plain modules on
the package's GEMM (``ops.linear``) that read the decoder's final hidden states of the action placeholder rows:

* ``L1RegressionActionHead``: the hidden states of the ``chunk * action_dim`` placeholder rows of one control step are
  regrouped to ``[chunk, action_dim * H]`` and mapped by a residual MLP to ``[chunk, action_dim]`` normalised actions;
  trained with an L1 loss.
* ``ProprioProjector``: ``Linear -> GELU -> Linear`` from the robot state to one pseudo-token of the language model's
  width, placed directly behind the image patch rows.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops


def _linear_param(out_dim: int, in_dim: int, dtype, device, gen: torch.Generator):
    w = torch.empty(out_dim, in_dim, dtype=torch.float32)
    bound = (1.0 / in_dim) ** 0.5
    w.uniform_(-bound, bound, generator=gen)
    return nn.Parameter(w.to(device=device, dtype=dtype)), nn.Parameter(torch.zeros(out_dim, dtype=dtype, device=device))


class _ResidualMLP(nn.Module):
    """``LayerNorm -> Linear -> ReLU -> [x + ReLU(Linear(LayerNorm(x)))] * blocks -> LayerNorm -> Linear``."""

    def __init__(self, in_dim: int, hidden_dim: int, out_dim: int, blocks: int, dtype, device, gen):
        super().__init__()
        self.blocks = blocks
        self.in_norm = nn.LayerNorm(in_dim, dtype=dtype, device=device)
        self.fc_in_weight, self.fc_in_bias = _linear_param(hidden_dim, in_dim, dtype, device, gen)
        for i in range(blocks):
            setattr(self, f"norm{i}", nn.LayerNorm(hidden_dim, dtype=dtype, device=device))
            w, b = _linear_param(hidden_dim, hidden_dim, dtype, device, gen)
            setattr(self, f"fc{i}_weight", w)
            setattr(self, f"fc{i}_bias", b)
        self.out_norm = nn.LayerNorm(hidden_dim, dtype=dtype, device=device)
        self.fc_out_weight, self.fc_out_bias = _linear_param(out_dim, hidden_dim, dtype, device, gen)

    @staticmethod
    def _ln(norm: nn.LayerNorm, x: torch.Tensor) -> torch.Tensor:
        return F.layer_norm(x.float(), norm.normalized_shape, norm.weight.float(), norm.bias.float(), norm.eps).to(x.dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shp = x.shape
        x = x.reshape(-1, shp[-1])
        x = F.relu(ops.linear(self._ln(self.in_norm, x), self.fc_in_weight, self.fc_in_bias))
        for i in range(self.blocks):
            y = ops.linear(self._ln(getattr(self, f"norm{i}"), x), getattr(self, f"fc{i}_weight"),
                           getattr(self, f"fc{i}_bias"))
            x = x + F.relu(y)
        x = self._ln(self.out_norm, x)
        # the last projection has ``action_dim`` (7) output columns: below the GEMM kernel's 8-column granule, and
        # tiny, so it is a plain matrix product
        y = x.float() @ self.fc_out_weight.float().t() + self.fc_out_bias.float()
        return y.reshape(*shp[:-1], y.shape[-1])


class L1RegressionActionHead(nn.Module):
    def __init__(self, hidden_size: int, action_dim: int = 7, head_hidden: Optional[int] = None, blocks: int = 2,
                 dtype=torch.bfloat16, device="cpu", seed: int = 0):
        super().__init__()
        gen = torch.Generator().manual_seed(seed)
        self.action_dim = action_dim
        self.mlp = _ResidualMLP(hidden_size * action_dim, head_hidden or hidden_size, action_dim, blocks, dtype, device,
                                gen)

    def predict_action(self, action_hidden: torch.Tensor) -> torch.Tensor:
        """``[N, chunk * action_dim, H]`` hidden states of the action rows -> ``[N, chunk, action_dim]`` fp32
        normalised actions (roughly in ``[-1, 1]``)."""
        N, rows, H = action_hidden.shape
        assert rows % self.action_dim == 0, "action rows come in groups of action_dim"
        return self.mlp(action_hidden.reshape(N, rows // self.action_dim, self.action_dim * H))

    def l1_loss(self, action_hidden: torch.Tensor, target_actions: torch.Tensor) -> torch.Tensor:
        return (self.predict_action(action_hidden) - target_actions.float()).abs().mean()


class ProprioProjector(nn.Module):
    def __init__(self, proprio_dim: int, llm_dim: int, dtype=torch.bfloat16, device="cpu", seed: int = 0):
        super().__init__()
        gen = torch.Generator().manual_seed(seed)
        self.proprio_dim = proprio_dim
        self.in_dim = (proprio_dim + 7) // 8 * 8       # the GEMM reads 16-byte rows: state vectors are zero-padded
        w, self.fc1_bias = _linear_param(llm_dim, self.in_dim, dtype, device, gen)
        with torch.no_grad():
            w[:, proprio_dim:].zero_()
        self.fc1_weight = w
        self.fc2_weight, self.fc2_bias = _linear_param(llm_dim, llm_dim, dtype, device, gen)

    def forward(self, proprio: torch.Tensor) -> torch.Tensor:
        """``[N, proprio_dim]`` normalised state -> ``[N, llm_dim]`` pseudo-token embeddings."""
        x = proprio.to(self.fc1_weight.device, self.fc1_weight.dtype)
        if x.shape[-1] != self.in_dim:
            x = F.pad(x, (0, self.in_dim - x.shape[-1]))
        x = F.gelu(ops.linear(x, self.fc1_weight, self.fc1_bias).float()).to(x.dtype)
        return ops.linear(x, self.fc2_weight, self.fc2_bias)


# ---- dataset statistics -------------------------------------------------------------------------------------------
def _bounds(stats: Dict[str, Sequence[float]], kind: str):
    if kind == "bounds":
        lo, hi = stats["min"], stats["max"]
    elif kind == "bounds_q99":
        lo, hi = stats["q01"], stats["q99"]
    else:
        raise ValueError(f"unknown normalisation type {kind!r} (expected 'bounds' or 'bounds_q99')")
    lo, hi = torch.as_tensor(lo, dtype=torch.float32), torch.as_tensor(hi, dtype=torch.float32)
    mask = torch.as_tensor(stats.get("mask", [True] * lo.numel()), dtype=torch.bool)
    return lo, hi, mask


def unnormalize_actions(normalized: torch.Tensor, stats: Dict[str, Sequence[float]], kind: str = "bounds_q99") -> torch.Tensor:
    """``[-1, 1]`` actions -> robot units: ``0.5 (a + 1) (high - low) + low`` on the dimensions the dataset marks (the
    gripper dimension is usually left as is)."""
    lo, hi, mask = _bounds(stats, kind)
    a = normalized.float().cpu()
    return torch.where(mask, 0.5 * (a + 1.0) * (hi - lo + 1e-8) + lo, a)


def normalize_proprio(proprio: torch.Tensor, stats: Dict[str, Sequence[float]], kind: str = "bounds_q99") -> torch.Tensor:
    """Robot state -> ``[-1, 1]`` with the same statistics convention (clipped)."""
    lo, hi, mask = _bounds(stats, kind)
    p = proprio.float().cpu()
    return torch.where(mask, (2.0 * (p - lo) / (hi - lo + 1e-8) - 1.0).clamp(-1.0, 1.0), p)
