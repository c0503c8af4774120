"""Continuous-action modules of OpenVLA-OFT: L1-regression action head, diffusion action head, proprioception projector,
and the (un)normalisation of actions / proprioceptive state with dataset statistics.

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
* ``DiffusionActionHead`` + ``DDIMSchedule``: the action rows carry the projected noisy action chunk, a timestep
  pseudo-token sits behind the patches, a residual MLP predicts the noise; sampling is deterministic DDIM
  (modeling_prismatic.py:1399-1483 ``_run_diffusion_prediction``).
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


# ---- diffusion head ------------------------------------------------------------------------------------------------
class DDIMSchedule:
    """Discrete-time diffusion with the squared-cosine noise schedule and deterministic (eta = 0) DDIM sampling of an
    epsilon-predicting model: ``x_t = sqrt(abar_t) x_0 + sqrt(1 - abar_t) eps``."""

    def __init__(self, num_train_steps: int = 100):
        import math
        self.num_train_steps = num_train_steps
        f = lambda u: math.cos((u + 0.008) / 1.008 * math.pi / 2) ** 2        # noqa: E731
        betas = [min(1.0 - f((i + 1) / num_train_steps) / f(i / num_train_steps), 0.999) for i in range(num_train_steps)]
        self.alphas_cumprod = torch.cumprod(1.0 - torch.tensor(betas, dtype=torch.float64), 0).float()

    def add_noise(self, x0: torch.Tensor, noise: torch.Tensor, t: torch.Tensor) -> torch.Tensor:
        ab = self.alphas_cumprod[t].reshape(-1, *([1] * (x0.dim() - 1)))
        return ab.sqrt() * x0 + (1.0 - ab).sqrt() * noise

    def inference_steps(self, n: int):
        """``(t, previous t)`` pairs from the noisiest step down; the previous step of the last one is -1 (clean)."""
        n = max(1, min(n, self.num_train_steps))
        ts = [int(round(i * (self.num_train_steps - 1) / max(n - 1, 1))) for i in range(n)][::-1] if n > 1 \
            else [self.num_train_steps - 1]
        return list(zip(ts, ts[1:] + [-1]))

    def step(self, eps: torch.Tensor, t: int, t_prev: int, x: torch.Tensor) -> torch.Tensor:
        ab = self.alphas_cumprod[t]
        ab_prev = self.alphas_cumprod[t_prev] if t_prev >= 0 else torch.tensor(1.0)
        x0 = ((x - (1.0 - ab).sqrt() * eps) / ab.sqrt()).clamp(-1.0, 1.0)        # actions live in [-1, 1]
        eps = (x - ab.sqrt() * x0) / (1.0 - ab).sqrt()
        return ab_prev.sqrt() * x0 + (1.0 - ab_prev).sqrt() * eps


class DiffusionActionHead(nn.Module):
    """OpenVLA-OFT's diffusion head: the decoder sees the noisy action chunk (every scalar projected to one row of the
    language model's width) plus a timestep pseudo-token, and a residual MLP predicts the noise from the hidden
    states of the action rows; sampling runs ``num_inference_steps`` DDIM steps, one decoder forward each."""

    def __init__(self, hidden_size: int, action_dim: int = 7, head_hidden: Optional[int] = None, blocks: int = 2,
                 num_train_steps: int = 100, num_inference_steps: int = 50, dtype=torch.bfloat16, device="cpu",
                 seed: int = 0):
        super().__init__()
        gen = torch.Generator().manual_seed(seed)
        self.action_dim, self.hidden_size = action_dim, hidden_size
        self.num_inference_steps = num_inference_steps
        self.schedule = DDIMSchedule(num_train_steps)
        self.mlp = _ResidualMLP(hidden_size * action_dim, head_hidden or hidden_size, action_dim, blocks, dtype, device,
                                gen)
        # noisy scalar -> row of the model's width: Linear(1, H) is an outer product, kept as a vector pair
        self.act_in_weight = nn.Parameter((torch.randn(hidden_size, generator=gen) * 0.5).to(device=device, dtype=dtype))
        self.act_in_bias = nn.Parameter(torch.zeros(hidden_size, dtype=dtype, device=device))
        self.act_out_weight, self.act_out_bias = _linear_param(hidden_size, hidden_size, dtype, device, gen)
        self.time_weight, self.time_bias = _linear_param(hidden_size, hidden_size, dtype, device, gen)

    def project_noisy_actions(self, x: torch.Tensor) -> torch.Tensor:
        """``[N, chunk, action_dim]`` noisy actions -> ``[N, chunk * action_dim, H]`` input rows."""
        w = self.act_in_weight
        v = x.reshape(x.shape[0], -1, 1).to(w.device, torch.float32)
        h = F.gelu(v * w.float() + self.act_in_bias.float()).to(w.dtype)
        return ops.linear(h.reshape(-1, self.hidden_size), self.act_out_weight, self.act_out_bias).reshape(
            x.shape[0], -1, self.hidden_size)

    def time_embedding(self, t: torch.Tensor) -> torch.Tensor:
        """Sinusoidal features of the timestep -> ``[N, H]`` pseudo-token."""
        import math
        half = self.hidden_size // 2
        freq = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32) / max(half - 1, 1))
        ang = t.float().reshape(-1, 1) * freq[None, :]
        emb = torch.cat([ang.sin(), ang.cos()], -1)
        if emb.shape[-1] < self.hidden_size:
            emb = F.pad(emb, (0, self.hidden_size - emb.shape[-1]))
        emb = emb.to(self.time_weight.device, self.time_weight.dtype)
        return ops.linear(emb, self.time_weight, self.time_bias)

    def predict_noise(self, action_hidden: torch.Tensor) -> torch.Tensor:
        N, rows, H = action_hidden.shape
        return self.mlp(action_hidden.reshape(N, rows // self.action_dim, self.action_dim * H))


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


def load_action_norm_stats(model_path: Optional[str], unnorm_key: str) -> Optional[Dict[str, Sequence[float]]]:
    """Action statistics of one dataset from a fine-tuned checkpoint: ``dataset_statistics.json`` beside the weights,
    else ``norm_stats`` inside ``config.json`` (where OpenVLA keeps them).  ``unnorm_key`` falls back to
    ``<key>_no_noops`` as the reference does (siirl/engine/rollout/embodied_rollout.py:197-200,
    siirl/engine/fsdp_workers.py:456-470).  ``None`` when the checkpoint carries no statistics (base checkpoints,
    random-init models): actions then stay in ``[-1, 1]``."""
    import json
    import os
    if not model_path or not os.path.isdir(str(model_path)):
        return None
    stats = None
    f = os.path.join(str(model_path), "dataset_statistics.json")
    if os.path.isfile(f):
        with open(f) as fh:
            stats = json.load(fh)
    else:
        c = os.path.join(str(model_path), "config.json")
        if os.path.isfile(c):
            with open(c) as fh:
                stats = json.load(fh).get("norm_stats")
    if not stats:
        return None
    key = unnorm_key if unnorm_key in stats else f"{unnorm_key}_no_noops"
    if key not in stats:
        raise KeyError(f"action un-normalisation key {unnorm_key!r} not found in the checkpoint's statistics "
                       f"(have: {sorted(stats)})")
    return stats[key].get("action", stats[key])
