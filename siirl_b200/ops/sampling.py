"""Token sampling (temperature / greedy by a Gumbel-max kernel; top-k / top-p by truncating the logits first)."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import lib as _lib
from . import reference as ref


def _truncate(logits: torch.Tensor, temperature: float, top_k: int, top_p: float) -> torch.Tensor:
    z = logits / max(temperature, 1e-6)
    if top_k is not None and 0 < top_k < z.shape[-1]:
        kth = torch.topk(z, top_k, dim=-1).values[..., -1:]
        z = z.masked_fill(z < kth, float("-inf"))
    if top_p is not None and top_p < 1.0:
        sp, si = torch.sort(torch.softmax(z, -1), dim=-1, descending=True)
        drop = (sp.cumsum(-1) - sp) >= top_p
        keep = torch.zeros_like(drop).scatter(-1, si, ~drop)
        z = z.masked_fill(~keep, float("-inf"))
    return z * max(temperature, 1e-6)


def sample(logits: torch.Tensor, temperature: float = 1.0, top_k: int = -1, top_p: float = 1.0, seed: int = 0,
           step: int = 0, generator: Optional[torch.Generator] = None,
           step_dev: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(token ids int64 [B], log-prob fp32 [B])``.  The log-prob is that of the chosen token under the
    full tempered distribution (what PPO needs as the behaviour log-prob).  ``temperature == 0`` is greedy.
    ``(seed, step [+ step_dev[0]])`` index the counter-based random stream (``step_dev`` is an int64 device counter
    for CUDA-graph replays), so equal logits give equal tokens on every rank."""
    if not logits.is_cuda:
        return ref.sample_tokens(logits, temperature, top_k, top_p, generator)
    L = _lib.get_lib()
    lf = logits.float().contiguous()
    B, V = lf.shape
    truncated = lf
    if temperature > 0 and ((top_k is not None and 0 < top_k < V) or (top_p is not None and top_p < 1.0)):
        truncated = _truncate(lf, temperature, top_k, top_p).contiguous()
    tokens = torch.empty(B, dtype=torch.int64, device=lf.device)
    logp = torch.empty(B, dtype=torch.float32, device=lf.device)
    # few rows, huge vocabulary: split every row over several blocks so the whole GPU reads the logits
    splits = max(1, min(32, (2 * 148) // max(B, 1), V // 4096))
    ws = torch.empty(B * splits * 4, dtype=torch.float32, device=lf.device) if splits > 1 else None
    _lib.check(L.sb_sample(_lib.ptr(truncated), _lib.ptr(lf), ctypes.c_longlong(lf.stride(0)),
                           ctypes.c_float(temperature), ctypes.c_ulonglong(seed & (2 ** 64 - 1)),
                           ctypes.c_ulonglong(step), _lib.ptr(step_dev), _lib.ptr(tokens), _lib.ptr(logp), B, V,
                           _lib.ptr(ws), splits, _lib.stream()), "sb_sample")
    return tokens, logp
