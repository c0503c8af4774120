"""Plain-PyTorch statements of every op in ``siirl_b200.ops``.

They are (1) the CPU path, so the whole framework runs under gloo on machines without a GPU, and
(2) the fp32 oracles the CUDA kernels are tested against.  Nothing here is tuned.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None):
    """Returns (y, h) with h = x + residual (or x) and y = h * rsqrt(mean(h^2)+eps) * weight."""
    h = x if residual is None else x + residual
    hf = h.float()
    rstd = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
    y = (hf * rstd * weight.float()).to(x.dtype)
    return y, h


def yarn_mscale(scale: float, mscale: float = 1.0) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


def scaled_inv_freq(head_dim: int, theta: float, scaling: Optional[dict], device=None):
    """Inverse rotary frequencies under a checkpoint's ``rope_scaling`` (public formulas: "linear" divides every
    frequency by ``factor``; "llama3" keeps the high frequencies, divides the low ones and blends between the two
    wavelength bounds; "yarn" blends interpolated and original frequencies with a linear ramp between the dimensions
    whose wavelength completes ``beta_fast`` / ``beta_slow`` rotations inside the original context).  Returns
    ``(inv_freq, attention_factor)``; cos / sin are multiplied by the factor (yarn's temperature correction)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64, device=device) / head_dim))
    if not scaling:
        return inv, 1.0
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    factor = float(scaling.get("factor", 1.0))
    if kind == "linear":
        return inv / factor, 1.0
    if kind == "llama3":
        lo, hi = float(scaling.get("low_freq_factor", 1.0)), float(scaling.get("high_freq_factor", 4.0))
        old = float(scaling.get("original_max_position_embeddings", 8192))
        wavelen = 2 * math.pi / inv
        smooth = ((old / wavelen - lo) / (hi - lo)).clamp(0, 1)
        blended = (1 - smooth) * inv / factor + smooth * inv
        out = torch.where(wavelen > old / lo, inv / factor, torch.where(wavelen < old / hi, inv, blended))
        return out, 1.0
    if kind == "yarn":
        old = float(scaling.get("original_max_position_embeddings", 4096))
        fast, slow = float(scaling.get("beta_fast", 32)), float(scaling.get("beta_slow", 1))

        def corr_dim(rot):
            return head_dim * math.log(old / (rot * 2 * math.pi)) / (2 * math.log(theta))
        low, high = corr_dim(fast), corr_dim(slow)
        if scaling.get("truncate", True):
            low, high = math.floor(low), math.ceil(high)
        low, high = max(low, 0), min(high, head_dim - 1)
        if low == high:
            high += 0.001
        ramp = ((torch.arange(head_dim // 2, dtype=torch.float64, device=device) - low) / (high - low)).clamp(0, 1)
        keep = 1 - ramp                                   # 1: original frequency, 0: interpolated
        out = inv / factor * (1 - keep) + inv * keep
        ms, ms_all = scaling.get("mscale"), scaling.get("mscale_all_dim")
        if scaling.get("attention_factor") is not None:
            att = float(scaling["attention_factor"])
        elif ms and ms_all:
            att = yarn_mscale(factor, float(ms)) / yarn_mscale(factor, float(ms_all))
        else:
            att = yarn_mscale(factor)
        return out, att
    return inv, 1.0


def rope_tables(head_dim: int, max_pos: int, theta: float, device=None, scaling: Optional[dict] = None):
    inv, att = scaled_inv_freq(head_dim, theta, scaling, device)
    t = torch.arange(max_pos, dtype=torch.float64, device=device)
    ang = torch.outer(t, inv)
    return (ang.cos() * att).float(), (ang.sin() * att).float()


def _select_pos(positions: torch.Tensor, half: int, mrope_section):
    """positions [T] or [3, T] -> per (token, freq) position index [T, half]."""
    if positions.dim() == 1:
        return positions[:, None].expand(-1, half)
    s0, s1 = mrope_section[0], mrope_section[0] + mrope_section[1]
    idx = torch.arange(half, device=positions.device)
    row = torch.where(idx < s0, 0, torch.where(idx < s1, 1, 2))
    return positions[row, :].t()


def rope(x: torch.Tensor, positions: torch.Tensor, cos_tab: torch.Tensor, sin_tab: torch.Tensor,
         mrope_section=None, inverse: bool = False) -> torch.Tensor:
    """x [T, n_heads, D] rotate-half RoPE; positions [T] (or [3,T] with mrope_section)."""
    T, nh, D = x.shape
    half = D // 2
    p = _select_pos(positions.long(), half, mrope_section)
    fi = torch.arange(half, device=x.device)[None, :].expand(T, -1)
    c = cos_tab[p, fi][:, None, :]
    s = sin_tab[p, fi][:, None, :]
    if inverse:
        s = -s
    xf = x.float()
    a, b = xf[..., :half], xf[..., half:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(x.dtype)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    g, u = gate_up.float().chunk(2, dim=-1)
    return (F.silu(g) * u).to(gate_up.dtype)


def attention_varlen(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                     causal: bool = True, scale: Optional[float] = None,
                     window: Optional[int] = None) -> torch.Tensor:
    """Packed variable-length attention.  q [T, Hq, D], k/v [T, Hkv, D]; sequences are
    the slices cu_seqlens[i]:cu_seqlens[i+1].  GQA by head repetition.  Returns [T, Hq, Dv]."""
    T, hq, D = q.shape
    hkv = k.shape[1]
    rep = hq // hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    out = q.new_empty(T, hq, v.shape[-1])      # the value width may differ from the query / key width
    cs = cu_seqlens.tolist()
    for i in range(len(cs) - 1):
        a, b = cs[i], cs[i + 1]
        if b <= a:
            continue
        qi = q[a:b].transpose(0, 1).float()
        ki = k[a:b].transpose(0, 1).repeat_interleave(rep, dim=0).float()
        vi = v[a:b].transpose(0, 1).repeat_interleave(rep, dim=0).float()
        s = torch.matmul(qi, ki.transpose(1, 2)) * scale
        L = b - a
        if causal:
            mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
            s = s.masked_fill(~mask, float("-inf"))
        if window is not None:
            idx = torch.arange(L, device=q.device)
            far = (idx[:, None] - idx[None, :]).abs() >= window
            s = s.masked_fill(far, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[a:b] = torch.matmul(p, vi).transpose(0, 1).to(q.dtype)
    return out


def lm_head_logprob_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                            temperature: float = 1.0, with_entropy: bool = True):
    """log p(label) and categorical entropy of softmax(hidden @ weight^T / temperature), fp32.

    Semantics of the reference's fused linear-cross-entropy family
    (siirl/utils/kernel/linear_cross_entropy.py:40-117)."""
    logits = (hidden.float() @ weight.float().t()) / temperature
    lse = torch.logsumexp(logits, dim=-1)
    logp = logits.gather(-1, labels.long()[:, None]).squeeze(-1) - lse
    ent = None
    if with_entropy:
        p = torch.softmax(logits, dim=-1)
        ent = lse - (p * logits).sum(-1)
    return logp, ent


def sample_tokens(logits: torch.Tensor, temperature: float, top_k: int, top_p: float,
                  generator: Optional[torch.Generator] = None):
    """Temperature / top-k / top-p sampling; returns (token ids, log-prob of the sampled id under the
    tempered, *untruncated* distribution).  temperature == 0 means greedy."""
    lf = logits.float()
    if temperature == 0.0:
        ids = lf.argmax(-1)
        lp = torch.log_softmax(lf, -1).gather(-1, ids[:, None]).squeeze(-1)
        return ids, lp
    lf = lf / temperature
    logp_full = torch.log_softmax(lf, -1)
    filt = lf.clone()
    if top_k is not None and top_k > 0 and top_k < lf.shape[-1]:
        kth = torch.topk(filt, top_k, dim=-1).values[..., -1:]
        filt = filt.masked_fill(filt < kth, float("-inf"))
    if top_p is not None and top_p < 1.0:
        sp, si = torch.sort(torch.softmax(filt, -1), dim=-1, descending=True)
        cum = sp.cumsum(-1)
        drop = (cum - sp) >= top_p
        sp = sp.masked_fill(drop, 0.0)
        probs = torch.zeros_like(sp).scatter(-1, si, sp)
    else:
        probs = torch.softmax(filt, -1)
    ids = torch.multinomial(probs, 1, generator=generator).squeeze(-1)
    return ids, logp_full.gather(-1, ids[:, None]).squeeze(-1)
