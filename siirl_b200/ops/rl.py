"""RL post-processing ops: GAE scan, GRPO group advantage, fused PPO token loss.

CUDA tensors use the kernels in ``csrc/rl_algos.cu``; CPU tensors use the vectorised PyTorch code below
(also the oracle in tests)."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import lib as _lib

_f = ctypes.c_float


def gae_scan_reference(rewards, values, mask, gamma: float, lam: float):
    B, R = rewards.shape
    nextvalues = torch.zeros(B, dtype=torch.float32, device=rewards.device)
    lastgaelam = torch.zeros_like(nextvalues)
    adv = torch.zeros_like(rewards, dtype=torch.float32)
    for t in reversed(range(R)):
        delta = rewards[:, t] + gamma * nextvalues - values[:, t]
        lg = delta + gamma * lam * lastgaelam
        m = mask[:, t]
        nextvalues = values[:, t] * m + (1 - m) * nextvalues
        lastgaelam = lg * m + (1 - m) * lastgaelam
        adv[:, t] = lastgaelam
    return adv, adv + values


def gae_scan(rewards: torch.Tensor, values: torch.Tensor, mask: torch.Tensor, gamma: float, lam: float):
    """Un-whitened GAE advantages and returns (= advantages + values), ``[B, R]`` fp32."""
    if not rewards.is_cuda:
        return gae_scan_reference(rewards.float(), values.float(), mask.float(), gamma, lam)
    L = _lib.get_lib()
    r, v, m = (t.float().contiguous() for t in (rewards, values, mask))
    adv, ret = torch.empty_like(r), torch.empty_like(r)
    B, R = r.shape
    _lib.check(L.sb_gae_scan(_lib.ptr(r), _lib.ptr(v), _lib.ptr(m), _lib.ptr(adv), _lib.ptr(ret), B, R,
                             _f(gamma), _f(lam), _lib.stream()), "sb_gae_scan")
    return adv, ret


def grpo_group_advantage(rewards: torch.Tensor, mask: torch.Tensor, group_ids: torch.Tensor, num_groups: int,
                         eps: float = 1e-6, norm_by_std: bool = True) -> torch.Tensor:
    """``adv[b, t] = (s_b - mean_g) / (std_g + eps) * mask`` with dense int group ids in ``[0, num_groups)``;
    a singleton group has mean 0 / std 1."""
    assert rewards.is_cuda
    L = _lib.get_lib()
    r, m = rewards.float().contiguous(), mask.float().contiguous()
    gid = group_ids.to(torch.int32).contiguous()
    B, R = r.shape
    scores = torch.empty(B, dtype=torch.float32, device=r.device)
    ws = torch.empty(3 * num_groups, dtype=torch.float32, device=r.device)
    adv = torch.empty_like(r)
    _lib.check(L.sb_grpo_group_adv(_lib.ptr(r), _lib.ptr(m), _lib.ptr(gid), _lib.ptr(scores), _lib.ptr(ws),
                                   _lib.ptr(adv), B, R, num_groups, _f(eps), int(norm_by_std), _lib.stream()),
               "sb_grpo_group_adv")
    return adv


_KL_KIND = {None: 0, "low_var_kl": 1, "k3": 1, "kl": 2, "k1": 2, "abs": 3, "mse": 4, "k2": 4}
_MODE = {"vanilla": 0, "gspo": 1, "cpgd": 2}


def agg_row_weights(mask: torch.Tensor, loss_agg_mode: str) -> torch.Tensor:
    """Per-row weight w_b such that the aggregated loss equals sum_bt w_b * m_bt * l_bt."""
    B, R = mask.shape
    mf = mask.float()
    if loss_agg_mode == "token-mean":
        return torch.full((B,), 1.0, device=mask.device) / (mf.sum() + 1e-8)
    if loss_agg_mode == "seq-mean-token-sum":
        return torch.full((B,), 1.0 / B, device=mask.device)
    if loss_agg_mode == "seq-mean-token-mean":
        return 1.0 / ((mf.sum(-1) + 1e-8) * B)
    if loss_agg_mode == "seq-mean-token-sum-norm":
        return torch.full((B,), 1.0 / R, device=mask.device)
    raise ValueError(f"Invalid loss_agg_mode: {loss_agg_mode}")


class _PpoLossFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logp, entropy, old_logp, adv, mask, ref_logp, mode, loss_agg_mode, clip_lo, clip_hi, clip_c,
                kl_kind, kl_coef, entropy_coef):
        L = _lib.get_lib()
        B, R = logp.shape
        lp = logp.float().contiguous()
        mf = mask.float().contiguous()
        agg = "seq-mean-token-mean" if mode == "gspo" else loss_agg_mode
        w = agg_row_weights(mf, agg).contiguous()
        seq_lr = None
        if mode == "gspo":
            seq_lr = (((lp - old_logp.float()) * mf).sum(-1) / mf.sum(-1).clamp(min=1)).contiguous()
        dlogp = torch.empty_like(lp)
        ent = entropy.float().contiguous() if entropy is not None else None
        dent = torch.empty_like(lp) if ent is not None else None
        stats = torch.empty(8, dtype=torch.float32, device=lp.device)
        _lib.check(L.sb_ppo_token_loss(
            _lib.ptr(lp), _lib.ptr(old_logp.float().contiguous()), _lib.ptr(adv.float().contiguous()),
            _lib.ptr(mf), _lib.ptr(ref_logp.float().contiguous() if ref_logp is not None else None),
            _lib.ptr(ent), _lib.ptr(w), _lib.ptr(seq_lr), _lib.ptr(dlogp), _lib.ptr(dent), _lib.ptr(stats), B, R,
            _MODE[mode], _f(clip_lo), _f(clip_hi), _f(clip_c), _KL_KIND[kl_kind if ref_logp is not None else None],
            _f(kl_coef), _f(entropy_coef), _f(1.0), _lib.stream()), "sb_ppo_token_loss")
        ctx.save_for_backward(dlogp, dent)
        pg_loss, kl_loss, ent_loss = stats[0], stats[4], stats[5]
        total = pg_loss + kl_coef * kl_loss - entropy_coef * ent_loss
        ctx.mark_non_differentiable(stats)
        return total, stats

    @staticmethod
    def backward(ctx, gtotal, _gstats):
        dlogp, dent = ctx.saved_tensors
        return (dlogp * gtotal, (dent * gtotal) if dent is not None else None) + (None,) * 12


def ppo_token_loss(logp, old_logp, adv, mask, *, entropy=None, ref_logp=None, mode: str = "vanilla",
                   loss_agg_mode: str = "token-mean", clip_lo: float = 0.2, clip_hi: float = 0.2,
                   clip_c: float = 3.0, kl_kind: Optional[str] = "low_var_kl", kl_coef: float = 0.0,
                   entropy_coef: float = 0.0) -> Tuple[torch.Tensor, dict]:
    """Fused actor loss ``pg + kl_coef * KL(logp, ref) - entropy_coef * H`` for CUDA tensors.

    Returns ``(loss, metrics)`` where metrics holds detached tensors ``pg_loss, pg_clipfrac, ppo_kl,
    pg_clipfrac_lower, kl_loss, entropy_loss``.  One kernel computes the forward statistics and
    d(loss)/d(logp), d(loss)/d(entropy)."""
    assert logp.is_cuda
    total, stats = _PpoLossFn.apply(logp, entropy, old_logp, adv, mask, ref_logp, mode, loss_agg_mode, clip_lo,
                                    clip_hi, clip_c, kl_kind, kl_coef, entropy_coef)
    msum = stats[6].clamp(min=1e-8)
    metrics = {"pg_loss": stats[0], "pg_clipfrac": stats[1] / msum, "ppo_kl": stats[2] / msum,
               "pg_clipfrac_lower": stats[3] / msum, "kl_loss": stats[4], "entropy_loss": stats[5]}
    return total, metrics
