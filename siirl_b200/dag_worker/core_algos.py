"""RL algorithm layer: advantage estimators, policy/value losses, KL penalties and controllers.

Semantics follow the reference (siirl/dag_worker/core_algos.py); the implementations are vectorised
(segmented reductions by ``uid`` instead of Python dict loops, scans instead of per-token Python)
so they run unchanged on GPU tensors.  All per-token tensors are ``[B, R]`` over the response part
and ``response_mask`` marks valid tokens.

Registries (same decorator API as the reference, core_algos.py:51-164):
``@register_adv_est(name)`` for ``fn(token_level_rewards, response_mask, **kw) -> (advantages, returns)``
and ``@register_policy_loss(name)`` for
``fn(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode, config, rollout_is_weights)
-> (pg_loss, pg_clipfrac, ppo_kl, pg_clipfrac_lower)``.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Tuple

import numpy as np
import torch

from ..execution.scheduler.enums import AdvantageEstimator

POLICY_LOSS_REGISTRY: Dict[str, Callable] = {}
ADV_ESTIMATOR_REGISTRY: Dict[str, Callable] = {}


def register_policy_loss(name: str):
    def deco(fn):
        POLICY_LOSS_REGISTRY[name] = fn
        return fn
    return deco


def get_policy_loss_fn(name: str) -> Callable:
    if name not in POLICY_LOSS_REGISTRY:
        raise ValueError(f"Unsupported loss mode: {name}. Supported modes are: {sorted(POLICY_LOSS_REGISTRY)}")
    return POLICY_LOSS_REGISTRY[name]


def register_adv_est(name):
    key = name.value if hasattr(name, "value") else name

    def deco(fn):
        if key in ADV_ESTIMATOR_REGISTRY and ADV_ESTIMATOR_REGISTRY[key] is not fn:
            raise ValueError(f"advantage estimator '{key}' already registered")
        ADV_ESTIMATOR_REGISTRY[key] = fn
        return fn
    return deco


def get_adv_estimator_fn(name) -> Callable:
    key = name.value if hasattr(name, "value") else name
    if key not in ADV_ESTIMATOR_REGISTRY:
        raise ValueError(f"Unknown advantage estimator: {key}")
    return ADV_ESTIMATOR_REGISTRY[key]


# ---------------------------------------------------------------------------------------------
# masked statistics
# ---------------------------------------------------------------------------------------------
def masked_sum(x, mask, dim=None):
    return (x * mask).sum() if dim is None else (x * mask).sum(dim)


def masked_mean(x, mask, dim=None):
    if dim is None:
        return (x * mask).sum() / (mask.sum() + 1e-8)
    return (x * mask).sum(dim) / (mask.sum(dim) + 1e-8)


def masked_var(x, mask, unbiased: bool = True):
    mean = masked_mean(x, mask)
    var = masked_mean((x - mean) ** 2, mask)
    if unbiased:
        n = mask.sum()
        if n.item() <= 1:
            return var
        var = var * (n / (n - 1))
    return var


def masked_whiten(x, mask, shift_mean: bool = True):
    mean, var = masked_mean(x, mask), masked_var(x, mask)
    out = (x - mean) * torch.rsqrt(var + 1e-8)
    if not shift_mean:
        out = out + mean
    return out


def compute_response_mask(batch) -> torch.Tensor:
    """Mask of the response part: the last R columns of ``attention_mask`` (R = responses.shape[1]);
    for embodied 3-D responses ``[B, traj, act]`` the flattened ``traj*act`` length is used
    (reference core_algos.py:89-125)."""
    responses = batch["responses"]
    R = responses.shape[1] if responses.dim() == 2 else responses.shape[1] * responses.shape[2]
    return batch["attention_mask"][:, -R:]


# ---------------------------------------------------------------------------------------------
# KL controllers
# ---------------------------------------------------------------------------------------------
class AdaptiveKLController:
    """beta <- beta * (1 + clip(kl/target - 1, +-0.2) * n_steps / horizon)  (arXiv 1909.08593)."""

    def __init__(self, init_kl_coef: float, target_kl: float, horizon: float):
        self.value = init_kl_coef
        self.target = target_kl
        self.horizon = horizon

    def update(self, current_kl: float, n_steps: int) -> None:
        err = float(np.clip(current_kl / self.target - 1, -0.2, 0.2))
        self.value *= 1 + err * n_steps / self.horizon


class FixedKLController:
    def __init__(self, kl_coef: float):
        self.value = kl_coef

    def update(self, current_kl: float, n_steps: int) -> None:
        pass


def get_kl_controller(kl_ctrl):
    if kl_ctrl.type == "fixed":
        return FixedKLController(kl_ctrl.kl_coef)
    if kl_ctrl.type == "adaptive":
        assert kl_ctrl.horizon > 0, f"horizon must be larger than 0. Got {kl_ctrl.horizon}"
        return AdaptiveKLController(kl_ctrl.kl_coef, kl_ctrl.target_kl, kl_ctrl.horizon)
    raise NotImplementedError(f"unknown KL controller type '{kl_ctrl.type}'")


# ---------------------------------------------------------------------------------------------
# advantage estimators
# ---------------------------------------------------------------------------------------------
@register_adv_est(AdvantageEstimator.GAE)
def compute_gae_advantage_return(token_level_rewards: torch.Tensor, values: torch.Tensor,
                                 response_mask: torch.Tensor, gamma: float = 1.0, lam: float = 1.0, **_):
    """Generalised advantage estimation with carry-through over masked tokens, then masked whitening.

    delta_t = r_t + gamma V_{t+1} - V_t ; A_t = delta_t + gamma lam A_{t+1}; at masked positions the
    running ``next value`` and ``last gae`` are carried unchanged.  returns = A + V (before whitening)."""
    with torch.no_grad():
        from ..ops import rl as _rl
        adv, ret = _rl.gae_scan(token_level_rewards.float(), values.float(), response_mask.float(), gamma, lam)
        adv = masked_whiten(adv, response_mask.float())
    return adv, ret


def _group_stats(scores: torch.Tensor, index) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per-sample group mean / unbiased std / count for groups given by ``index`` (any hashable ids)."""
    if isinstance(index, torch.Tensor):
        idx_t = index.to(scores.device)
        _, inv = torch.unique(idx_t, return_inverse=True)
    else:
        arr = np.asarray(index)
        _, inv_np = np.unique(arr.astype(str) if arr.dtype == object else arr, return_inverse=True)
        inv = torch.as_tensor(inv_np, device=scores.device, dtype=torch.long)
    G = int(inv.max().item()) + 1 if inv.numel() else 0
    ones = torch.ones_like(scores)
    cnt = torch.zeros(G, device=scores.device, dtype=scores.dtype).index_add_(0, inv, ones)
    s1 = torch.zeros(G, device=scores.device, dtype=scores.dtype).index_add_(0, inv, scores)
    mean = s1 / cnt.clamp(min=1)
    dev2 = torch.zeros(G, device=scores.device, dtype=scores.dtype).index_add_(0, inv, (scores - mean[inv]) ** 2)
    std = torch.sqrt(dev2 / (cnt - 1).clamp(min=1))
    single = cnt <= 1
    mean = torch.where(single, torch.zeros_like(mean), mean)
    std = torch.where(single, torch.ones_like(std), std)
    return mean[inv], std[inv], cnt[inv], inv


@register_adv_est(AdvantageEstimator.GRPO)
def compute_grpo_outcome_advantage(token_level_rewards: torch.Tensor, response_mask: torch.Tensor, index=None,
                                   epsilon: float = 1e-6, norm_adv_by_std_in_grpo: bool = True, **_):
    """Outcome-reward GRPO: s_i = sum_t r_it; A_i = (s_i - mean_g)/(std_g + eps) with the unbiased std of
    the prompt group; a group of one uses mean 0 / std 1.  ``norm_adv_by_std_in_grpo=False`` is Dr.GRPO."""
    with torch.no_grad():
        scores = token_level_rewards.float().sum(-1)
        mean, std, _, _ = _group_stats(scores, index)
        adv = (scores - mean) / (std + epsilon) if norm_adv_by_std_in_grpo else scores - mean
        adv = adv.unsqueeze(-1) * response_mask
    return adv, adv


@register_adv_est(AdvantageEstimator.CPGD)
def compute_cpgd_outcome_advantage(token_level_rewards: torch.Tensor, response_mask: torch.Tensor, index=None,
                                   epsilon: float = 1e-6, weight_factor_in_cpgd: str = "STD_weight", **_):
    """CPGD group baseline with three weightings: ``STD_weight`` (GRPO), ``clip_filter_like_weight``
    ((s - mean) * min(B / #groups-with-nonzero-std, 3)) and ``naive`` (s - mean)."""
    with torch.no_grad():
        scores = token_level_rewards.float().sum(-1)
        mean, std, cnt, inv = _group_stats(scores, index)
        if weight_factor_in_cpgd == "STD_weight":
            adv = (scores - mean) / (std + epsilon)
        elif weight_factor_in_cpgd == "clip_filter_like_weight":
            G = int(inv.max().item()) + 1
            gstd = torch.zeros(G, device=scores.device).scatter_(0, inv, std)
            nonzero = (gstd != 0).sum().clamp(min=1).float()
            adv = (scores - mean) * torch.clamp(scores.shape[0] / nonzero, max=3.0)
        elif weight_factor_in_cpgd == "naive":
            adv = scores - mean
        else:
            raise NotImplementedError(weight_factor_in_cpgd)
        adv = adv.unsqueeze(-1) * response_mask
    return adv, adv


def compute_marft_gae_advantage_return(batch, pre_agent_group_ids, gamma: float, lam: float) -> None:
    """Multi-agent (MARFT) GAE over interleaved agent turns (reference core_algos.py:351-458).

    For every trajectory (rows sharing ``request_id``; ``traj_len`` consecutive rows) the scan runs
    backwards over turns and, inside a turn, over agents in reverse order; the value that follows the
    last token of agent k is the first-token value of agent k+1 in the same turn, and for the last
    agent it is the first-token value of agent 0 in the neighbouring turn row.  Results are written to
    ``agent_group_{k}_advantages/returns`` and, for the last agent, ``advantages/returns``."""
    prefix = "agent_group_"
    ids = list(pre_agent_group_ids)
    dev_rewards = [batch[f"{prefix}{g}_token_level_rewards"] for g in ids] + [batch["token_level_rewards"]]
    dev_values = [batch[f"{prefix}{g}_values"] for g in ids] + [batch["values"]]
    dev_masks = [batch[f"{prefix}{g}_response_mask"] for g in ids] + [batch["response_mask"]]
    n_agents = len(dev_rewards)
    # the scan is sequential over (turn, agent, token): run it on host copies (one transfer per tensor instead of a
    # device synchronisation per token), then move the results back
    rewards = [r.detach().float().cpu() for r in dev_rewards]
    values = [v.detach().float().cpu() for v in dev_values]
    lens = [m.detach().float().cpu().sum(-1).long().tolist() for m in dev_masks]
    adv = [torch.zeros_like(v) for v in values]
    ret = [torch.zeros_like(v) for v in values]
    req = list(batch["request_id"])
    traj_len = list(batch["traj_len"])
    seen = set()
    starts = [i for i, s in enumerate(req) if s not in seen and not seen.add(s)]
    for b0 in starts:
        gae = 0.0
        for t_idx in range(int(traj_len[b0])):
            row = b0 + t_idx
            for a in reversed(range(n_agents)):
                L = int(lens[a][row])
                if L == 0:
                    continue
                v_row = values[a][row, :L].tolist()
                if a == n_agents - 1:
                    v_after = 0.0 if t_idx == 0 else float(values[0][row - 1, 0])
                else:
                    v_after = float(values[a + 1][row, 0])
                last_reward = float(rewards[a][row, L - 1])
                a_row = [0.0] * L
                for t in reversed(range(L)):
                    if t == L - 1:
                        delta = last_reward + gamma * v_after - v_row[t]
                    else:
                        delta = gamma * v_row[t + 1] - v_row[t]
                    gae = delta + gamma * lam * gae
                    a_row[t] = gae
                adv[a][row, :L] = torch.tensor(a_row)
                ret[a][row, :L] = adv[a][row, :L] + values[a][row, :L]
    for a in range(n_agents):
        dev = dev_values[a].device
        adv_a = masked_whiten(adv[a].to(dev), dev_masks[a].float())
        if a < n_agents - 1:
            batch[f"{prefix}{ids[a]}_advantages"] = adv_a
            batch[f"{prefix}{ids[a]}_returns"] = ret[a].to(dev)
        else:
            batch["advantages"] = adv_a
            batch["returns"] = ret[a].to(dev)


# ---------------------------------------------------------------------------------------------
# rewards / aggregation
# ---------------------------------------------------------------------------------------------
def compute_rewards(token_level_scores, old_log_prob, ref_log_prob, kl_ratio):
    return token_level_scores - (old_log_prob - ref_log_prob) * kl_ratio


def agg_loss(loss_mat: torch.Tensor, loss_mask: torch.Tensor, loss_agg_mode: str) -> torch.Tensor:
    """``token-mean`` | ``seq-mean-token-sum`` | ``seq-mean-token-mean`` | ``seq-mean-token-sum-norm``."""
    if loss_agg_mode == "token-mean":
        return masked_mean(loss_mat, loss_mask)
    if loss_agg_mode == "seq-mean-token-sum":
        return (loss_mat * loss_mask).sum(-1).mean()
    if loss_agg_mode == "seq-mean-token-mean":
        return ((loss_mat * loss_mask).sum(-1) / (loss_mask.sum(-1) + 1e-8)).mean()
    if loss_agg_mode == "seq-mean-token-sum-norm":
        return (loss_mat * loss_mask).sum() / loss_mask.shape[-1]
    raise ValueError(f"Invalid loss_agg_mode: {loss_agg_mode}")


def _clip_cfg(config):
    eps = config.clip_ratio
    lo = config.clip_ratio_low if config.clip_ratio_low is not None else eps
    hi = config.clip_ratio_high if config.clip_ratio_high is not None else eps
    return eps, lo, hi


_ZERO = lambda ref: torch.zeros((), device=ref.device)  # noqa: E731


# ---------------------------------------------------------------------------------------------
# policy losses
# ---------------------------------------------------------------------------------------------
@register_policy_loss("vanilla")
def compute_policy_loss_vanilla(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                                config=None, rollout_is_weights=None):
    """PPO clipped surrogate with dual-clip (arXiv 1912.09729): ratio from a log-ratio clamped to +-20,
    ``max(-A r, -A clip(r))``, and for A<0 additionally ``min(., -A c)`` with c = ``clip_ratio_c`` (3)."""
    _, lo, hi = _clip_cfg(config)
    c = getattr(config, "clip_ratio_c", 3.0)
    assert c > 1.0, f"clip_ratio_c must be > 1.0, got {c}"
    neg_kl = torch.clamp(log_prob - old_log_prob, min=-20.0, max=20.0)
    ratio = torch.exp(neg_kl)
    ppo_kl = masked_mean(-neg_kl, response_mask)
    l1 = -advantages * ratio
    l2 = -advantages * torch.clamp(ratio, 1 - lo, 1 + hi)
    clip1 = torch.maximum(l1, l2)
    pg_clipfrac = masked_mean(torch.gt(l2, l1).float(), response_mask)
    l3 = -advantages * c
    clip2 = torch.min(l3, clip1)
    pg_clipfrac_lower = masked_mean((torch.gt(clip1, l3) * (advantages < 0)).float(), response_mask)
    pg_losses = torch.where(advantages < 0, clip2, clip1)
    if rollout_is_weights is not None:
        pg_losses = pg_losses * rollout_is_weights
    return agg_loss(pg_losses, response_mask, loss_agg_mode), pg_clipfrac, ppo_kl, pg_clipfrac_lower


@register_policy_loss("gspo")
def compute_policy_loss_gspo(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="seq-mean-token-mean",
                             config=None, rollout_is_weights=None):
    """GSPO (arXiv 2507.18071): sequence-level ratio s_i = exp(mean_t(logp - old)); the token ratio is
    ``exp(logp - sg(logp) + sg(log s_i))`` with its log clamped at 10; clipped surrogate without dual
    clip; aggregation is always ``seq-mean-token-mean``."""
    _, lo, hi = _clip_cfg(config)
    neg_kl = log_prob - old_log_prob
    seq_len = response_mask.sum(-1).clamp(min=1)
    log_seq_ratio = (neg_kl * response_mask).sum(-1) / seq_len
    log_tok = log_prob - log_prob.detach() + log_seq_ratio.detach().unsqueeze(-1)
    log_tok = torch.clamp(log_tok, max=10.0)
    ratio = torch.exp(log_tok)
    l1 = -advantages * ratio
    l2 = -advantages * torch.clamp(ratio, 1 - lo, 1 + hi)
    pg_losses = torch.maximum(l1, l2)
    if rollout_is_weights is not None:
        pg_losses = pg_losses * rollout_is_weights
    pg_loss = agg_loss(pg_losses, response_mask, "seq-mean-token-mean")
    pg_clipfrac = masked_mean(torch.gt(l2, l1).float(), response_mask)
    ppo_kl = masked_mean(-neg_kl, response_mask)
    return pg_loss, pg_clipfrac, ppo_kl, _ZERO(pg_loss)


@register_policy_loss("cpgd")
def compute_policy_loss_cpgd(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                             config=None, rollout_is_weights=None):
    """CPGD: clip the *log-probability* instead of the ratio — for A>0 ``min(logp, old + log(1+eps_hi))``,
    else ``max(logp, old + log(1-eps_lo))`` — and use ``-clipped * A``."""
    _, lo, hi = _clip_cfg(config)
    neg_kl = log_prob - old_log_prob
    ppo_kl = masked_mean(-neg_kl, response_mask)
    up = old_log_prob + float(np.log(1 + hi))
    dn = old_log_prob + float(np.log(1 - lo))
    clipped = torch.where(advantages > 0, torch.minimum(log_prob, up), torch.maximum(log_prob, dn))
    pg_losses = -clipped * advantages
    is_clipped = torch.where(advantages > 0, log_prob > up, log_prob < dn)
    pg_clipfrac = masked_mean((is_clipped & (advantages > 0)).float(), response_mask)
    pg_clipfrac_lower = masked_mean((is_clipped & (advantages <= 0)).float(), response_mask)
    if rollout_is_weights is not None:
        pg_losses = pg_losses * rollout_is_weights
    return agg_loss(pg_losses, response_mask, loss_agg_mode), pg_clipfrac, ppo_kl, pg_clipfrac_lower


def cpgd_policy_drift(old_log_prob, log_prob, response_mask, loss_agg_mode: str) -> torch.Tensor:
    """CPGD drift regulariser ``clamp(exp(sg(logp) - old) - 1, max=2) * logp`` aggregated like the loss
    (reference: siirl/engine/actor/dp_actor.py:488-494)."""
    w = (torch.exp(log_prob.detach() - old_log_prob) - 1).clamp(max=2.0)
    return agg_loss(w * log_prob, response_mask, loss_agg_mode)


@register_policy_loss("gpg")
def compute_policy_loss_gpg(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                            config=None, rollout_is_weights=None):
    pg_losses = -log_prob * advantages
    if rollout_is_weights is not None:
        pg_losses = pg_losses * rollout_is_weights
    loss = agg_loss(pg_losses, response_mask, loss_agg_mode)
    return loss, _ZERO(loss), _ZERO(loss), _ZERO(loss)


@register_policy_loss("clip_cov")
def compute_policy_loss_clip_cov(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                                 config=None, rollout_is_weights=None):
    """Clip-Cov (arXiv 2505.22617): besides PPO clipping, a random subset (``clip_cov_ratio`` of the valid
    tokens) of tokens whose (advantage, log-prob) covariance lies in (lb, ub) has its gradient dropped."""
    _, lo, hi = _clip_cfg(config)
    pl = config.policy_loss
    ratio_cfg, lb, ub = pl.clip_cov_ratio, pl.clip_cov_lb, pl.clip_cov_ub
    assert ratio_cfg > 0
    neg_kl = log_prob - old_log_prob
    ratio = torch.exp(neg_kl)
    ppo_kl = masked_mean(-neg_kl, response_mask)
    l1 = -advantages * ratio
    l2 = -advantages * torch.clamp(ratio, 1 - lo, 1 + hi)
    valid = response_mask > 0
    clip_by_origin = (l2 > l1) & valid
    cov = (advantages - masked_mean(advantages, response_mask)) * (
        log_prob - masked_mean(log_prob.detach(), response_mask))
    cov = cov.detach().masked_fill(~valid | clip_by_origin, float("-inf"))
    clip_num = max(int(ratio_cfg * response_mask.sum().item()), 1)
    cand = torch.nonzero((cov < ub) & (cov > lb) & valid)
    corr = torch.ones_like(advantages)
    if len(cand) > 0:
        perm = torch.randperm(len(cand), device=cand.device)
        pick = cand[perm[: min(clip_num, len(cand))]]
        corr[pick[:, 0], pick[:, 1]] = 0
    pg_clipfrac = masked_mean((corr == 0).float(), response_mask)
    pg_losses = torch.maximum(l1, l2) * corr
    if rollout_is_weights is not None:
        pg_losses = pg_losses * rollout_is_weights
    loss = agg_loss(pg_losses, response_mask, loss_agg_mode)
    return loss, pg_clipfrac, ppo_kl, _ZERO(loss)


@register_policy_loss("kl_cov")
def compute_policy_loss_kl_cov(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                               config=None, rollout_is_weights=None):
    """KL-Cov: the top ``kl_cov_ratio`` fraction of valid tokens by covariance gets an extra
    ``ppo_kl_coef * |logp - old|`` penalty; the rest use the unclipped surrogate."""
    pl = config.policy_loss
    kl_cov_ratio, coef = pl.kl_cov_ratio, pl.ppo_kl_coef
    assert kl_cov_ratio > 0
    neg_kl = log_prob - old_log_prob
    abs_kl = neg_kl.abs()
    ratio = torch.exp(neg_kl)
    ppo_kl_abs = masked_mean(abs_kl, response_mask)
    base = -advantages * ratio
    with_kl = base + coef * abs_kl
    valid = response_mask > 0
    n_valid = int(valid.sum().item())
    select = torch.zeros_like(valid)
    if n_valid > 0:
        a = advantages[valid].detach()
        lp = log_prob[valid].detach()
        cov = (a - a.mean()) * (lp - lp.mean())
        k = max(1, int(n_valid * kl_cov_ratio))
        top = torch.topk(cov, k, largest=True).indices
        flat_idx = torch.nonzero(valid.reshape(-1), as_tuple=True)[0][top]
        select.view(-1)[flat_idx] = True
    pg_losses = torch.where(select, with_kl, base)
    if rollout_is_weights is not None:
        pg_losses = pg_losses * rollout_is_weights
    loss = agg_loss(pg_losses, response_mask, loss_agg_mode)
    return loss, _ZERO(loss), ppo_kl_abs, _ZERO(loss)


@register_policy_loss("geo_mean")
def compute_policy_loss_geo_mean(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean",
                                 config=None, rollout_is_weights=None):
    """GMPO (arXiv 2507.20673): clip token log-ratios to [-eps_lo, eps_hi] on the side chosen by the sign
    of the advantage, then use the geometric mean of the token ratios as the sequence ratio."""
    _, lo, hi = _clip_cfg(config)
    neg_kl = log_prob - old_log_prob
    ppo_kl = masked_mean(-neg_kl, response_mask)
    sgn = torch.sign(advantages)
    clamp = torch.clamp(neg_kl, -lo, hi)
    chosen = sgn * torch.min(sgn * neg_kl, sgn * clamp)
    n = response_mask.sum(-1)
    ratio = torch.exp((chosen * response_mask).sum(-1) / (n + 1e-8))
    adv_seq = (advantages * response_mask).sum(-1) / (n + 1e-8)
    pg_losses = -adv_seq * ratio
    if rollout_is_weights is not None:
        w = torch.exp((torch.log(rollout_is_weights + 1e-10) * response_mask).sum(-1) / (n + 1e-8))
        pg_losses = pg_losses * w
    clipped = torch.ne(neg_kl, clamp)
    pg_clipfrac = masked_mean((clipped * (advantages > 0)).float(), response_mask)
    pg_clipfrac_lower = masked_mean((clipped * (advantages < 0)).float(), response_mask)
    return pg_losses.mean(), pg_clipfrac, ppo_kl, pg_clipfrac_lower


def compute_entropy_loss(entropy: torch.Tensor, response_mask: torch.Tensor, loss_agg_mode: str = "token-mean"):
    return agg_loss(entropy, response_mask, loss_agg_mode)


def compute_value_loss(vpreds, returns, values, response_mask, cliprange_value: float,
                       loss_agg_mode: str = "token-mean"):
    """Clipped value loss ``0.5 * agg(max((v-R)^2, (clip(v, v_old +- eps)-R)^2))`` and its clip fraction."""
    vclip = torch.clamp(vpreds, values - cliprange_value, values + cliprange_value)
    l1 = (vpreds - returns) ** 2
    l2 = (vclip - returns) ** 2
    vf_loss = 0.5 * agg_loss(torch.max(l1, l2), response_mask, loss_agg_mode)
    vf_clipfrac = masked_mean(torch.gt(l2, l1).float(), response_mask)
    return vf_loss, vf_clipfrac


def kl_penalty(logprob: torch.Tensor, ref_logprob: torch.Tensor, kl_penalty: str) -> torch.Tensor:
    """Token-wise KL estimators: ``kl|k1``, ``abs``, ``mse|k2``, ``low_var_kl|k3`` (clamped to +-10 with the
    log-ratio clamped to +-20); a ``+`` suffix keeps the value but routes the gradient of k2
    (straight-through), as in the reference (core_algos.py:1215-1276)."""
    straight = kl_penalty.endswith("+")
    kind = kl_penalty.rstrip("+")
    fwd = _kl_penalty_forward(logprob, ref_logprob, kind)
    if not straight or kind in ("mse", "k2"):
        return fwd
    bwd = _kl_penalty_forward(logprob, ref_logprob, "k2")
    return bwd - bwd.detach() + fwd.detach()


def _kl_penalty_forward(logprob, ref_logprob, kind: str) -> torch.Tensor:
    if kind in ("kl", "k1"):
        return logprob - ref_logprob
    if kind == "abs":
        return (logprob - ref_logprob).abs()
    if kind in ("mse", "k2"):
        return 0.5 * (logprob - ref_logprob).square()
    if kind in ("low_var_kl", "k3"):
        k = torch.clamp(ref_logprob - logprob, min=-20, max=20)
        return torch.clamp(torch.exp(k) - k - 1, min=-10, max=10)
    if kind == "full":
        raise NotImplementedError("'full' KL needs the full distributions")
    raise NotImplementedError(f"unknown kl penalty '{kind}'")


def compute_pf_ppo_reweight_data(batch, reweight_method: str = "pow", weight_pow: float = 2.0,
                                 generator: Optional[torch.Generator] = None):
    """Preference-feedback PPO: resample the batch (with replacement) with weights derived from the
    sequence scores: ``pow`` |s|^p, ``max_min`` (only extreme scores), ``max_random`` (0.4 for max, 0.1 else)."""
    scores = batch["token_level_scores"].sum(-1).float()
    if reweight_method == "pow":
        w = scores.abs().pow(weight_pow)
    elif reweight_method == "max_min":
        w = ((scores == scores.max()) | (scores == scores.min())).float()
    elif reweight_method == "max_random":
        w = torch.where(scores == scores.max(), 0.4, 0.1)
    else:
        raise ValueError(f"Unsupported reweight_method: {reweight_method}")
    w = torch.clamp(w + 1e-8, min=1e-8)
    idx = torch.multinomial(w.cpu(), scores.shape[0], replacement=True, generator=generator)
    return batch.select_idxs(idx)


def apply_kl_penalty(batch, kl_ctrl, kl_penalty_kind: str = "kl"):
    """token_level_rewards = scores - beta * KL(old || ref) * mask; updates the controller with the
    batch-mean of per-sequence mean KL.  Returns (batch, metrics)."""
    mask = batch["response_mask"].float()
    scores = batch["token_level_scores"]
    kld = kl_penalty(batch["old_log_probs"], batch["ref_log_prob"], kl_penalty_kind) * mask
    beta = kl_ctrl.value
    batch["token_level_rewards"] = scores - beta * kld
    current_kl = masked_mean(kld, mask, dim=-1).mean().item()
    kl_ctrl.update(current_kl=current_kl, n_steps=scores.shape[0])
    return batch, {"actor/reward_kl_penalty": current_kl, "actor/reward_kl_penalty_coeff": beta}


def compute_advantage(batch, adv_estimator, gamma: float = 1.0, lam: float = 1.0,
                      norm_adv_by_std_in_grpo: bool = True, weight_factor_in_cpgd: str = "STD_weight", **kwargs):
    """Dispatcher used by the ``calculate_advantages`` node (reference core_algos.py:1400-1492)."""
    if "response_mask" not in batch:
        batch["response_mask"] = compute_response_mask(batch)
    key = adv_estimator.value if hasattr(adv_estimator, "value") else adv_estimator
    mask = batch["response_mask"]
    if kwargs.get("multi_turn", False) and "loss_mask" in batch:
        R = batch["responses"].shape[1]
        mask = batch["loss_mask"][:, -R:]
    if key == "gae":
        adv, ret = compute_gae_advantage_return(batch["token_level_rewards"], batch["values"], mask, gamma, lam)
        batch["advantages"], batch["returns"] = adv, ret
        if kwargs.get("use_pf_ppo", False):
            batch = compute_pf_ppo_reweight_data(batch, kwargs.get("pf_ppo_reweight_method", "pow"),
                                                 kwargs.get("pf_ppo_weight_pow", 2.0))
    elif key == "grpo":
        responses = batch["responses"]
        if "finish_step" in batch and responses.dim() == 3:
            B, traj, act = responses.shape
            steps = torch.arange(traj * act, device=responses.device)[None, :]
            mask = (steps < (batch["finish_step"].to(responses.device) * act)[:, None]).to(torch.float32)
            batch["response_mask"] = mask
        adv, ret = compute_grpo_outcome_advantage(batch["token_level_rewards"], mask, batch["uid"],
                                                  norm_adv_by_std_in_grpo=norm_adv_by_std_in_grpo)
        batch["advantages"], batch["returns"] = adv, ret
    elif key == "cpgd":
        adv, ret = compute_cpgd_outcome_advantage(batch["token_level_rewards"], mask, batch["uid"],
                                                  weight_factor_in_cpgd=weight_factor_in_cpgd)
        batch["advantages"], batch["returns"] = adv, ret
    elif key == "gae_marft":
        compute_marft_gae_advantage_return(batch, kwargs["agent_group_ids"], gamma, lam)
    else:
        fn = get_adv_estimator_fn(key)
        adv, ret = fn(token_level_rewards=batch["token_level_rewards"], response_mask=mask,
                      index=batch.get("uid"), values=batch.get("values"), gamma=gamma, lam=lam, **kwargs)
        batch["advantages"], batch["returns"] = adv, ret
    return batch


__all__ = [n for n in dir() if not n.startswith("_")]
