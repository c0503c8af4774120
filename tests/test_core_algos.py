"""Golden tests of the algorithm layer against direct statements of the formulas."""
import math
import types

import numpy as np
import pytest
import torch

from siirl_b200.dag_worker import core_algos as A
from siirl_b200.data_coordinator import Batch


def _mask(B, R, seed=0):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(1, R + 1, (B,), generator=g)
    return (torch.arange(R)[None, :] < lens[:, None]).float()


def _cfg(**kw):
    base = dict(clip_ratio=0.2, clip_ratio_low=0.2, clip_ratio_high=0.28, clip_ratio_c=3.0,
                policy_loss=types.SimpleNamespace(clip_cov_ratio=0.2, clip_cov_lb=-5.0, clip_cov_ub=5.0,
                                                  kl_cov_ratio=0.1, ppo_kl_coef=0.1))
    base.update(kw)
    return types.SimpleNamespace(**base)


def test_agg_loss_modes():
    x = torch.tensor([[1., 2., 3.], [4., 5., 6.]])
    m = torch.tensor([[1., 1., 0.], [1., 0., 0.]])
    assert A.agg_loss(x, m, "token-mean").item() == pytest.approx(7 / 3, rel=1e-5)
    assert A.agg_loss(x, m, "seq-mean-token-sum").item() == pytest.approx((3 + 4) / 2)
    assert A.agg_loss(x, m, "seq-mean-token-mean").item() == pytest.approx((1.5 + 4) / 2, rel=1e-5)
    assert A.agg_loss(x, m, "seq-mean-token-sum-norm").item() == pytest.approx(7 / 3)
    with pytest.raises(ValueError):
        A.agg_loss(x, m, "nope")


def test_grpo_matches_per_group_formula():
    torch.manual_seed(0)
    B, R = 12, 7
    m = _mask(B, R)
    r = torch.zeros(B, R)
    r[torch.arange(B), (m.sum(-1) - 1).long()] = torch.rand(B)
    uid = np.array(["a", "a", "a", "b", "b", "c", "d", "d", "d", "d", "e", "e"], dtype=object)
    adv, ret = A.compute_grpo_outcome_advantage(r, m, uid)
    s = r.sum(-1)
    for g in set(uid):
        idx = [i for i in range(B) if uid[i] == g]
        if len(idx) == 1:
            mu, sd = 0.0, 1.0
        else:
            mu, sd = s[idx].mean(), s[idx].std()
        for i in idx:
            want = (s[i] - mu) / (sd + 1e-6)
            torch.testing.assert_close(adv[i], want * m[i], rtol=1e-5, atol=1e-6)
    assert torch.equal(adv, ret)
    adv2, _ = A.compute_grpo_outcome_advantage(r, m, uid, norm_adv_by_std_in_grpo=False)
    i = 0
    torch.testing.assert_close(adv2[i], (s[i] - s[[0, 1, 2]].mean()) * m[i])
    # integer tensor ids give the same answer
    ids = torch.tensor([0, 0, 0, 1, 1, 2, 3, 3, 3, 3, 4, 4])
    adv3, _ = A.compute_grpo_outcome_advantage(r, m, ids)
    torch.testing.assert_close(adv3, adv)


def test_gae_matches_reference_loop_and_whitening():
    torch.manual_seed(1)
    B, R = 5, 9
    m = _mask(B, R, 1)
    m[0, 2] = 0  # hole
    r, v = torch.randn(B, R), torch.randn(B, R)
    gamma, lam = 0.97, 0.9
    adv, ret = A.compute_gae_advantage_return(r, v, m, gamma, lam)
    nextv = torch.zeros(B); last = torch.zeros(B); outs = []
    for t in reversed(range(R)):
        delta = r[:, t] + gamma * nextv - v[:, t]
        l_ = delta + gamma * lam * last
        nextv = v[:, t] * m[:, t] + (1 - m[:, t]) * nextv
        last = l_ * m[:, t] + (1 - m[:, t]) * last
        outs.append(last)
    raw = torch.stack(outs[::-1], 1)
    torch.testing.assert_close(ret, raw + v, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(adv, A.masked_whiten(raw, m), rtol=1e-4, atol=1e-5)
    assert abs(A.masked_mean(adv, m).item()) < 1e-5


def test_cpgd_weightings():
    r = torch.zeros(4, 3); r[:, -1] = torch.tensor([1., 0., 1., 1.])
    m = torch.ones(4, 3)
    uid = torch.tensor([0, 0, 1, 1])
    a_std, _ = A.compute_cpgd_outcome_advantage(r, m, uid, weight_factor_in_cpgd="STD_weight")
    a_grpo, _ = A.compute_grpo_outcome_advantage(r, m, uid)
    torch.testing.assert_close(a_std, a_grpo)
    a_naive, _ = A.compute_cpgd_outcome_advantage(r, m, uid, weight_factor_in_cpgd="naive")
    torch.testing.assert_close(a_naive[:, 0], torch.tensor([0.5, -0.5, 0., 0.]))
    a_clip, _ = A.compute_cpgd_outcome_advantage(r, m, uid, weight_factor_in_cpgd="clip_filter_like_weight")
    torch.testing.assert_close(a_clip[:, 0], torch.tensor([0.5, -0.5, 0., 0.]) * 3.0)  # 4 / 1 non-zero-std group -> clamp 3


def test_vanilla_loss_clipping_and_dual_clip():
    old = torch.zeros(1, 4)
    logp = torch.log(torch.tensor([[1.5, 0.5, 5.0, 1.0]]))
    adv = torch.tensor([[1.0, 1.0, -1.0, -1.0]])
    m = torch.ones(1, 4)
    loss, clipfrac, kl, clip_lower = A.compute_policy_loss_vanilla(old, logp, adv, m, "token-mean", _cfg())
    # token0: A>0 ratio 1.5 -> clipped to 1.28 ; token1: ratio .5 -> unclipped (max(-0.5, -0.8) = -0.5)
    # token2: A<0 ratio 5 -> max(5, 1.28)=5 -> dual clip min(3, 5) = 3 ; token3: ratio 1 -> 1
    want = (-1.28 - 0.5 + 3.0 + 1.0) / 4
    assert loss.item() == pytest.approx(want, rel=1e-5)
    assert clipfrac.item() == pytest.approx(1 / 4) and clip_lower.item() == pytest.approx(1 / 4)
    assert kl.item() == pytest.approx(-logp.mean().item(), rel=1e-5)


def test_gspo_sequence_ratio():
    torch.manual_seed(2)
    B, R = 3, 5
    m = _mask(B, R, 2)
    old = -torch.rand(B, R)
    logp = (old + 0.05 * torch.randn(B, R)).requires_grad_()
    adv = torch.randn(B, 1).expand(B, R)
    loss, clipfrac, kl, _ = A.compute_policy_loss_gspo(old, logp, adv, m, "token-mean", _cfg(clip_ratio_low=3e-4,
                                                                                            clip_ratio_high=4e-4))
    s = torch.exp(((logp - old) * m).sum(-1) / m.sum(-1)).detach()
    l1 = -adv * s[:, None]
    l2 = -adv * s[:, None].clamp(1 - 3e-4, 1 + 4e-4)
    want = ((torch.maximum(l1, l2) * m).sum(-1) / m.sum(-1)).mean()
    assert loss.item() == pytest.approx(want.item(), rel=1e-5)
    loss.backward()
    assert torch.isfinite(logp.grad).all() and logp.grad.abs().sum() > 0


def test_cpgd_and_gpg_losses():
    old = torch.zeros(1, 2)
    logp = torch.tensor([[0.5, -0.5]])
    adv = torch.tensor([[1.0, -1.0]])
    m = torch.ones(1, 2)
    loss, cf, kl, cfl = A.compute_policy_loss_cpgd(old, logp, adv, m, "token-mean", _cfg())
    want = (-(math.log(1.28)) * 1.0 + -(math.log(0.8)) * -1.0) / 2
    assert loss.item() == pytest.approx(want, rel=1e-5)
    assert cf.item() == 0.5 and cfl.item() == 0.5
    g, *_ = A.compute_policy_loss_gpg(old, logp, adv, m)
    assert g.item() == pytest.approx((-0.5 * 1 + -(-0.5) * -1) / 2)


def test_cov_and_geo_losses_run_and_are_finite():
    torch.manual_seed(3)
    B, R = 4, 16
    m = _mask(B, R, 3)
    old = -torch.rand(B, R)
    for fn in (A.compute_policy_loss_clip_cov, A.compute_policy_loss_kl_cov, A.compute_policy_loss_geo_mean):
        logp = (old + 0.1 * torch.randn(B, R)).requires_grad_()
        out = fn(old, logp, torch.randn(B, R), m, "token-mean", _cfg())
        assert len(out) == 4 and torch.isfinite(out[0])
        out[0].backward()
        assert torch.isfinite(logp.grad).all()


def test_kl_penalties_and_controllers():
    lp, ref = torch.tensor([0.0, -1.0]), torch.tensor([-0.5, -0.2])
    torch.testing.assert_close(A.kl_penalty(lp, ref, "kl"), lp - ref)
    torch.testing.assert_close(A.kl_penalty(lp, ref, "abs"), (lp - ref).abs())
    torch.testing.assert_close(A.kl_penalty(lp, ref, "mse"), 0.5 * (lp - ref) ** 2)
    k = ref - lp
    torch.testing.assert_close(A.kl_penalty(lp, ref, "low_var_kl"), torch.exp(k) - k - 1)
    x = lp.clone().requires_grad_()
    A.kl_penalty(x, ref, "low_var_kl+").sum().backward()
    torch.testing.assert_close(x.grad, lp - ref)          # straight-through k2 gradient
    ctl = A.AdaptiveKLController(0.1, target_kl=0.1, horizon=100)
    ctl.update(0.3, 10)
    assert ctl.value == pytest.approx(0.1 * (1 + 0.2 * 10 / 100))
    assert isinstance(A.get_kl_controller(types.SimpleNamespace(type="fixed", kl_coef=0.3)), A.FixedKLController)


def test_value_loss_and_apply_kl_penalty():
    v = torch.tensor([[1.0, 3.0]]); old = torch.tensor([[0.0, 0.0]]); ret = torch.tensor([[0.0, 0.0]])
    m = torch.ones(1, 2)
    loss, frac = A.compute_value_loss(v, ret, old, m, 0.5)
    assert loss.item() == pytest.approx(0.5 * (1.0 + 9.0) / 2) and frac.item() == 0.0
    b = Batch({"token_level_scores": torch.ones(2, 3), "old_log_probs": torch.zeros(2, 3),
               "ref_log_prob": -torch.ones(2, 3), "response_mask": torch.ones(2, 3)})
    b, met = A.apply_kl_penalty(b, A.FixedKLController(0.1), "kl")
    torch.testing.assert_close(b["token_level_rewards"], torch.full((2, 3), 0.9))
    assert met["actor/reward_kl_penalty"] == pytest.approx(1.0)


def test_dispatcher_and_registry():
    b = Batch({"token_level_rewards": torch.rand(4, 5), "response_mask": torch.ones(4, 5),
               "responses": torch.zeros(4, 5, dtype=torch.long), "uid": torch.tensor([0, 0, 1, 1]),
               "values": torch.zeros(4, 5)})
    assert "advantages" in A.compute_advantage(b, "grpo")
    assert "returns" in A.compute_advantage(b, "gae", gamma=1.0, lam=1.0)

    @A.register_adv_est("my_est")
    def my(token_level_rewards, response_mask, **kw):
        return token_level_rewards * 0 + 1, token_level_rewards

    out = A.compute_advantage(b, "my_est")
    assert out["advantages"].eq(1).all()
    with pytest.raises(ValueError):
        A.get_policy_loss_fn("zzz")

    @A.register_policy_loss("my_loss")
    def ml(old_log_prob, log_prob, advantages, response_mask, loss_agg_mode="token-mean", config=None,
           rollout_is_weights=None):
        return log_prob.sum(), None, None, None
    assert A.get_policy_loss_fn("my_loss") is ml


def test_embodied_grpo_mask_from_finish_step():
    b = Batch({"token_level_rewards": torch.rand(2, 6), "response_mask": torch.ones(2, 6),
               "responses": torch.zeros(2, 3, 2, dtype=torch.long), "uid": torch.tensor([0, 0]),
               "finish_step": torch.tensor([1, 3])})
    out = A.compute_advantage(b, "grpo")
    assert out["response_mask"].tolist() == [[1, 1, 0, 0, 0, 0], [1, 1, 1, 1, 1, 1]]


def test_pf_ppo_and_marft():
    b = Batch({"token_level_scores": torch.tensor([[0., 1.], [0., 0.], [2., 0.]]), "x": torch.arange(3)})
    out = A.compute_pf_ppo_reweight_data(b, "max_min", generator=torch.Generator().manual_seed(0))
    assert set(out["x"].tolist()) <= {1, 2}
    # two agents, one trajectory of two turns
    mk = lambda: torch.ones(2, 2)
    bb = Batch({"agent_group_0_token_level_rewards": torch.zeros(2, 2), "agent_group_0_values": torch.zeros(2, 2),
                "agent_group_0_response_mask": mk(), "token_level_rewards": torch.tensor([[0., 1.], [0., 1.]]),
                "values": torch.zeros(2, 2), "response_mask": mk()},
               {"request_id": ["r", "r"], "traj_len": [2, 2]})
    A.compute_marft_gae_advantage_return(bb, [0], 1.0, 1.0)
    assert "agent_group_0_advantages" in bb and bb["returns"].shape == (2, 2)
