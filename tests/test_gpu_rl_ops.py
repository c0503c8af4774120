"""RL post-processing kernels against the PyTorch statements of the same formulas."""
import types

import pytest
import torch

from siirl_b200.dag_worker import core_algos as A
from siirl_b200.ops import rl

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _mask(B, R):
    lens = torch.randint(1, R + 1, (B,))
    m = (torch.arange(R)[None, :] < lens[:, None]).float()
    m[0, 3:7] = 0  # a hole inside a response (multi-turn style)
    return m


def test_gae_scan_matches_loop():
    torch.manual_seed(0)
    B, R = 37, 301
    r, v, m = torch.randn(B, R), torch.randn(B, R), _mask(B, R)
    adv_ref, ret_ref = rl.gae_scan_reference(r, v, m, 0.99, 0.95)
    adv, ret = rl.gae_scan(r.to(DEV), v.to(DEV), m.to(DEV), 0.99, 0.95)
    torch.testing.assert_close(adv.cpu(), adv_ref, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(ret.cpu(), ret_ref, rtol=1e-4, atol=1e-4)


def test_grpo_group_adv_matches_formula():
    torch.manual_seed(1)
    B, R, G = 48, 64, 13
    rewards = torch.zeros(B, R)
    m = _mask(B, R)
    rewards[torch.arange(B), (m.sum(-1) - 1).long().clamp(min=0)] = torch.rand(B)
    gid = torch.randint(0, G, (B,))
    gid[0] = G - 1
    gid[1:][gid[1:] == G - 1] = 0  # make one singleton group
    want, _ = A.compute_grpo_outcome_advantage(rewards, m, gid)
    got = rl.grpo_group_advantage(rewards.to(DEV), m.to(DEV), gid.to(DEV), G)
    torch.testing.assert_close(got.cpu(), want, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("mode", ["vanilla", "gspo", "cpgd"])
@pytest.mark.parametrize("agg", ["token-mean", "seq-mean-token-sum", "seq-mean-token-mean", "seq-mean-token-sum-norm"])
def test_fused_ppo_loss_matches_torch(mode, agg):
    torch.manual_seed(2)
    B, R = 16, 50
    m = _mask(B, R).to(DEV)
    old = (-torch.rand(B, R) * 3).to(DEV)
    logp = (old + 0.3 * torch.randn(B, R, device=DEV)).requires_grad_()
    ref_lp = old + 0.2 * torch.randn(B, R, device=DEV)
    adv = torch.randn(B, R, device=DEV)
    ent = torch.rand(B, R, device=DEV).requires_grad_()
    cfg = types.SimpleNamespace(clip_ratio=0.2, clip_ratio_low=0.2, clip_ratio_high=0.28, clip_ratio_c=3.0)
    loss, met = rl.ppo_token_loss(logp, old, adv, m, entropy=ent, ref_logp=ref_lp, mode=mode, loss_agg_mode=agg,
                                  clip_lo=0.2, clip_hi=0.28, clip_c=3.0, kl_kind="low_var_kl", kl_coef=0.01,
                                  entropy_coef=0.001)
    loss.backward()
    lp2 = logp.detach().clone().requires_grad_()
    ent2 = ent.detach().clone().requires_grad_()
    fn = A.get_policy_loss_fn(mode)
    pg, clipfrac, ppo_kl, clip_lower = fn(old, lp2, adv, m, agg, cfg)
    agg_eff = "seq-mean-token-mean" if mode == "gspo" else agg
    kl = A.agg_loss(A.kl_penalty(lp2, ref_lp, "low_var_kl"), m, agg_eff)
    el = A.agg_loss(ent2, m, agg_eff)
    total = pg + 0.01 * kl - 0.001 * el
    total.backward()
    torch.testing.assert_close(loss.detach(), total.detach(), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(met["pg_loss"], pg.detach(), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(met["pg_clipfrac"], clipfrac.detach(), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(met["ppo_kl"], ppo_kl.detach(), rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(logp.grad, lp2.grad, rtol=1e-3, atol=1e-6)
    torch.testing.assert_close(ent.grad, ent2.grad, rtol=1e-4, atol=1e-7)
