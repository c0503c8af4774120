"""tcgen05 varlen attention forward/backward against an eager fp32 statement."""
import math

import pytest
import torch

from siirl_b200.ops import lib, reference as ref
from siirl_b200.ops.attention import SeqInfo, attention_packed

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _ref(qkv, seqlens, hq, hkv, d, causal):
    T = qkv.shape[0]
    x = qkv.detach().float().requires_grad_()
    q, k, v = x.split([hq * d, hkv * d, hkv * d], dim=-1)
    out = ref.attention_varlen(q.reshape(T, hq, d), k.reshape(T, hkv, d), v.reshape(T, hkv, d),
                               torch.tensor([0] + list(torch.tensor(seqlens).cumsum(0))), causal=causal,
                               scale=1.0 / math.sqrt(d))
    return x, out.reshape(T, hq * d)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("cfg", [
    (128, 4, 2, [128]),
    (128, 4, 2, [64, 200, 37, 300]),
    (64, 4, 4, [100, 129, 256]),
    (128, 7, 1, [513, 90]),
    (32, 4, 2, [40, 77]),
])
def test_attention_fwd_bwd(cfg, causal):
    d, hq, hkv, seqlens = cfg
    torch.manual_seed(0)
    T = sum(seqlens)
    qkv = (0.5 * torch.randn(T, (hq + 2 * hkv) * d, device=DEV)).to(torch.bfloat16).requires_grad_()
    info = SeqInfo(seqlens, device=DEV)
    out = attention_packed(qkv, info, hq, hkv, d, causal=causal)
    lib.check_status()
    xr, outr = _ref(qkv, seqlens, hq, hkv, d, causal)
    assert _rel(out, outr) < 2e-2
    g = torch.randn_like(out)
    out.backward(g)
    lib.check_status()
    outr.backward(g.float())
    hq_w, hk_w = hq * d, hkv * d
    assert _rel(qkv.grad[:, :hq_w], xr.grad[:, :hq_w]) < 3e-2
    assert _rel(qkv.grad[:, hq_w:hq_w + hk_w], xr.grad[:, hq_w:hq_w + hk_w]) < 3e-2
    assert _rel(qkv.grad[:, hq_w + hk_w:], xr.grad[:, hq_w + hk_w:]) < 3e-2
