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
    (128, 4, 2, [1024, 384]),
    (64, 2, 2, [257]),
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
    # element-wise bounds as well: a Frobenius norm hides a wrong row or column (bf16 rounding of O(1) values is
    # ~4e-3; gradients are sums of a few hundred such terms)
    assert (out.float() - outr).abs().max().item() < 3e-2
    gmax = xr.grad.abs().max().item()
    assert (qkv.grad.float() - xr.grad).abs().max().item() < 4e-2 * max(gmax, 1.0)
    # per-row check: no single token's gradient is off
    row_err = (qkv.grad.float() - xr.grad).norm(dim=1) / (xr.grad.norm(dim=1) + 1e-3)
    assert row_err.max().item() < 0.1, row_err.argmax().item()
