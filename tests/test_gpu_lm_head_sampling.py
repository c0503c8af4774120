"""LM-head log-prob/entropy, sampler and paged decode attention against PyTorch statements."""
import math

import pytest
import torch

from siirl_b200.ops import kv_cache as kvc
from siirl_b200.ops import lib, reference as ref
from siirl_b200.ops.lm_head import lm_head_logprob_entropy
from siirl_b200.ops.sampling import sample

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("T,V,H,temp", [(37, 1000, 128, 1.0), (300, 5003 // 8 * 8, 256, 0.7), (257, 2048, 192, 1.3)])
def test_lm_head_fwd_bwd(T, V, H, temp, fused, monkeypatch):
    from siirl_b200.ops import lm_head
    monkeypatch.setattr(lm_head, "FUSED_EPILOGUE", fused)
    torch.manual_seed(0)
    h = (0.5 * torch.randn(T, H, device=DEV)).to(torch.bfloat16).requires_grad_()
    w = (0.2 * torch.randn(V, H, device=DEV)).to(torch.bfloat16).requires_grad_()
    y = torch.randint(0, V, (T,), device=DEV)
    lp, ent = lm_head_logprob_entropy(h, w, y, temp)
    lib.check_status()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lpr, entr = ref.lm_head_logprob_entropy(hr, wr, y, temp)
    torch.testing.assert_close(lp, lpr, rtol=2e-3, atol=2e-3)
    torch.testing.assert_close(ent, entr, rtol=2e-3, atol=2e-3)
    g1, g2 = torch.randn(T, device=DEV), 0.1 * torch.randn(T, device=DEV)
    (lp * g1 + ent * g2).sum().backward()
    (lpr * g1 + entr * g2).sum().backward()
    assert _rel(h.grad, hr.grad) < 3e-2
    assert _rel(w.grad, wr.grad) < 3e-2


def test_sampler_greedy_and_distribution():
    torch.manual_seed(1)
    B, V = 64, 512
    logits = torch.randn(B, V, device=DEV) * 2
    tok, lp = sample(logits, temperature=0.0)
    assert torch.equal(tok, logits.argmax(-1))
    torch.testing.assert_close(lp, torch.log_softmax(logits, -1).gather(-1, tok[:, None]).squeeze(-1), rtol=1e-4,
                               atol=1e-4)
    # empirical distribution of one row over many steps matches softmax(z / T)
    row = logits[:1].repeat(4096, 1)
    counts = torch.zeros(V, device=DEV)
    for step in range(8):
        t, l = sample(row, temperature=0.8, seed=7, step=step)
        counts += torch.bincount(t, minlength=V).float()
    emp = counts / counts.sum()
    want = torch.softmax(logits[0] / 0.8, -1)
    assert (emp - want).abs().max().item() < 0.02
    # log-prob is the tempered full-distribution one
    t, l = sample(logits, temperature=0.8, seed=3, step=1)
    torch.testing.assert_close(l, torch.log_softmax(logits / 0.8, -1).gather(-1, t[:, None]).squeeze(-1), rtol=1e-4,
                               atol=1e-4)
    # same (seed, step) -> same tokens; device counter shifts the stream
    t2, _ = sample(logits, temperature=0.8, seed=3, step=1)
    assert torch.equal(t, t2)
    t3, _ = sample(logits, temperature=0.8, seed=3, step=0, step_dev=torch.ones(1, dtype=torch.int64, device=DEV))
    assert torch.equal(t, t3)


def test_sampler_top_k_top_p_support():
    torch.manual_seed(2)
    logits = torch.randn(256, 100, device=DEV)
    t, _ = sample(logits, temperature=1.0, top_k=5, seed=1)
    top5 = torch.topk(logits, 5, -1).indices
    assert (top5 == t[:, None]).any(-1).all()
    t, _ = sample(logits, temperature=1.0, top_p=0.3, seed=2)
    sp, si = torch.sort(torch.softmax(logits, -1), -1, descending=True)
    keep = (sp.cumsum(-1) - sp) < 0.3
    allowed = torch.zeros_like(keep).scatter(-1, si, keep)
    assert allowed.gather(-1, t[:, None]).all()


@pytest.mark.parametrize("D,hq,hkv", [(128, 28, 4), (64, 14, 2), (128, 8, 8)])
def test_decode_attention_matches_eager(D, hq, hkv):
    torch.manual_seed(3)
    B, nblocks, max_blocks = 5, 40, 6
    cache = (0.5 * torch.randn(nblocks, 2, hkv, kvc.BLOCK, D, device=DEV)).to(torch.bfloat16)
    seq_lens = torch.tensor([1, 64, 65, 200, 0], dtype=torch.int32, device=DEV)
    perm = torch.randperm(nblocks)[: B * max_blocks].reshape(B, max_blocks).to(torch.int32).to(DEV)
    q = (0.5 * torch.randn(B, (hq + 2 * hkv) * D, device=DEV)).to(torch.bfloat16)
    out = kvc.decode_attention(q, cache, seq_lens, perm, hq, hkv, D)
    lib.check_status()
    want = kvc.decode_attention(q.cpu().float(), cache.cpu().float(), seq_lens.cpu(), perm.cpu(), hq, hkv, D)
    assert _rel(out[:4].cpu(), want[:4]) < 2e-2
    assert out[4].abs().max().item() == 0


@pytest.mark.parametrize("D,hq,hkv", [(128, 28, 4), (64, 14, 2), (128, 32, 4), (128, 8, 8)])
def test_split_decode_attention_matches_eager(D, hq, hkv):
    """Persistent split-K/V decode kernel: contexts below one chunk (written directly), across several chunks
    (partials + merge), ragged lengths, an empty slot, and more work items than SMs."""
    torch.manual_seed(5)
    lens = [1, 64, 65, 200, 0, 1024, 1025, 2300, 3000, 777] + [1500 + 37 * i for i in range(40)]
    B = len(lens)
    max_blocks = 48
    need = sum((n + kvc.BLOCK - 1) // kvc.BLOCK for n in lens)
    nblocks = need + 8
    cache = (0.5 * torch.randn(nblocks, 2, hkv, kvc.BLOCK, D, device=DEV)).to(torch.bfloat16)
    order = torch.randperm(nblocks)
    table = torch.full((B, max_blocks), -1, dtype=torch.int32)
    at = 0
    for i, n in enumerate(lens):
        nb = (n + kvc.BLOCK - 1) // kvc.BLOCK
        table[i, :nb] = order[at:at + nb].to(torch.int32)
        at += nb
    table = table.to(DEV)
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    q = (0.5 * torch.randn(B, (hq + 2 * hkv) * D, device=DEV)).to(torch.bfloat16)
    kvc.set_decode_kernel("split")
    try:
        out = kvc.decode_attention(q, cache, seq_lens, table, hq, hkv, D)
        lib.check_status()
        again = kvc.decode_attention(q, cache, seq_lens, table, hq, hkv, D)      # barriers / workspace reuse
        lib.check_status()
        kvc.set_decode_kernel("simple")
        simple = kvc.decode_attention(q, cache, seq_lens, table, hq, hkv, D)
        lib.check_status()
    finally:
        kvc.set_decode_kernel("split")
    want = kvc.decode_attention(q.cpu().float(), cache.cpu().float(), seq_lens.cpu(), table.cpu().clamp(min=0), hq, hkv, D)
    assert torch.equal(out, again)
    live = [i for i, n in enumerate(lens) if n > 0]
    for i in live:
        assert _rel(out[i].cpu(), want[i]) < 2e-2, (i, lens[i])
    assert _rel(out[live].cpu(), simple[live].cpu()) < 1e-2
    assert out[4].abs().max().item() == 0


def test_kv_append_and_fork():
    torch.manual_seed(4)
    hq, hkv, D = 4, 2, 64
    T = 10
    cache = torch.zeros(8, 2, hkv, kvc.BLOCK, D, dtype=torch.bfloat16, device=DEV)
    qkv = torch.randn(T, (hq + 2 * hkv) * D, device=DEV).to(torch.bfloat16)
    bt = torch.tensor([[3, 5], [1, -1]], dtype=torch.int32, device=DEV)
    seq = torch.tensor([0] * 6 + [1] * 3 + [-1], dtype=torch.int32, device=DEV)
    pos = torch.tensor([60, 61, 62, 63, 64, 65, 0, 1, 2, 0], dtype=torch.int32, device=DEV)
    kvc.kv_append(qkv, seq, pos, bt, cache, hq, hkv, D)
    want = torch.zeros_like(cache).cpu()
    kvc.kv_append(qkv.cpu(), seq.cpu(), pos.cpu(), bt.cpu(), want, hq, hkv, D)
    assert torch.equal(cache.cpu(), want)
    kvc.kv_copy_blocks(cache, torch.tensor([3], dtype=torch.int32, device=DEV),
                       torch.tensor([7], dtype=torch.int32, device=DEV))
    assert torch.equal(cache[7], cache[3])
