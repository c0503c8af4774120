"""Mixture-of-experts path on one GPU: grouped tcgen05 GEMM (forward, dgrad, per-expert wgrad), dispatch / combine
kernels, against the per-expert PyTorch fp32 reference."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,H,I,E,k", [(300, 256, 128, 8, 2), (1000, 512, 256, 16, 4), (64, 128, 64, 4, 1)])
def test_moe_forward_backward_matches_reference(T, H, I, E, k):
    from siirl_b200.models.moe import moe_forward, moe_forward_reference
    from siirl_b200.ops import lib
    g = torch.Generator().manual_seed(3)
    rw = 0.5 * torch.randn(E, H, generator=g)
    gu = 0.1 * torch.randn(E, 2 * I, H, generator=g)
    dn = 0.1 * torch.randn(E, H, I, generator=g)
    x = torch.randn(T, H, generator=g)
    go = torch.randn(T, H, generator=g)
    rd = lambda t: t.to(torch.bfloat16).float()  # noqa: E731
    xg = x.cuda().bfloat16().requires_grad_()
    gug, dng = gu.cuda().bfloat16().requires_grad_(), dn.cuda().bfloat16().requires_grad_()
    y = moe_forward(xg, rw.cuda().bfloat16(), gug, dng, k, True)
    y.backward(go.cuda().bfloat16())
    torch.cuda.synchronize()
    lib.check_status()
    xo, guo, dno = rd(x).requires_grad_(), rd(gu).requires_grad_(), rd(dn).requires_grad_()
    yo = moe_forward_reference(xo, rd(rw), guo, dno, k, True)
    yo.backward(rd(go))

    def close(a, b, what):
        err = (a.float().cpu() - b).abs().max().item()
        assert err <= 0.05 * max(1.0, b.abs().max().item()), f"{what}: {err}"

    close(y, yo.detach(), "y")
    close(xg.grad, xo.grad, "dx")
    close(gug.grad, guo.grad, "d gate_up")
    close(dng.grad, dno.grad, "d down")


def test_grouped_wgrad_accumulates_into_main_grad():
    from siirl_b200.ops import moe as M
    E, N, K, k, T = 4, 128, 64, 1, 500
    idx = torch.randint(0, E, (1, T, k), device="cuda", dtype=torch.int32)
    lay = M.build_layout(idx, E, 1, 0)
    ep = M.ExpertParallel()
    x = torch.randn(T, K, device="cuda").bfloat16()
    W = torch.nn.Parameter((0.1 * torch.randn(E, N, K, device="cuda")).bfloat16())
    W.main_grad = torch.ones(E, N, K, device="cuda")
    xs = M.dispatch(x, ep, lay)
    ys = M.grouped_linear(xs, W, lay)
    dy = torch.randn_like(ys)
    ys.backward(dy)
    assert W.grad is None
    rows = lay.group_rows.tolist()
    for e in range(E):
        want = 1.0 + dy[rows[e]:rows[e + 1]].float().t() @ xs[rows[e]:rows[e + 1]].float()
        assert (W.main_grad[e] - want).abs().max().item() < 0.05 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("T,E,k,norm,dtype", [(257, 128, 8, True, torch.float32), (64, 8, 2, False, torch.float32),
                                             (1000, 60, 4, True, torch.bfloat16), (5, 256, 32, True, torch.float32),
                                             (33, 4, 1, True, torch.float32)])
def test_route_topk_kernel_matches_fp32_reference(T, E, k, norm, dtype):
    from siirl_b200.ops import lib
    from siirl_b200.ops.moe import route_topk, route_topk_reference
    g = torch.Generator().manual_seed(T + E)
    logits = (2.0 * torch.randn(T, E, generator=g)).to(dtype)
    dw = torch.randn(T, k, generator=g)
    lg = logits.cuda().requires_grad_()
    w, idx = route_topk(lg, k, norm)
    (w * dw.cuda()).sum().backward()
    torch.cuda.synchronize()
    lib.check_status()
    lo = logits.float().requires_grad_()
    wo, io = route_topk_reference(lo, k, norm)
    (wo * dw).sum().backward()
    assert idx.dtype == torch.int64 and w.dtype == torch.float32
    # the selected SET must carry the same probabilities (bf16 logits can tie: compare sorted weights, and ids where
    # the probabilities are distinct)
    assert torch.allclose(w.cpu(), wo, rtol=1e-4, atol=1e-6)
    pk = torch.softmax(logits.float(), -1).topk(min(k + 1, E), -1).values          # incl. the first one left out
    distinct = (pk[:, :-1] - pk[:, 1:]).abs().min(-1).values > 1e-7 if E > 1 else torch.ones(T, dtype=torch.bool)
    assert torch.equal(idx.cpu()[distinct], io[distinct])
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert torch.allclose(lg.grad.float().cpu()[distinct], lo.grad[distinct], rtol=tol, atol=tol * 1e-1)


@pytest.mark.parametrize("W,T,k,E,rank,cap", [(1, 300, 2, 8, 0, None), (2, 1000, 4, 16, 1, None), (4, 513, 8, 128, 2, None),
                                              (1, 64, 1, 4, 0, None), (2, 700, 2, 256, 0, 1024), (1, 5000, 8, 128, 0, None)])
def test_fused_layout_kernels_match_device_op_construction(W, T, k, E, rank, cap):
    from siirl_b200.ops import lib
    from siirl_b200.ops import moe as M
    g = torch.Generator().manual_seed(W * 1000 + T)
    idx = torch.randint(0, E, (W, T, k), generator=g, dtype=torch.int32)
    idx[:, T - T // 7:, :] = -1                     # padding tokens at the end of every rank's rows
    if E >= 8:
        idx[idx == 3] = 5                           # an expert without tokens
    idx = idx.cuda()
    fused = M.build_layout(idx, E, W, rank, cap)
    torch.cuda.synchronize()
    lib.check_status()
    M._FUSED_LAYOUT = False
    try:
        ref = M.build_layout(idx, E, W, rank, cap)
    finally:
        M._FUSED_LAYOUT = True
    assert fused.capacity == ref.capacity
    for name in ("pair_rank", "pair_slot", "slot_src_rank", "slot_src_row", "slot_pair", "tile_group", "group_rows"):
        a, b = getattr(fused, name), getattr(ref, name)
        assert a.dtype == b.dtype and a.shape == b.shape, name
        assert torch.equal(a, b), name
