"""CUDA kernels of siirl_b200.ops.dense against plain PyTorch fp32 statements of the same op."""
import pytest
import torch

from siirl_b200 import ops
from siirl_b200.ops import dense, lib, reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("tile_n", [128, 256])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (300, 520, 200), (1024, 4608, 3584)])
def test_gemm_nt(shape, tile_n):
    M, N, K = shape
    torch.manual_seed(0)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    out = ops.gemm(a, b, bias=bias, tile_n=tile_n)
    lib.check_status()
    want = a.float() @ b.float().t() + bias.float()
    assert _rel_err(out, want) < 1e-2
    out32 = ops.gemm(a, b, epi=dense.EPI_F32, tile_n=tile_n)
    lib.check_status()
    assert _rel_err(out32, a.float() @ b.float().t()) < 1e-3


@pytest.mark.parametrize("shape", [(128, 128, 64), (256, 320, 192), (520, 384, 264), (2048, 3584, 4608)])
def test_gemm_dgrad_layout(shape):
    """B stored [K, N] (weight [out,in] used for dx = dy @ W)."""
    M, N, K = shape
    torch.manual_seed(1)
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(K, N, device=DEV, dtype=torch.bfloat16)
    out = ops.gemm(a, b, b_mn=True)
    lib.check_status()
    assert _rel_err(out, a.float() @ b.float()) < 1e-2


@pytest.mark.parametrize("shape", [(128, 128, 64), (320, 256, 192), (384, 520, 1000), (3584, 4608, 2048)])
def test_gemm_wgrad_layout(shape):
    """A stored [K, M], B stored [K, N]; fp32 accumulate epilogue (dW += dy^T x)."""
    M, N, K = shape
    torch.manual_seed(2)
    a = torch.randn(K, M, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(K, N, device=DEV, dtype=torch.bfloat16)
    acc = torch.randn(M, N, device=DEV, dtype=torch.float32)
    want = acc + a.float().t() @ b.float()
    ops.gemm(a, b, out=acc, a_mn=True, b_mn=True, epi=dense.EPI_F32_ACC)
    lib.check_status()
    assert _rel_err(acc, want) < 1e-3


def test_linear_autograd_matches_torch():
    torch.manual_seed(3)
    x = torch.randn(4, 96, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(384, 256, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    b = torch.randn(384, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = ops.linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 1e-2
    assert _rel_err(w.grad, wr.grad) < 1e-2
    assert _rel_err(b.grad, br.grad) < 1e-2


@pytest.mark.parametrize("H", [128, 3584, 8192])
@pytest.mark.parametrize("with_res", [False, True])
def test_rmsnorm_fwd_bwd(H, with_res):
    torch.manual_seed(4)
    T = 77
    x = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True) if with_res else None
    w = (1 + 0.1 * torch.randn(H, device=DEV)).to(torch.bfloat16).requires_grad_()
    y, h = ops.rmsnorm(x, w, 1e-6, residual=r)
    gy, gh = torch.randn_like(y), torch.randn_like(y)
    (y.float() * gy.float()).sum().add((h.float() * gh.float()).sum()).backward()
    xr = x.detach().float().requires_grad_()
    rr = r.detach().float().requires_grad_() if with_res else None
    wr = w.detach().float().requires_grad_()
    hr = xr + rr if with_res else xr
    if with_res:
        hr = hr + (hr.to(torch.bfloat16).float() - hr).detach()  # kernel rounds h to bf16
    yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * wr
    ((yr * gy.float()).sum() + (hr * gh.float()).sum()).backward()
    assert _rel_err(y, yr) < 1e-2
    assert _rel_err(x.grad, xr.grad) < 2e-2
    assert _rel_err(w.grad, wr.grad) < 2e-2
    if with_res:
        assert _rel_err(r.grad, rr.grad) < 2e-2


def test_rope_matches_reference_and_inverse():
    torch.manual_seed(5)
    T, hq, hk, D = 50, 4, 2, 128
    qkv = torch.randn(T, (hq + 2 * hk) * D, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    pos = torch.randint(0, 500, (T,), device=DEV)
    cos, sin = ops.rope_tables(D, 512, 1e6, device=DEV)
    out = ops.rope(qkv, hq + hk, D, pos, cos, sin)
    want = ref.rope(qkv.detach()[:, : (hq + hk) * D].reshape(T, hq + hk, D), pos, cos, sin).reshape(T, -1)
    assert _rel_err(out[:, : (hq + hk) * D], want) < 1e-2
    assert torch.equal(out[:, (hq + hk) * D:], qkv[:, (hq + hk) * D:])
    g = torch.randn_like(out)
    out.backward(g)
    want_g = ref.rope(g[:, : (hq + hk) * D].reshape(T, hq + hk, D), pos, cos, sin, inverse=True).reshape(T, -1)
    assert _rel_err(qkv.grad[:, : (hq + hk) * D], want_g) < 1e-2


def test_mrope_sections():
    torch.manual_seed(6)
    T, nh, D = 33, 3, 128
    x = torch.randn(T, nh * D, device=DEV, dtype=torch.bfloat16)
    pos = torch.randint(0, 100, (3, T), device=DEV)
    cos, sin = ops.rope_tables(D, 128, 1e6, device=DEV)
    sec = (16, 24, 24)
    out = ops.rope(x, nh, D, pos, cos, sin, mrope_section=sec)
    want = ref.rope(x.reshape(T, nh, D), pos, cos, sin, mrope_section=sec).reshape(T, -1)
    assert _rel_err(out, want) < 1e-2


def test_swiglu_fwd_bwd():
    torch.manual_seed(7)
    gu = torch.randn(65, 2 * 352, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    out = ops.swiglu(gu)
    g = torch.randn_like(out)
    out.backward(g)
    gr = gu.detach().float().requires_grad_()
    a, b = gr.chunk(2, -1)
    outr = torch.nn.functional.silu(a) * b
    outr.backward(g.float())
    assert _rel_err(out, outr) < 1e-2
    assert _rel_err(gu.grad, gr.grad) < 1e-2


def test_embedding_fwd_bwd():
    torch.manual_seed(8)
    V, H = 1000, 256
    table = torch.randn(V, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, V, (7, 19), device=DEV)
    out = ops.embedding(ids, table)
    assert torch.equal(out, table.detach()[ids])
    g = torch.randn_like(out)
    out.backward(g)
    want = torch.zeros(V, H, device=DEV).index_add_(0, ids.reshape(-1), g.reshape(-1, H).float())
    assert _rel_err(table.grad, want) < 1e-2


@pytest.mark.parametrize("shape", [(64, 3584, 3584), (7, 3584, 18944), (128, 4608, 3584), (33, 256, 1024),
                                   (200, 4608, 3584), (256, 3584, 18944), (256, 37888, 3584), (300, 1000, 1024),
                                   (512, 3584, 1792), (129, 136, 64)])
def test_skinny_split_k_linear(shape):
    M, N, K = shape
    torch.manual_seed(9)
    x = (0.5 * torch.randn(M, K, device=DEV)).to(torch.bfloat16)
    w = (0.05 * torch.randn(N, K, device=DEV)).to(torch.bfloat16)
    b = torch.randn(N, device=DEV).to(torch.bfloat16)
    with torch.no_grad():
        y = ops.linear(x, w, b)
    lib.check_status()
    want = x.float() @ w.float().t() + b.float()
    assert _rel_err(y, want) < 1e-2
    # no row or column of the (possibly transposed-store) tile went astray: element-wise bound, bf16 output rounding
    assert (y.float() - want).abs().max().item() < 0.05 * want.abs().max().item() + 0.05
    assert dense._skinny_splits(64, 3584, 18944) > 1
    if M > 128:     # the operand-swapped form and the plain form agree
        dense.SWAP_OPERANDS_ABOVE_128_ROWS = False
        try:
            with torch.no_grad():
                y2 = ops.linear(x, w, b)
        finally:
            dense.SWAP_OPERANDS_ABOVE_128_ROWS = True
        assert _rel_err(y, y2) < 1e-2


def test_optimizer_state_offload_round_trip():
    """Adam moments parked in pinned host memory between steps give the same updates as resident ones."""
    import torch

    from siirl_b200.parallel.flat_params import FlatParamStore

    def make():
        torch.manual_seed(0)
        m = torch.nn.Linear(256, 512, bias=True).cuda().bfloat16()
        return m, FlatParamStore(m)

    (ma, sa), (mb, sb) = make(), make()
    g = torch.Generator(device="cuda").manual_seed(1)
    for step in range(3):
        grad = torch.randn(sa.total, device="cuda", generator=g)
        for s in (sa, sb):
            s.flat_grad.copy_(grad)
        # no clipping: the clip factor comes from an atomically accumulated norm whose last bits vary run to run
        sa.step(1e-2, max_grad_norm=0.0)
        sb.step(1e-2, max_grad_norm=0.0)
        sb.offload_state()
        assert sb.exp_avg is None and sb._host_state["exp_avg"].is_pinned()
    sb.reload_state()
    assert torch.equal(sa.flat_param, sb.flat_param) and torch.equal(sa.exp_avg, sb.exp_avg)
    assert torch.equal(sa.exp_avg_sq, sb.exp_avg_sq)
