"""Per-kernel benchmark: one JSON line per case with the achieved rate and the fraction of the measured roofline.

    python -m siirl_b200.benchmarks.kernels --case all            # everything, production shapes
    python -m siirl_b200.benchmarks.kernels --case gemm --small   # small shapes for a profiler capture

Timing: CUDA events on the launching stream, 3 warm-up iterations, L2 flushed (a 256 MB buffer is overwritten)
between timed iterations, median of the timed iterations.  Denominators come from ``MEASURED_PEAKS.json`` at the
repository root when present (copy bandwidth and cuBLAS bf16 throughput measured on this pool), else from the
fallback figures 6.65 TB/s and 1.59 PFLOP/s."""
from __future__ import annotations

import argparse
import json
import os

import torch

from .. import ops
from ..ops import dense, lib
from ..ops.attention import SeqInfo, attention_packed
from ..ops.lm_head import lm_head_logprob_entropy


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    path = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "source": "fallback"}


_flush = None


def timeit(fn, iters: int = 10, warm: int = 3, flush: bool = True) -> float:
    global _flush
    if flush and _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            _flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def report(name, ms, flops=None, bytes_=None, **extra):
    pk = peaks()
    out = {"kernel": name, "ms": round(ms, 4), **extra}
    if flops:
        out["tflops"] = round(flops / ms / 1e9, 1)
        out["frac_of_%s_gemm_peak" % pk["source"]] = round(flops / ms / 1e9 / pk["tflops"], 3)
    if bytes_:
        out["gbs"] = round(bytes_ / ms / 1e6, 1)
        out["frac_of_%s_copy_bw" % pk["source"]] = round(bytes_ / ms / 1e6 / pk["hbm_gbs"], 3)
    print(json.dumps(out), flush=True)


def bench_gemm(small: bool):
    shapes = [(2048, 4608, 3584)] if small else [(8192, 4608, 3584), (8192, 3584, 3584), (8192, 37888, 3584),
                                                 (8192, 3584, 18944), (2048, 152064, 3584)]
    for M, N, K in shapes:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fl = 2.0 * M * N * K
        report("gemm_bf16_tcgen05 fwd (x W^T), CTA-pair kernel", timeit(lambda: ops.gemm(a, b, out=out)), fl, M=M, N=N,
               K=K)
        if small:
            continue
        dense.set_pair_kernel(False)
        report("gemm_bf16_tcgen05 fwd (x W^T), one-CTA kernel", timeit(lambda: ops.gemm(a, b, out=out)), fl, M=M, N=N,
               K=K)
        dense.set_pair_kernel(True)
        report("cublas bf16 (torch.matmul)", timeit(lambda: torch.matmul(a, b.t(), out=out)), fl, M=M, N=N, K=K)
        bt = torch.randn(K, N, device="cuda", dtype=torch.bfloat16)
        report("gemm_bf16_tcgen05 dgrad layout", timeit(lambda: ops.gemm(a, bt, out=out, b_mn=True)), fl, M=M, N=N, K=K)
        at = torch.randn(K, M, device="cuda", dtype=torch.bfloat16)
        acc = torch.zeros(M, N, device="cuda", dtype=torch.float32)
        report("gemm_bf16_tcgen05 wgrad layout (fp32 +=)",
               timeit(lambda: ops.gemm(at, bt, out=acc, a_mn=True, b_mn=True, epi=dense.EPI_F32_ACC)), fl, M=M, N=N, K=K)
    lib.check_status()


def bench_attention(small: bool):
    cases = [(28, 4, 128, [1024] * 2)] if small else [(28, 4, 128, [2048] * 8), (28, 4, 128, [640 + 64 * i for i in range(16)]),
                                                       (28, 4, 128, [16384])]
    for hq, hkv, d, lens in cases:
        T = sum(lens)
        qkv = (0.5 * torch.randn(T, (hq + 2 * hkv) * d, device="cuda")).to(torch.bfloat16).requires_grad_()
        info = SeqInfo(lens, device="cuda")
        fl = 4.0 * hq * d * sum(0.5 * s * s for s in lens)
        with torch.no_grad():
            report("fmha_fwd (causal, GQA)", timeit(lambda: attention_packed(qkv, info, hq, hkv, d)), fl, T=T,
                   seqs=len(lens))
        out = attention_packed(qkv, info, hq, hkv, d)
        g = torch.randn_like(out)

        def bwd():
            qkv.grad = None
            out.backward(g, retain_graph=True)

        report("fmha_bwd (causal, GQA)", timeit(bwd), 2.5 * fl, T=T, seqs=len(lens))
        if small:
            continue
        try:        # the library bar on the same box and shapes: flash-attn's varlen kernels (what the reference calls)
            from flash_attn import flash_attn_varlen_func
        except Exception:  # noqa: BLE001
            continue
        q = qkv.detach()[:, : hq * d].reshape(T, hq, d).contiguous().requires_grad_()
        k = qkv.detach()[:, hq * d:(hq + hkv) * d].reshape(T, hkv, d).contiguous().requires_grad_()
        v = qkv.detach()[:, (hq + hkv) * d:].reshape(T, hkv, d).contiguous().requires_grad_()
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
        mx = max(lens)
        with torch.no_grad():
            report("flash_attn 2.8 varlen fwd (library bar)",
                   timeit(lambda: flash_attn_varlen_func(q, k, v, cu, cu, mx, mx, causal=True)), fl, T=T, seqs=len(lens))
        o2 = flash_attn_varlen_func(q, k, v, cu, cu, mx, mx, causal=True)
        g2 = torch.randn_like(o2)

        def bwd2():
            q.grad = k.grad = v.grad = None
            o2.backward(g2, retain_graph=True)

        report("flash_attn 2.8 varlen bwd (library bar)", timeit(bwd2), 2.5 * fl, T=T, seqs=len(lens))
    lib.check_status()


def bench_lm_head(small: bool):
    """Log-prob + entropy over the 152k vocabulary: the GEMM whose epilogue folds the softmax statistics (no logits in
    memory) against the earlier GEMM -> fp32 logits -> row-reduction form, forward and forward + backward."""
    from ..ops import lm_head as LM
    T, V, H = (1024, 152064, 3584) if small else (8192, 152064, 3584)
    h = (0.5 * torch.randn(T, H, device="cuda")).to(torch.bfloat16).requires_grad_()
    w = (0.02 * torch.randn(V, H, device="cuda")).to(torch.bfloat16).requires_grad_()
    w.main_grad = torch.zeros(V, H, device="cuda", dtype=torch.float32)
    y = torch.randint(0, V, (T,), device="cuda")
    g = torch.randn(T, device="cuda")
    for fused in ((True,) if small else (True, False)):
        LM.FUSED_EPILOGUE = fused
        tag = "fused epilogue" if fused else "fp32 logits chunk + reduction kernel"
        with torch.no_grad():
            report(f"lm_head logprob+entropy fwd ({tag})",
                   timeit(lambda: lm_head_logprob_entropy(h, w, y, 1.0), iters=5), 2.0 * T * V * H, T=T, V=V)
        if small:
            continue

        def fb():
            h.grad = None
            lp, ent = lm_head_logprob_entropy(h, w, y, 1.0)
            (lp * g + 0.01 * ent).sum().backward()

        report(f"lm_head fwd+bwd ({tag})", timeit(fb, iters=3), 2.0 * T * V * H * 4, T=T, V=V)
    LM.FUSED_EPILOGUE = True
    lib.check_status()


def bench_memory_bound(small: bool):
    T, H, I = (4096, 3584, 18944) if small else (16384, 3584, 18944)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    r = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        report("rmsnorm_fwd (+residual)", timeit(lambda: ops.rmsnorm(x, w, 1e-6, residual=r)), bytes_=T * H * 2 * 4, T=T)
        gu = torch.randn(T, 2 * I, device="cuda", dtype=torch.bfloat16)
        report("swiglu_fwd", timeit(lambda: ops.swiglu(gu)), bytes_=T * I * 2 * 3, T=T)
    n = 1 << 28
    g = torch.randn(n, device="cuda")
    from ..parallel.flat_params import FlatParamStore

    class _M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.p = torch.nn.Parameter(torch.zeros(n, device="cuda", dtype=torch.bfloat16))

    store = FlatParamStore(_M())
    store.flat_grad.copy_(g)
    report("sumsq + adamw (fp32 master/m/v, bf16 copy)", timeit(lambda: store.step(1e-4), iters=5),
           bytes_=n * (4 + 4 * 4 + 3 * 4 + 2), n=n)
    lib.check_status()


def bench_gemm_decode(small: bool):
    """The four projections of a Qwen2.5-7B layer at decode batch sizes, through the path the rollout engine takes
    (``ops.linear`` without autograd: split-K tcgen05 GEMM + slab reduction).  These are weight-streaming bound: the
    figure of merit is the fraction of the measured copy bandwidth."""
    shapes = [(3584, 18944, "down_proj")] if small else [(4608, 3584, "qkv_proj"), (3584, 3584, "o_proj"),
                                                          (37888, 3584, "gate_up_proj"), (3584, 18944, "down_proj")]
    for M in ((256,) if small else (64, 256)):
        for N, K, name in shapes:
            x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
            w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
            with torch.no_grad():
                ms = timeit(lambda: ops.linear(x, w))
            report(f"decode {name}" + (" (weights in the A operand, transposed store)" if M > 128 else
                                       " (split-K GEMM + reduce)"), ms, bytes_=N * K * 2, M=M, N=N, K=K)
            if M > 128:
                dense.SWAP_OPERANDS_ABOVE_128_ROWS = False
                with torch.no_grad():
                    ms = timeit(lambda: ops.linear(x, w))
                dense.SWAP_OPERANDS_ABOVE_128_ROWS = True
                report(f"decode {name} (x in the A operand: two 128-row blocks)", ms, bytes_=N * K * 2, M=M, N=N, K=K)
    lib.check_status()


def bench_moe(small: bool, skip_library: bool = False):
    """Mixture-of-experts MLP of the Qwen3-30B-A3B shape on one GPU (all experts local): dispatch + two grouped
    tcgen05 GEMMs + SwiGLU + combine, against a loop of per-expert cuBLAS GEMMs (torch.matmul) over the same routing."""
    from ..models.moe import moe_forward, route_topk
    T, H, I, E, k = (2048, 2048, 768, 128, 8) if small else (8192, 2048, 768, 128, 8)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    rw = (0.5 * torch.randn(E, H, device="cuda")).to(torch.bfloat16)
    gu = (0.05 * torch.randn(E, 2 * I, H, device="cuda")).to(torch.bfloat16)
    dn = (0.05 * torch.randn(E, H, I, device="cuda")).to(torch.bfloat16)
    fl = 2.0 * T * k * H * 3 * I

    def library_loop():
        w, idx = route_topk(x, rw, k, True)
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=E).tolist()
        xs = x.index_select(0, order // k)
        outs, start = [], 0
        for e in range(E):
            n = counts[e]
            if n:
                h = torch.matmul(xs[start:start + n], gu[e].t())
                h = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
                outs.append(torch.matmul(h, dn[e].t()))
                start += n
        ys = torch.cat(outs) * w.reshape(-1)[order].to(x.dtype)[:, None]
        return torch.zeros(T, H, dtype=ys.dtype, device="cuda").index_add_(0, order // k, ys)

    with torch.no_grad():
        t_lib = float("nan") if skip_library else timeit(library_loop, iters=5)
        t_own = timeit(lambda: moe_forward(x, rw, gu, dn, k, True), iters=5)
    report("moe_mlp fwd: dispatch + grouped tcgen05 GEMMs + combine", t_own, fl, T=T, E=E, top_k=k,
           per_expert_cublas_loop_ms=round(t_lib, 4), speedup_vs_loop=round(t_lib / t_own, 3))
    # router: one kernel against softmax + topk + sum + div on the same bf16 logits
    from ..ops.moe import route_topk as route_kernel, route_topk_reference
    logits = torch.randn(T, E, device="cuda").to(torch.bfloat16)
    with torch.no_grad():
        t_ref = timeit(lambda: route_topk_reference(logits, k, True), iters=10)
        t_k = timeit(lambda: route_kernel(logits, k, True), iters=10)
    print(json.dumps({"kernel": "moe_route_topk fwd", "ms": round(t_k, 4), "T": T, "E": E, "top_k": k,
                      "library_softmax_topk_ms": round(t_ref, 4), "speedup": round(t_ref / t_k, 2)}))
    lib.check_status()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all", choices=["all", "gemm", "gemm_decode", "attention", "lm_head", "memory", "moe"])
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--skip-library", action="store_true", help="moe: time only this repo's path (short launch lists)")
    a = ap.parse_args()
    print(json.dumps({"peaks": peaks(), "device": torch.cuda.get_device_name()}))
    if a.case in ("all", "gemm"):
        bench_gemm(a.small)
    if a.case in ("all", "gemm_decode"):
        bench_gemm_decode(a.small)
    if a.case in ("all", "attention"):
        bench_attention(a.small)
    if a.case in ("all", "lm_head"):
        bench_lm_head(a.small)
    if a.case in ("all", "memory"):
        bench_memory_bound(a.small)
    if a.case in ("all", "moe"):
        bench_moe(a.small, a.skip_library)


if __name__ == "__main__":
    main()
