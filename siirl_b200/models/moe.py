"""Mixture-of-experts MLP (Qwen3-MoE style: softmax router, top-k, optional renormalisation, SwiGLU experts).

The reference reaches MoE through Megatron-core (``moe_grouped_gemm`` + all-to-all dispatcher,
siirl/models/mcore/config_converter.py qwen3moe branch).  Here the single-GPU / data-parallel path sorts tokens by
expert and runs each expert's two GEMMs on the tcgen05 GEMM (the expert-parallel all-to-all path lives in
``siirl_b200.parallel.expert_parallel``)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import ops


def route_topk(x: torch.Tensor, router_weight: torch.Tensor, top_k: int, norm_topk_prob: bool):
    """Router probabilities (fp32 softmax over experts), top-k ids and weights per token."""
    logits = ops.linear(x, router_weight).float() if x.is_cuda else F.linear(x.float(), router_weight.float())
    probs = torch.softmax(logits, dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if norm_topk_prob:
        w = w / w.sum(-1, keepdim=True)
    return w, idx


def moe_forward(x: torch.Tensor, router_weight: torch.Tensor, experts_gate_up: torch.Tensor,
                experts_down: torch.Tensor, top_k: int, norm_topk_prob: bool = True) -> torch.Tensor:
    """``x [T, H]`` -> ``[T, H]``.  experts_gate_up ``[E, 2I, H]``, experts_down ``[E, H, I]``."""
    T, H = x.shape
    E = experts_gate_up.shape[0]
    w, idx = route_topk(x, router_weight, top_k, norm_topk_prob)
    flat_e = idx.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    tok = (order // top_k)
    counts = torch.bincount(flat_e, minlength=E).tolist()
    xs = x.index_select(0, tok)                       # tokens grouped by expert
    ws = w.reshape(-1).index_select(0, order).to(x.dtype)
    outs = []
    start = 0
    for e in range(E):
        n = counts[e]
        if n == 0:
            continue
        xe = xs[start:start + n]
        he = ops.swiglu(ops.linear(xe, experts_gate_up[e]))
        outs.append(ops.linear(he, experts_down[e]))
        start += n
    ys = torch.cat(outs, dim=0) * ws[:, None]
    out = torch.zeros(T, H, dtype=ys.dtype, device=x.device).index_add_(0, tok, ys)
    return out.to(x.dtype)
