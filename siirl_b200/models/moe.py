"""Mixture-of-experts MLP (Qwen3-MoE style: softmax router, top-k, optional renormalisation, SwiGLU experts).

The reference reaches MoE through Megatron-core (``moe_grouped_gemm`` + all-to-all dispatcher,
siirl/models/mcore/config_converter.py qwen3moe branch).  Here the single-GPU / data-parallel path sorts tokens by
expert and runs each expert's two GEMMs on the tcgen05 GEMM (the expert-parallel all-to-all path lives in
``siirl_b200.parallel.expert_parallel``)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from .. import ops


def route_topk(x: torch.Tensor, router_weight: torch.Tensor, top_k: int, norm_topk_prob: bool):
    """Router probabilities (fp32 softmax over experts), top-k ids and weights per token."""
    if x.is_cuda and router_weight.shape[0] % 8 == 0:
        logits = ops.linear(x, router_weight)          # bf16; the routing kernel does its softmax in fp32
    else:       # CPU, or an expert count the 16-byte epilogue stores cannot address
        logits = F.linear(x.float(), router_weight.float())
    from ..ops.moe import route_topk as _route
    return _route(logits, top_k, norm_topk_prob)


_LOCAL_EP = None


def route_deepseek(x: torch.Tensor, router_weight: torch.Tensor, bias: Optional[torch.Tensor], cfg):
    """DeepSeek-V3 router (public architecture; the reference reaches it through Megatron's ``moe_router_*`` options,
    siirl/models/mcore/config_converter.py:187-275): sigmoid (or soft-max) scores; experts are CHOSEN by score plus
    the load-balancing bias, restricted to the ``topk_group`` best of ``n_group`` expert groups (a group's rank is the
    sum of its two best biased scores); the mixing WEIGHTS are the unbiased scores of the chosen experts, normalised
    and multiplied by ``routed_scaling_factor``.  Returns ``(w [T, k] fp32, idx [T, k] int64)``."""
    T = x.shape[0]
    E, k = router_weight.shape[0], cfg.num_experts_per_tok
    logits = x.float() @ router_weight.float().t()
    scores = torch.sigmoid(logits) if cfg.scoring_func == "sigmoid" else torch.softmax(logits, -1)
    choice = scores + bias.float()[None] if bias is not None else scores
    if cfg.n_group > 1:
        grp = choice.reshape(T, cfg.n_group, E // cfg.n_group)
        if bias is not None:
            rank = grp.topk(min(2, grp.shape[-1]), dim=-1).values.sum(-1)
        else:
            rank = grp.max(-1).values
        keep = torch.zeros_like(rank).scatter_(1, rank.topk(cfg.topk_group, dim=-1, sorted=False).indices, 1.0)
        mask = keep[:, :, None].expand(T, cfg.n_group, E // cfg.n_group).reshape(T, E) > 0
        choice = choice.masked_fill(~mask, 0.0 if bias is not None else float("-inf"))
    idx = choice.detach().topk(k, dim=-1, sorted=False).indices
    w = scores.gather(1, idx)
    if cfg.norm_topk_prob and k > 1:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * cfg.routed_scaling_factor, idx


def _local_ep():
    global _LOCAL_EP
    if _LOCAL_EP is None:
        from ..ops.moe import ExpertParallel
        _LOCAL_EP = ExpertParallel()
    return _LOCAL_EP


def moe_forward(x: torch.Tensor, router_weight: torch.Tensor, experts_gate_up: torch.Tensor,
                experts_down: torch.Tensor, top_k: int, norm_topk_prob: bool = True, ep=None,
                pad_tokens: int = 0, routed=None) -> torch.Tensor:
    """``x [T, H]`` -> ``[T, H]``.  ``experts_gate_up [E_local, 2I, H]``, ``experts_down [E_local, H, I]`` hold the
    experts hosted by this rank (all of them without expert parallelism); ``router_weight [E, H]`` is replicated.
    One dispatch (rows pulled into the expert-sorted, 128-padded layout), two grouped GEMMs around SwiGLU, one
    combine (top-k weighted sum while pulling the rows back); with ``ep`` the pulls cross NVLink."""
    from ..ops import moe as M
    ep = ep if ep is not None else _local_ep()
    T, H = x.shape
    E = router_weight.shape[0]
    # ``routed``: (weights, expert ids) from a family-specific router instead of soft-max top-k
    w, idx = routed if routed is not None else route_topk(x, router_weight, top_k, norm_topk_prob)
    if ep.world > 1 and pad_tokens:
        # ranks hold different token counts: pad to the static bound; padding rows are routed nowhere (id -1)
        assert T <= pad_tokens, f"{T} tokens exceed the expert-parallel bound {pad_tokens}"
        pad = pad_tokens - T
        x = torch.cat([x, x.new_zeros(pad, H)])
        w = torch.cat([w, w.new_zeros(pad, top_k)])
        idx = torch.cat([idx, idx.new_full((pad, top_k), -1)])
    all_idx = ep.all_gather(idx.to(torch.int32))
    w_all = ep.all_gather(w.detach().float()) if ep.world > 1 else w.detach().float().unsqueeze(0)
    layout = M.build_layout(all_idx, E, ep.world, ep.rank)
    xs = M.dispatch(x, ep, layout)
    hs = ops.swiglu(M.grouped_linear(xs, experts_gate_up, layout))
    ys = M.grouped_linear(hs, experts_down, layout)
    return M.combine(ys, w, w_all, ep, layout).to(x.dtype)[:T]


def moe_forward_reference(x: torch.Tensor, router_weight: torch.Tensor, experts_gate_up: torch.Tensor,
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
