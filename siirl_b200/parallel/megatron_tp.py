"""Tensor parallelism (and Megatron-style sequence parallelism) for TRAINING the packed decoder.

The reference trains tensor-parallel models through Megatron-core (``initialize_model_parallel(tp, pp, ...)``,
siirl/engine/megatron_workers.py:82-476; its legacy Llama / Qwen2 models in siirl/models/llama/megatron and
siirl/models/qwen2/megatron are column- / row-parallel by hand) and ships two utilities around it: vocabulary-parallel
entropy / log-probs (siirl/utils/megatron/tensor_parallel.py:109-158) and ``per_tensor_generator``, which regathers the
shards of every parameter for the rollout engine (siirl/utils/megatron/megatron_utils.py:829-944).  This module is the
native counterpart:

* ``shard_decoder(model, ctx)`` turns a :class:`DecoderLM` into this rank's tensor-parallel slice in place: QKV and
  gate/up projections keep the rows of the local heads / FFN columns (column parallel), attention-output and FFN-down
  projections keep the matching input columns (row parallel), the LM head keeps a contiguous range of vocabulary rows;
  norms and the embedding stay replicated.  The layer forward then runs on ``heads / tp`` heads and ``I / tp`` FFN
  columns with the four region mappings below around the parallel blocks.
* region mappings (autograd functions): ``copy_to_tp`` (identity / all-reduce), ``reduce_from_tp`` (all-reduce /
  identity); with ``sequence_parallel`` the activations between the blocks are split along the token dimension and the
  mappings become ``gather_from_sp`` (all-gather / reduce-scatter) and ``scatter_to_sp`` (reduce-scatter / all-gather).
* ``vocab_parallel_logprob_entropy``: every rank reduces its vocabulary slice to online-softmax statistics (the fused
  LM-head epilogue on GPUs), the ranks exchange four floats per token, and backward forms the gradient of the local
  logits from the global log-sum-exp and entropy -- no rank ever holds more than its ``V / tp`` logits columns.
* ``per_tensor_generator(model, ctx)`` yields ``(name, full tensor)`` for every parameter by gathering the shards
  (checkpoint export, a rollout engine with another tensor-parallel width).

The rollout engine of a tensor-parallel trainer uses the SAME shards (``TPDecoder.from_shards``) when the rollout's
tensor-parallel width equals the trainer's, so the train -> rollout hand-off moves no weights.
"""
from __future__ import annotations

from typing import Iterator, List, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


class TPTrainContext:
    def __init__(self, group, sequence_parallel: bool = False):
        self.group = group
        self.size = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.sequence_parallel = bool(sequence_parallel) and self.size > 1


# ---------------------------------------------------------------------------------------------------------------------
# region mappings
# ---------------------------------------------------------------------------------------------------------------------
def _all_reduce(x: torch.Tensor, group) -> torch.Tensor:
    y = x.contiguous().clone()
    dist.all_reduce(y, group=group)
    return y


def _all_gather_rows(x: torch.Tensor, group) -> torch.Tensor:
    n = dist.get_world_size(group)
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, 0)


def _reduce_scatter_rows(x: torch.Tensor, group) -> torch.Tensor:
    """Sum over the group, keep this rank's block of rows (rows are a multiple of the group size)."""
    n, r = dist.get_world_size(group), dist.get_rank(group)
    rows = x.shape[0] // n
    y = x.contiguous()
    if y.is_cuda:
        out = torch.empty(rows, *y.shape[1:], dtype=y.dtype, device=y.device)
        dist.reduce_scatter_tensor(out, y, group=group)
        return out
    y = y.clone()
    dist.all_reduce(y, group=group)             # gloo has no reduce-scatter
    return y[r * rows:(r + 1) * rows].clone()


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        return _all_reduce(g, ctx.group), None


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        return _all_reduce(x, group)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherFromSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _all_gather_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_rows(g, ctx.group), None


class _ScatterToSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _reduce_scatter_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_rows(g, ctx.group), None


def enter_parallel_block(x: torch.Tensor, tp: TPTrainContext) -> torch.Tensor:
    """Activations in front of a column-parallel projection: every rank needs all rows."""
    if tp.size == 1:
        return x
    return _GatherFromSP.apply(x, tp.group) if tp.sequence_parallel else _CopyToTP.apply(x, tp.group)


def leave_parallel_block(x: torch.Tensor, tp: TPTrainContext) -> torch.Tensor:
    """Partial sums behind a row-parallel projection: add the ranks' contributions."""
    if tp.size == 1:
        return x
    return _ScatterToSP.apply(x, tp.group) if tp.sequence_parallel else _ReduceFromTP.apply(x, tp.group)


def split_rows_for_sp(x: torch.Tensor, tp: TPTrainContext) -> torch.Tensor:
    """This rank's block of token rows (the stream is padded to a multiple of the group size by the caller)."""
    rows = x.shape[0] // tp.size
    return x[tp.rank * rows:(tp.rank + 1) * rows]


class _TakeRowsGatherGrad(torch.autograd.Function):
    """This rank's block of token rows; backward gathers the ranks' row gradients, so that whatever produced the
    rows (the replicated embedding) sees the gradient of all of them on every rank."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n, r = dist.get_world_size(group), dist.get_rank(group)
        rows = x.shape[0] // n
        return x[r * rows:(r + 1) * rows].contiguous()

    @staticmethod
    def backward(ctx, g):
        return _all_gather_rows(g, ctx.group), None


def take_rows_for_sp(x: torch.Tensor, tp: TPTrainContext) -> torch.Tensor:
    return _TakeRowsGatherGrad.apply(x, tp.group)


def gather_rows_from_sp(x: torch.Tensor, tp: TPTrainContext) -> torch.Tensor:
    return _GatherRowsNoReduce.apply(x, tp.group)


def allreduce_sequence_parallel_grads(model, tp: TPTrainContext) -> None:
    """With sequence parallelism the norm weights see only this rank's block of tokens: add the ranks' gradients
    before the optimizer step (Megatron's ``allreduce_layernorm_grads``)."""
    if not tp.sequence_parallel:
        return
    for name, p in model.named_parameters():
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("input_layernorm", "post_attention_layernorm", "norm", "q_norm", "k_norm"):
            g = getattr(p, "main_grad", None)
            if g is None:
                g = p.grad
            if g is not None:
                if p.grad is not None and g is not p.grad and p.grad.data_ptr() != g.data_ptr():
                    g.add_(p.grad.to(g.dtype))     # fold what plain autograd left on the parameter
                    p.grad = None
                dist.all_reduce(g, group=tp.group)


class _GatherRowsNoReduce(torch.autograd.Function):
    """All-gather of token rows whose backward keeps this rank's block (the consumer is replicated computation:
    every rank derives the same loss from the gathered tensor)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _all_gather_rows(x, group)

    @staticmethod
    def backward(ctx, g):
        n, r = dist.get_world_size(ctx.group), dist.get_rank(ctx.group)
        rows = g.shape[0] // n
        return g[r * rows:(r + 1) * rows].contiguous(), None


# ---------------------------------------------------------------------------------------------------------------------
# sharding a decoder
# ---------------------------------------------------------------------------------------------------------------------
def _rows_qkv(cfg, rank: int, size: int) -> torch.Tensor:
    D = cfg.head_dim
    hq, hk = cfg.num_heads // size, cfg.num_kv_heads // size
    q0, k0, v0 = 0, cfg.num_heads * D, (cfg.num_heads + cfg.num_kv_heads) * D
    return torch.cat([torch.arange(q0 + rank * hq * D, q0 + (rank + 1) * hq * D),
                      torch.arange(k0 + rank * hk * D, k0 + (rank + 1) * hk * D),
                      torch.arange(v0 + rank * hk * D, v0 + (rank + 1) * hk * D)])


def _rows_gate_up(cfg, rank: int, size: int) -> torch.Tensor:
    I = cfg.intermediate_size
    Il = I // size
    return torch.cat([torch.arange(rank * Il, (rank + 1) * Il), torch.arange(I + rank * Il, I + (rank + 1) * Il)])


def shard_decoder(model, tp: TPTrainContext, vocab_parallel: bool = False) -> None:
    """Replace the parameters of ``model`` by this rank's tensor-parallel slices (in place; call it right after the
    model was built or loaded, before any parameter store is created).  ``vocab_parallel`` also splits the LM head by
    vocabulary rows (a trainer-only model: a rollout engine sampling from the same module needs the whole head)."""
    import copy
    cfg = model.cfg
    n = tp.size
    if n == 1:
        return
    if cfg.is_moe:
        raise NotImplementedError("tensor-parallel training of MoE layers: use expert parallelism")
    if cfg.num_heads % n or cfg.num_kv_heads % n or cfg.intermediate_size % (8 * n):
        raise ValueError(f"tensor_model_parallel_size={n} must divide heads ({cfg.num_heads}/{cfg.num_kv_heads}) and "
                         f"intermediate_size / 8 ({cfg.intermediate_size})")
    dev = model.embed_tokens.device
    D = cfg.head_dim
    hq, Il = cfg.num_heads // n, cfg.intermediate_size // n
    qkv_rows = _rows_qkv(cfg, tp.rank, n).to(dev)
    gu_rows = _rows_gate_up(cfg, tp.rank, n).to(dev)
    local = copy.copy(cfg)
    local.num_heads, local.num_kv_heads = cfg.num_heads // n, cfg.num_kv_heads // n
    local.intermediate_size = Il
    with torch.no_grad():
        for layer in model.layers:
            def keep(name, t):
                old = getattr(layer, name)
                setattr(layer, name, nn.Parameter(t.contiguous().clone(), requires_grad=old.requires_grad))
            keep("qkv_proj_weight", layer.qkv_proj_weight.data.index_select(0, qkv_rows))
            if layer.qkv_proj_bias is not None:
                keep("qkv_proj_bias", layer.qkv_proj_bias.data.index_select(0, qkv_rows))
            keep("o_proj_weight", layer.o_proj_weight.data[:, tp.rank * hq * D:(tp.rank + 1) * hq * D])
            keep("gate_up_proj_weight", layer.gate_up_proj_weight.data.index_select(0, gu_rows))
            keep("down_proj_weight", layer.down_proj_weight.data[:, tp.rank * Il:(tp.rank + 1) * Il])
            layer.tp = tp
            layer.full_cfg = cfg
            layer.cfg = local
        if vocab_parallel and model.lm_head is not None and cfg.vocab_size % n == 0 and not cfg.value_head:
            V = cfg.vocab_size // n
            model.lm_head = nn.Parameter(model.lm_head.data[tp.rank * V:(tp.rank + 1) * V].contiguous().clone(),
                                         requires_grad=model.lm_head.requires_grad)
            model.vocab_range = (tp.rank * V, (tp.rank + 1) * V)
    model.tp = tp
    model.full_cfg = cfg


def per_tensor_generator(model, tp: TPTrainContext) -> Iterator[Tuple[str, torch.Tensor]]:
    """``(name, full tensor)`` of every parameter of a sharded decoder, gathered across the tensor-parallel group one
    tensor at a time (a collective: every rank of the group iterates in the same order)."""
    cfg = getattr(model, "full_cfg", model.cfg)
    n = tp.size

    def gather(t: torch.Tensor) -> List[torch.Tensor]:
        parts = [torch.empty_like(t) for _ in range(n)]
        dist.all_gather(parts, t.contiguous(), group=tp.group)
        return parts

    D = cfg.head_dim
    hq, hk, Il = cfg.num_heads // n, cfg.num_kv_heads // n, cfg.intermediate_size // n
    for name, p in model.named_parameters():
        t = p.data
        leaf = name.rsplit(".", 1)[-1]
        if n == 1 or not name.startswith("layers.") and leaf != "lm_head":
            yield name, t
        elif leaf in ("qkv_proj_weight", "qkv_proj_bias"):
            parts = gather(t)
            q = torch.cat([x[: hq * D] for x in parts], 0)
            k = torch.cat([x[hq * D:(hq + hk) * D] for x in parts], 0)
            v = torch.cat([x[(hq + hk) * D:] for x in parts], 0)
            yield name, torch.cat([q, k, v], 0)
        elif leaf == "gate_up_proj_weight":
            parts = gather(t)
            yield name, torch.cat([x[:Il] for x in parts] + [x[Il:] for x in parts], 0)
        elif leaf in ("o_proj_weight", "down_proj_weight"):
            yield name, torch.cat(gather(t), 1)
        elif leaf == "lm_head" and hasattr(model, "vocab_range"):
            yield name, torch.cat(gather(t), 0)
        else:
            yield name, t


# ---------------------------------------------------------------------------------------------------------------------
# vocabulary-parallel log-prob + entropy
# ---------------------------------------------------------------------------------------------------------------------
def _local_stats(hidden: torch.Tensor, w: torch.Tensor, labels_local: torch.Tensor, inv_t: float):
    """Per token over this rank's vocabulary rows: (max, sum exp(z - max), sum exp(z - max) * z, z[label] or -inf)."""
    z = F.linear(hidden.float(), w.float()) * inv_t
    m = z.max(-1).values
    e = torch.exp(z - m[:, None])
    s, t = e.sum(-1), (e * z).sum(-1)
    ok = (labels_local >= 0) & (labels_local < w.shape[0])
    zl = torch.where(ok, z.gather(-1, labels_local.clamp(0, w.shape[0] - 1)[:, None]).squeeze(-1),
                     torch.full_like(m, float("-inf")))
    return torch.stack([m, s, t, zl], -1)


class _VocabParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, vocab_start, temperature, group):
        T = hidden.shape[0]
        V = weight.shape[0]
        inv_t = 1.0 / temperature
        local_labels = labels.to(torch.int64) - vocab_start
        local_labels = torch.where((local_labels >= 0) & (local_labels < V), local_labels,
                                   torch.full_like(local_labels, -1))
        if hidden.is_cuda and V % 8 == 0:
            # the fused vocabulary GEMM: per-tile statistics from TMEM, then one merge over this rank's tiles
            import ctypes

            from ..ops import lib as _lib
            L = _lib.get_lib()
            tiles = (V + 255) // 256
            partial = torch.empty(T * tiles * 4, dtype=torch.float32, device=hidden.device)
            ll, f = ctypes.c_longlong, ctypes.c_float
            h = hidden.contiguous()
            _lib.check(L.sb_gemm_lmstat_bf16(_lib.ptr(h), _lib.ptr(weight), T, V, h.shape[1], ll(h.stride(0)),
                                             ll(weight.stride(0)), _lib.ptr(local_labels), f(inv_t), _lib.ptr(partial),
                                             _lib.ptr(_lib.status_word(hidden.device)), _lib.stream()),
                       "sb_gemm_lmstat_bf16")
            p4 = partial.view(T, tiles, 4)
            m = p4[..., 0].max(-1).values
            sc = torch.exp(p4[..., 0] - m[:, None])
            stats = torch.stack([m, (p4[..., 1] * sc).sum(-1), (p4[..., 2] * sc).sum(-1), p4[..., 3].max(-1).values], -1)
        else:
            stats = _local_stats(hidden, weight, local_labels, inv_t)
        n = dist.get_world_size(group)
        allst = [torch.empty_like(stats) for _ in range(n)]
        dist.all_gather(allst, stats.contiguous(), group=group)
        a = torch.stack(allst, 0)                               # [tp, T, 4]
        m = a[..., 0].max(0).values
        sc = torch.exp(a[..., 0] - m[None])
        s, t = (a[..., 1] * sc).sum(0), (a[..., 2] * sc).sum(0)
        zl = a[..., 3].max(0).values
        lse = m + torch.log(s)
        logp = torch.where(torch.isfinite(zl), zl - lse, torch.zeros_like(lse))
        ent = lse - t / s
        ctx.save_for_backward(hidden, weight, local_labels, lse, ent)
        ctx.valid = torch.isfinite(zl)          # the target id exists in some rank's slice (not an ignored token)
        ctx.meta = (inv_t, group)
        ctx.weight_ref = weight
        return logp, ent

    @staticmethod
    def backward(ctx, g_logp, g_ent):
        hidden, weight, local_labels, lse, ent = ctx.saved_tensors
        inv_t, group = ctx.meta
        V = weight.shape[0]
        g_logp = g_logp.float()
        g_ent = g_ent.float() if g_ent is not None else torch.zeros_like(g_logp)
        mg = getattr(ctx.weight_ref, "main_grad", None)
        T, H = hidden.shape
        if hidden.is_cuda and V % 8 == 0:
            import ctypes

            from ..ops import dense
            from ..ops import lib as _lib
            L = _lib.get_lib()
            ll, f = ctypes.c_longlong, ctypes.c_float
            # targets of other ranks' slices are marked -2: their softmax term still contributes here
            lab = torch.where(local_labels >= 0, local_labels, torch.where(ctx.valid, torch.full_like(local_labels, -2),
                                                                           torch.full_like(local_labels, -1)))
            rows = min(max(128, ((1 << 30) // (2 * V)) // 128 * 128), max(T, 1))
            dl_buf = torch.empty(rows, V, dtype=torch.bfloat16, device=hidden.device)
            dh = torch.empty(T, H, dtype=hidden.dtype, device=hidden.device)
            dw_acc = mg if mg is not None else torch.zeros(V, H, dtype=torch.float32, device=hidden.device)
            h = hidden.contiguous()
            gl, ge = g_logp.contiguous(), g_ent.contiguous()
            for s0 in range(0, T, rows):
                e0 = min(s0 + rows, T)
                dl = dl_buf[: e0 - s0]
                hs = h[s0:e0]
                _lib.check(L.sb_gemm_dlogits_bf16(_lib.ptr(hs), _lib.ptr(weight), _lib.ptr(dl), e0 - s0, V, H,
                                                  ll(hs.stride(0)), ll(weight.stride(0)), ll(V), _lib.ptr(lab[s0:e0]),
                                                  f(inv_t), _lib.ptr(lse[s0:e0]), _lib.ptr(ent[s0:e0]),
                                                  _lib.ptr(gl[s0:e0]), _lib.ptr(ge[s0:e0]),
                                                  _lib.ptr(_lib.status_word(hidden.device)), _lib.stream()),
                           "sb_gemm_dlogits_bf16")
                dense.gemm(dl, weight, out=dh[s0:e0], b_mn=True)
                dense.gemm(dl, hs, out=dw_acc, a_mn=True, b_mn=True, epi=dense.EPI_F32_ACC)
            dhf = dh.float()
            dist.all_reduce(dhf, group=group)
            dw = None if mg is not None else dw_acc.to(weight.dtype)
            return dhf.to(hidden.dtype), dw, None, None, None, None
        has = local_labels >= 0
        z = F.linear(hidden.float(), weight.float()) * inv_t
        p = torch.exp(z - lse[:, None])
        onehot = torch.zeros_like(z)
        onehot[has, local_labels[has]] = 1.0
        dz = (g_logp * ctx.valid)[:, None] * (onehot - p) - g_ent[:, None] * p * (z - lse[:, None] + ent[:, None])
        dlogits = (dz * inv_t).to(hidden.dtype)
        dh = dlogits.float() @ weight.float()
        dist.all_reduce(dh, group=group)                        # every rank holds one vocabulary slice of the sum
        dw = dlogits.float().t() @ hidden.float()
        if mg is not None:
            mg.add_(dw)
            dw = None
        else:
            dw = dw.to(weight.dtype)
        return dh.to(hidden.dtype), dw, None, None, None, None


def vocab_parallel_logprob_entropy(hidden: torch.Tensor, weight_shard: torch.Tensor, labels: torch.Tensor,
                                   vocab_start: int, group, temperature: float = 1.0
                                   ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``log p(label)`` and entropy per token when the vocabulary rows of the LM head are split over ``group``
    (``weight_shard`` = rows ``[vocab_start, vocab_start + V_local)``); ``hidden`` and ``labels`` are the same on every
    rank of the group.  Equals ``lm_head_logprob_entropy`` on the gathered weight."""
    return _VocabParallelFn.apply(hidden, weight_shard, labels, int(vocab_start), float(temperature), group)
