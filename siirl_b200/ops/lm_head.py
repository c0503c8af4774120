"""Fused LM-head log-prob + entropy: ``(logp[T], entropy[T]) = f(hidden[T,H], weight[V,H], labels[T])``.

Forward: the vocabulary GEMM (tcgen05, 128 x 256 tiles) reduces every row of every tile to online-softmax partial
statistics in its epilogue -- (max, sum exp, sum exp * z, z[label]) read from the accumulator in TMEM -- and writes
only those ``[T, V / 256]`` partials; a merge kernel folds them into log p(label), entropy and log-sum-exp.  No
logits reach memory.  Backward recomputes the GEMM with an epilogue that writes the bf16 gradient of the logits
directly (from the saved log-sum-exp / entropy and the incoming gradients), chunk by chunk, and feeds the two gradient
GEMMs (``d_weight`` accumulates in fp32 in the GEMM epilogue).  API and semantics of the reference's
``linear_cross_entropy`` (siirl/utils/kernel/linear_cross_entropy.py:40-117; kernels siirl/utils/kernel/kernels.py:
153-287 forward, 1263-1375 backward): logits are divided by ``temperature`` first.

``FUSED_EPILOGUE = False`` selects the earlier two-kernel form (fp32 logits chunk in memory, then a row-reduction
kernel), kept as the comparison point of ``benchmarks/kernels.py``."""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from . import dense
from . import lib as _lib
from . import reference as ref

_f = ctypes.c_float
FUSED_EPILOGUE = True
_TILE_V = 256           # vocabulary columns per GEMM tile of the fused epilogues


def _chunk_rows(V: int, budget_bytes: int = 1 << 30) -> int:
    rows = max(128, (budget_bytes // (4 * V)) // 128 * 128)
    return rows


class _LmHeadFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, labels, temperature, with_entropy):
        L = _lib.get_lib()
        T, H = hidden.shape
        V = weight.shape[0]
        inv_t = 1.0 / temperature
        labels = labels.to(torch.int64).contiguous()
        logp = torch.empty(T, dtype=torch.float32, device=hidden.device)
        ent = torch.empty(T, dtype=torch.float32, device=hidden.device) if with_entropy else None
        lse = torch.empty(T, dtype=torch.float32, device=hidden.device)
        ctx.fused = bool(FUSED_EPILOGUE and V % 8 == 0)
        if ctx.fused:
            tiles = (V + _TILE_V - 1) // _TILE_V
            rows = min(16384, max(T, 1))
            partial = torch.empty(rows * tiles * 4, dtype=torch.float32, device=hidden.device)
            ll = ctypes.c_longlong
            for s in range(0, T, rows):
                e = min(s + rows, T)
                h = hidden[s:e]
                _lib.check(L.sb_gemm_lmstat_bf16(_lib.ptr(h), _lib.ptr(weight), e - s, V, H, ll(h.stride(0)),
                                                 ll(weight.stride(0)), _lib.ptr(labels[s:e]), _f(inv_t),
                                                 _lib.ptr(partial), _lib.ptr(_lib.status_word(hidden.device)),
                                                 _lib.stream()), "sb_gemm_lmstat_bf16")
                _lib.check(L.sb_lmhead_merge(_lib.ptr(partial), tiles, _lib.ptr(labels[s:e]), _lib.ptr(logp[s:e]),
                                             _lib.ptr(ent[s:e] if ent is not None else None), _lib.ptr(lse[s:e]),
                                             e - s, V, _lib.stream()), "sb_lmhead_merge")
            rows = min(max(128, ((1 << 30) // (2 * V)) // 128 * 128), max(T, 1))    # backward: bf16 d_logits chunk
        else:
            rows = min(_chunk_rows(V), max(T, 1))
            logits = torch.empty(rows, V, dtype=torch.float32, device=hidden.device)
        for s in (range(0, T, rows) if not ctx.fused else ()):
            e = min(s + rows, T)
            lg = logits[: e - s]
            dense.gemm(hidden[s:e], weight, out=lg, epi=dense.EPI_F32)
            _lib.check(L.sb_lmhead_stats(_lib.ptr(lg), ctypes.c_longlong(V), _lib.ptr(labels[s:e]), _f(inv_t),
                                         _lib.ptr(logp[s:e]), _lib.ptr(ent[s:e] if ent is not None else None),
                                         _lib.ptr(lse[s:e]), e - s, V, _lib.stream()), "sb_lmhead_stats")
        ctx.save_for_backward(hidden, weight, labels, lse, ent if ent is not None else lse)
        ctx.weight_ref = weight
        ctx.meta = (inv_t, with_entropy, rows)
        if ent is None:
            ent = torch.zeros(0, device=hidden.device)
            ctx.mark_non_differentiable(ent)
        return logp, ent

    @staticmethod
    def backward(ctx, g_logp, g_ent):
        hidden, weight, labels, lse, ent = ctx.saved_tensors
        inv_t, with_entropy, rows = ctx.meta
        L = _lib.get_lib()
        T, H = hidden.shape
        V = weight.shape[0]
        g_logp = g_logp.float().contiguous()
        g_ent = g_ent.float().contiguous() if (with_entropy and g_ent is not None and g_ent.numel() == T) else None
        dh = torch.empty_like(hidden) if ctx.needs_input_grad[0] else None
        mg = getattr(ctx.weight_ref, "main_grad", None)
        need_dw = ctx.needs_input_grad[1]
        dw_acc = mg if mg is not None else (torch.zeros(V, H, dtype=torch.float32, device=hidden.device)
                                            if need_dw else None)
        logits = None if ctx.fused else torch.empty(rows, V, dtype=torch.float32, device=hidden.device)
        dlogits = torch.empty(rows, V, dtype=torch.bfloat16, device=hidden.device)
        ll = ctypes.c_longlong
        for s in range(0, T, rows):
            e = min(s + rows, T)
            dl = dlogits[: e - s]
            if ctx.fused:
                h = hidden[s:e]
                _lib.check(L.sb_gemm_dlogits_bf16(
                    _lib.ptr(h), _lib.ptr(weight), _lib.ptr(dl), e - s, V, H, ll(h.stride(0)), ll(weight.stride(0)),
                    ll(V), _lib.ptr(labels[s:e]), _f(inv_t), _lib.ptr(lse[s:e]),
                    _lib.ptr(ent[s:e] if with_entropy else None), _lib.ptr(g_logp[s:e]),
                    _lib.ptr(g_ent[s:e] if g_ent is not None else None),
                    _lib.ptr(_lib.status_word(hidden.device)), _lib.stream()), "sb_gemm_dlogits_bf16")
            else:
                lg = logits[: e - s]
                dense.gemm(hidden[s:e], weight, out=lg, epi=dense.EPI_F32)
                _lib.check(L.sb_lmhead_dlogits(
                    _lib.ptr(lg), ctypes.c_longlong(V), _lib.ptr(labels[s:e]), _lib.ptr(lse[s:e]),
                    _lib.ptr(ent[s:e] if with_entropy else None), _lib.ptr(g_logp[s:e]),
                    _lib.ptr(g_ent[s:e] if g_ent is not None else None), _f(inv_t), _lib.ptr(dl),
                    ctypes.c_longlong(V), e - s, V, _lib.stream()), "sb_lmhead_dlogits")
            if dh is not None:
                dense.gemm(dl, weight, out=dh[s:e], b_mn=True)
            if need_dw:
                dense.gemm(dl, hidden[s:e], out=dw_acc, a_mn=True, b_mn=True, epi=dense.EPI_F32_ACC)
        dw = None
        if need_dw and mg is None:
            dw = dw_acc.to(weight.dtype)
        return dh, dw, None, None, None


def lm_head_logprob_entropy(hidden: torch.Tensor, weight: torch.Tensor, labels: torch.Tensor,
                            temperature: float = 1.0, with_entropy: bool = True
                            ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """fp32 ``log p(label)`` and (optionally) entropy per token."""
    if not hidden.is_cuda:
        return ref.lm_head_logprob_entropy(hidden, weight, labels, temperature, with_entropy)
    _lib.use_native(hidden)
    logp, ent = _LmHeadFn.apply(hidden.contiguous(), weight, labels, float(temperature), bool(with_entropy))
    return logp, (ent if with_entropy else None)


def lm_head_logits(hidden: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """fp32 logits ``[T, V]`` (decode path: T = number of running sequences)."""
    if not hidden.is_cuda:
        return hidden.float() @ weight.float().t()
    return dense.gemm(hidden.contiguous(), weight, epi=dense.EPI_F32)
