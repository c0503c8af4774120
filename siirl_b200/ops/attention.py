"""Packed variable-length attention (training / log-prob / prefill path).

``qkv`` is one packed buffer ``[T, (Hq + 2*Hkv) * D]`` (q heads | k heads | v heads per token), sequences are
consecutive row ranges described by :class:`SeqInfo`.  CUDA tensors use the tcgen05 kernels of
``csrc/fmha_fwd.cu`` / ``csrc/fmha_bwd.cu``; CPU tensors use the eager statement in ``reference``."""
from __future__ import annotations

import ctypes
import math
from typing import List, Optional, Sequence

import torch

from . import lib as _lib
from . import reference as ref


class SeqInfo:
    """Sequence boundaries of a packed batch plus the 128-row tile lists the attention kernels need."""

    def __init__(self, seqlens: Sequence[int], device=None):
        self.seqlens: List[int] = [int(x) for x in seqlens]
        cu = [0]
        for n in self.seqlens:
            cu.append(cu[-1] + n)
        self.cu_seqlens_cpu = cu
        self.total = cu[-1]
        self.max_seqlen = max(self.seqlens) if self.seqlens else 0
        self.device = device
        self._tiles = None
        self._cu_dev = None
        self._pos = None

    @property
    def cu_seqlens(self) -> torch.Tensor:
        if self._cu_dev is None:
            self._cu_dev = torch.tensor(self.cu_seqlens_cpu, dtype=torch.int32, device=self.device)
        return self._cu_dev

    @property
    def positions(self) -> torch.Tensor:
        """Position of every packed token inside its sequence, int32 ``[T]``."""
        if self._pos is None:
            pos = torch.cat([torch.arange(n, dtype=torch.int32) for n in self.seqlens]) if self.seqlens else \
                torch.zeros(0, dtype=torch.int32)
            self._pos = pos.to(self.device) if self.device is not None else pos
        return self._pos

    def tiles(self, q_start: Optional[Sequence[int]] = None):
        """(seq_start, seq_len, offset) int32 device tensors, one entry per 128-row tile; longest
        sequences' last tiles first so the heaviest causal tiles start early.  ``q_start[i]`` (a multiple of 128)
        leaves out the query tiles of sequence i below that row: chunked prefill computes only the new rows."""
        if q_start is not None:
            start, length, off = [], [], []
            for i, n in enumerate(self.seqlens):
                for t0 in range(int(q_start[i]) // 128 * 128, n, 128):
                    start.append(self.cu_seqlens_cpu[i])
                    length.append(n)
                    off.append(t0)
            order = sorted(range(len(off)), key=lambda k: -off[k])
            mk = lambda xs: torch.tensor([xs[k] for k in order], dtype=torch.int32, device=self.device)  # noqa: E731
            return (mk(start), mk(length), mk(off), len(off))
        if self._tiles is None:
            start, length, off = [], [], []
            for i, n in enumerate(self.seqlens):
                for t0 in range(0, n, 128):
                    start.append(self.cu_seqlens_cpu[i])
                    length.append(n)
                    off.append(t0)
            order = sorted(range(len(off)), key=lambda k: -off[k])
            mk = lambda xs: torch.tensor([xs[k] for k in order], dtype=torch.int32, device=self.device)  # noqa: E731
            self._tiles = (mk(start), mk(length), mk(off), len(off))
        return self._tiles


class _AttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, info: SeqInfo, hq, hkv, d, causal, scale, q_start=None):
        L = _lib.get_lib()
        T = qkv.shape[0]
        out = torch.empty(T, hq * d, dtype=qkv.dtype, device=qkv.device)
        lse = torch.empty(hq, T, dtype=torch.float32, device=qkv.device)
        ts, tl, t0, n = info.tiles(q_start)
        rc = L.sb_fmha_fwd(_lib.ptr(qkv), _lib.ptr(out), _lib.ptr(lse), _lib.ptr(ts), _lib.ptr(tl), _lib.ptr(t0), n, T,
                           hq, hkv, d, int(causal), ctypes.c_float(scale), _lib.ptr(_lib.status_word(qkv.device)),
                           _lib.stream())
        _lib.check(rc, "sb_fmha_fwd")
        ctx.save_for_backward(qkv, out, lse)
        ctx.meta = (info, hq, hkv, d, causal, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        info, hq, hkv, d, causal, scale = ctx.meta
        L = _lib.get_lib()
        T = qkv.shape[0]
        dout = dout.contiguous()
        dqkv = torch.empty_like(qkv)
        delta = torch.empty(hq, T, dtype=torch.float32, device=qkv.device)
        dq_acc = torch.empty(T, hq * d, dtype=torch.float32, device=qkv.device)
        ts, tl, t0, n = info.tiles()
        rc = L.sb_fmha_bwd(_lib.ptr(qkv), _lib.ptr(out), _lib.ptr(dout), _lib.ptr(lse), _lib.ptr(delta),
                           _lib.ptr(dq_acc), _lib.ptr(dqkv), _lib.ptr(ts), _lib.ptr(tl), _lib.ptr(t0), n, T, hq, hkv,
                           d, int(causal), ctypes.c_float(scale), _lib.ptr(_lib.status_word(qkv.device)),
                           _lib.stream())
        _lib.check(rc, "sb_fmha_bwd")
        return dqkv, None, None, None, None, None, None, None


def _pad_heads(qkv: torch.Tensor, n_heads_total: int, d: int, d_pad: int) -> torch.Tensor:
    T = qkv.shape[0]
    x = qkv.reshape(T, n_heads_total, d)
    return torch.nn.functional.pad(x, (0, d_pad - d)).reshape(T, n_heads_total * d_pad)


def attention_packed(qkv: torch.Tensor, info: SeqInfo, n_heads: int, n_kv_heads: int, head_dim: int,
                     causal: bool = True, scale: Optional[float] = None,
                     q_start: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Attention over a packed batch; returns ``[T, n_heads * head_dim]``.  ``q_start`` (inference only): rows of
    sequence i below ``q_start[i] // 128 * 128`` are not computed (their output rows are undefined)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    T = qkv.shape[0]
    if not qkv.is_cuda:
        q, k, v = qkv.split([n_heads * head_dim, n_kv_heads * head_dim, n_kv_heads * head_dim], dim=-1)
        out = ref.attention_varlen(q.reshape(T, n_heads, head_dim), k.reshape(T, n_kv_heads, head_dim),
                                   v.reshape(T, n_kv_heads, head_dim), torch.tensor(info.cu_seqlens_cpu),
                                   causal=causal, scale=scale)
        return out.reshape(T, n_heads * head_dim)
    _lib.use_native(qkv)
    if q_start is not None:
        assert not (torch.is_grad_enabled() and qkv.requires_grad), "q_start is an inference-only option"
    if head_dim in (64, 128):
        return _AttnFn.apply(qkv.contiguous(), info, n_heads, n_kv_heads, head_dim, causal, scale, q_start)
    d_pad = 64 if head_dim < 64 else 128
    assert head_dim <= 128, "head_dim > 128 is not supported"
    padded = _pad_heads(qkv, n_heads + 2 * n_kv_heads, head_dim, d_pad)
    out = _AttnFn.apply(padded, info, n_heads, n_kv_heads, d_pad, causal, scale, q_start)
    return out.reshape(T, n_heads, d_pad)[..., :head_dim].reshape(T, n_heads * head_dim)


def attention_wide_heads(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, info: SeqInfo, causal: bool = True,
                         scale: Optional[float] = None) -> torch.Tensor:
    """Attention with query/key width and value width outside the tcgen05 kernels' set (multi-head latent attention:
    192 / 128).  ``q, k [T, nh, dq]``, ``v [T, nh, dv]`` packed -> ``[T, nh, dv]``.  On GPUs this is a library call
    (the flash-attn variable-length kernel with the values zero-padded to ``dq``, as the reference does in
    siirl/models/transformers/kimi_vl.py:172-221; PyTorch's fused attention per sequence when flash-attn is absent);
    on CPU the eager statement."""
    T, nh, dq = q.shape
    dv = v.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(dq)
    if not q.is_cuda:
        return ref.attention_varlen(q, k, v, torch.tensor(info.cu_seqlens_cpu), causal=causal, scale=scale).to(q.dtype)
    import torch.nn.functional as F
    vp = F.pad(v, (0, dq - dv)) if dv < dq else v
    try:
        from flash_attn import flash_attn_varlen_func
        cu = torch.tensor(info.cu_seqlens_cpu, dtype=torch.int32, device=q.device)
        mx = max(info.seqlens) if len(info.seqlens) else 0
        out = flash_attn_varlen_func(q, k, vp, cu, cu, mx, mx, softmax_scale=scale, causal=causal)
    except ImportError:
        outs, at = [], 0
        for n in info.seqlens:
            o = F.scaled_dot_product_attention(q[at:at + n].transpose(0, 1)[None], k[at:at + n].transpose(0, 1)[None],
                                               vp[at:at + n].transpose(0, 1)[None], is_causal=causal, scale=scale)
            outs.append(o[0].transpose(0, 1))
            at += n
        out = torch.cat(outs) if outs else q.new_zeros(0, nh, dq)
    return out[..., :dv]
