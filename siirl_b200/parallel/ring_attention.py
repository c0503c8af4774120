"""Ring (context-parallel) causal attention over peer memory.

Every sequence of the packed batch is cut into ``cp`` equal chunks; rank r holds chunk r of every sequence (its
``qkv`` rows and a ``SeqInfo`` of the chunk lengths, identical on all ranks).  Causality means rank r attends to
the K/V chunks of ranks 0..r.  The reference gets this from Megatron-core / Transformer-Engine's NCCL send/recv
ring (``context_parallel_size`` in siirl/params/model_args.py, MegatronArguments).  Here a rank publishes its
``qkv`` rows in symmetric memory once and every consumer pulls the K/V columns of the chunk it needs with one
strided peer-load kernel (``sb_block_pull``), on a side stream while the tcgen05 attention kernel works on the
previous chunk; partial results are merged with their log-sum-exp.  The backward recomputes block by block with the
FINAL ``out`` / ``lse`` (as flash attention does), accumulates dQ locally and returns dK/dV of remote chunks to
their owners through a second pull.

Two chunk assignments:

* contiguous (``zigzag=False``): rank r holds chunk r of ``cp`` and does r + 1 blocks of work: the last rank sets the
  pace with ``cp`` blocks while rank 0 does one.
* zig-zag (``zigzag=True``, the balanced assignment Megatron-core / Transformer-Engine use): every sequence is cut into
  ``2 cp`` chunks and rank r holds chunks r ("low") and ``2 cp - 1 - r`` ("high"), stored one after the other.  Its
  own pair is one causal block over the concatenation; against a rank j < r all local queries see j's low chunk only;
  against a rank j > r only the high queries see anything, and they see both of j's chunks.  Every remote step is two
  ``c x c`` unmasked blocks, so all ranks do the same ``2 cp + 1`` half-blocks of work.
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import lib as _lib
from ..ops.attention import SeqInfo
from .ulysses import _PullBlock


def _eager_blocks(qkv, info: SeqInfo, hq, hkv, d, causal, scale):
    """Per sequence: (row range, q, k, v as fp32 ``[n, hq, d]``, scores ``[hq, n, n]`` with the mask applied)."""
    cu = info.cu_seqlens_cpu
    rep = hq // hkv
    for i in range(len(cu) - 1):
        a, b = cu[i], cu[i + 1]
        if b == a:
            continue
        q, k, v = qkv[a:b].float().split([hq * d, hkv * d, hkv * d], dim=-1)
        q = q.reshape(b - a, hq, d)
        k = k.reshape(b - a, hkv, d).repeat_interleave(rep, dim=1)
        v = v.reshape(b - a, hkv, d).repeat_interleave(rep, dim=1)
        sc = torch.einsum("qhd,khd->hqk", q, k) * scale
        if causal:
            keep = torch.ones(b - a, b - a, dtype=torch.bool, device=qkv.device).tril()
            sc = sc.masked_fill(~keep[None], float("-inf"))
        yield a, b, q, k, v, sc


def _block_fwd(qkv, info: SeqInfo, hq, hkv, d, causal, scale) -> Tuple[torch.Tensor, torch.Tensor]:
    T = qkv.shape[0]
    if not qkv.is_cuda:                                  # eager statement of the kernel (same outputs: out, lse)
        out = torch.zeros(T, hq * d, dtype=qkv.dtype)
        lse = torch.zeros(hq, T, dtype=torch.float32)
        for a, b, q, k, v, sc in _eager_blocks(qkv, info, hq, hkv, d, causal, scale):
            lse[:, a:b] = torch.logsumexp(sc, dim=-1)
            out[a:b] = torch.einsum("hqk,khd->qhd", torch.softmax(sc, -1), v).reshape(b - a, hq * d).to(qkv.dtype)
        return out, lse
    L = _lib.get_lib()
    out = torch.empty(T, hq * d, dtype=qkv.dtype, device=qkv.device)
    lse = torch.empty(hq, T, dtype=torch.float32, device=qkv.device)
    ts, tl, t0, n = info.tiles()
    _lib.check(L.sb_fmha_fwd(_lib.ptr(qkv), _lib.ptr(out), _lib.ptr(lse), _lib.ptr(ts), _lib.ptr(tl), _lib.ptr(t0), n,
                             T, hq, hkv, d, int(causal), ctypes.c_float(scale),
                             _lib.ptr(_lib.status_word(qkv.device)), _lib.stream()), "sb_fmha_fwd")
    return out, lse


def _block_bwd(qkv, out, lse, dout, info: SeqInfo, hq, hkv, d, causal, scale) -> torch.Tensor:
    T = qkv.shape[0]
    if not qkv.is_cuda:          # flash-attention backward with the FINAL out / lse: P = exp(S - lse), dS = P (dP - delta)
        dqkv = torch.zeros_like(qkv)
        rep = hq // hkv
        for a, b, q, k, v, sc in _eager_blocks(qkv, info, hq, hkv, d, causal, scale):
            n = b - a
            p = torch.exp(sc - lse[:, a:b, None])
            do = dout[a:b].float().reshape(n, hq, d)
            delta = (do * out[a:b].float().reshape(n, hq, d)).sum(-1).t()          # [hq, n]
            dv = torch.einsum("hqk,qhd->khd", p, do)
            ds = p * (torch.einsum("qhd,khd->hqk", do, v) - delta[:, :, None])
            dq = torch.einsum("hqk,khd->qhd", ds, k) * scale
            dk = torch.einsum("hqk,qhd->khd", ds, q) * scale
            dk = dk.reshape(n, hkv, rep, d).sum(2)
            dv = dv.reshape(n, hkv, rep, d).sum(2)
            dqkv[a:b] = torch.cat([dq.reshape(n, -1), dk.reshape(n, -1), dv.reshape(n, -1)], -1).to(qkv.dtype)
        return dqkv
    L = _lib.get_lib()
    dqkv = torch.empty_like(qkv)
    delta = torch.empty(hq, T, dtype=torch.float32, device=qkv.device)
    dq_acc = torch.empty(T, hq * d, dtype=torch.float32, device=qkv.device)
    ts, tl, t0, n = info.tiles()
    _lib.check(L.sb_fmha_bwd(_lib.ptr(qkv), _lib.ptr(out), _lib.ptr(dout), _lib.ptr(lse), _lib.ptr(delta),
                             _lib.ptr(dq_acc), _lib.ptr(dqkv), _lib.ptr(ts), _lib.ptr(tl), _lib.ptr(t0), n, T, hq, hkv,
                             d, int(causal), ctypes.c_float(scale), _lib.ptr(_lib.status_word(qkv.device)),
                             _lib.stream()), "sb_fmha_bwd")
    return dqkv


class RingContext:
    """Symmetric staging of one context-parallel group: two alternating ``qkv`` buffers and the dK/dV return slots.

    ``comm``: the group's symmetric-memory communicator (GPUs).  ``emulate=True`` (CPU ranks under ``gloo``) stands in
    for it with all-gathers: publishing a buffer hands every rank a copy of every rank's instance, and a "pull" reads
    from that copy, so the block algorithms below run unchanged where there is no peer memory."""

    def __init__(self, group, comm=None, max_rows: int = 0, qkv_width: int = 0, kv_width: int = 0,
                 zigzag: bool = False, emulate: bool = False):
        self.group, self.comm = group, comm
        self.zigzag = bool(zigzag)
        self.cp = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.stage = None
        self.emulate = bool(emulate) and comm is None and self.cp > 1
        if comm is not None and self.cp > 1:
            self.stage = [comm.alloc(max_rows * qkv_width, torch.bfloat16) for _ in range(2)]
            self.gstage = comm.alloc(self.cp * max_rows * kv_width, torch.bfloat16)
            self._turn = 0
            comm.barrier()
        elif self.emulate:
            self.stage = [None, None]
            self._turn = 0
            self._copies = {}
            self._slot = (max_rows, kv_width)
            self.gstage = None

    # ---- publication ----------------------------------------------------------------------------------------------
    def _gather(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty(self.cp * x.numel(), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous().reshape(-1), group=self.group)
        return out.view(self.cp, -1)

    def publish(self, x: torch.Tensor) -> torch.Tensor:
        """Make ``x`` readable by the group; returns the handle to pass to ``pull_blocks``."""
        if self.emulate:
            buf = x.detach().reshape(-1).clone()
            self._copies = {id(buf): self._gather(buf)}
            return buf
        buf = self.stage[self._turn]
        self._turn ^= 1
        buf[: x.numel()].copy_(x.reshape(-1))
        self.comm.barrier()
        return buf

    def return_slots(self, like: torch.Tensor) -> torch.Tensor:
        """``[cp, slot]`` buffer of the gradient return: slot s is read by the rank ``s`` places below."""
        if self.emulate:
            rows, kvw = self._slot
            self.gstage = torch.zeros(self.cp * max(rows, like.shape[0]) * kvw, dtype=like.dtype, device=like.device)
        return self.gstage.view(self.cp, -1)

    def returns_written(self) -> None:
        if self.emulate:
            self._copies[id(self.gstage)] = self._gather(self.gstage)
        else:
            self.comm.barrier()

    def returns_read(self) -> None:
        """The return slots may be rewritten from here on."""
        if self.emulate:
            self._copies.pop(id(self.gstage), None)
        else:
            self.comm.barrier()

    def pull_cols(self, buf: torch.Tensor, src_rank: int, out: torch.Tensor, src_off_elems: int, dst_off_elems: int,
                  src_pitch: int, dst_pitch: int, rows: int, cols: int) -> None:
        """Copy ``rows x cols`` bf16 elements from ``src_rank``'s instance of ``buf`` into ``out``."""
        self.pull_blocks(buf, out, [(src_rank, src_off_elems, dst_off_elems, src_pitch, dst_pitch, rows, cols)])

    def pull_blocks(self, buf: torch.Tensor, out: torch.Tensor, blocks) -> None:
        """``blocks``: (source rank, source offset, destination offset, source pitch, destination pitch, rows,
        columns), all in elements; launched 64 blocks at a time."""
        if self.emulate:
            flat = out.view(-1)
            for r, so, do, sp_, dp_, rows, cols in blocks:
                src = self._copies[id(buf)][r]
                flat.as_strided((rows, cols), (dp_, 1), flat.storage_offset() + do).copy_(
                    src.as_strided((rows, cols), (sp_, 1), src.storage_offset() + so))
            return
        L = _lib.get_lib()
        peers = self.comm.peers_of(buf).ptr_array
        for at in range(0, len(blocks), 64):
            part = blocks[at:at + 64]
            arr = (_PullBlock * len(part))()
            for i, (r, so, do, sp_, dp_, rows, cols) in enumerate(part):
                arr[i] = _PullBlock(so * 2, do * 2, sp_ * 2, dp_ * 2, rows, cols * 2, r, 0)
            _lib.check(L.sb_block_pull(peers, self.cp, arr, len(part), _lib.ptr(out), _lib.stream()), "sb_block_pull")


class _Side:
    """The copy stream of the ring: a CUDA side stream on GPUs, the caller's own order on CPU."""

    def __init__(self, device):
        self.stream = torch.cuda.Stream() if device.type == "cuda" else None

    def run(self, fn):
        """Run ``fn()`` (returns a tensor) on the side stream; returns (tensor, event or None)."""
        if self.stream is None:
            return fn(), None
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            blk = fn()
            ev = torch.cuda.Event()
            ev.record(self.stream)
        blk.record_stream(torch.cuda.current_stream())
        return blk, ev

    @staticmethod
    def wait(ev) -> None:
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)


def _merge(out, lse, o_s, lse_s):
    """Log-sum-exp merge of two partial attention results (``lse`` is ``[heads, T]``, outputs ``[T, heads*d]``)."""
    new = torch.logaddexp(lse, lse_s)
    T, hq = out.shape[0], lse.shape[0]
    wa = torch.exp(lse - new).t().reshape(T, hq, 1)
    wb = torch.exp(lse_s - new).t().reshape(T, hq, 1)
    merged = out.float().reshape(T, hq, -1) * wa + o_s.float().reshape(T, hq, -1) * wb
    return merged.reshape(T, -1).to(out.dtype), new


class _RingAttn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, rc: RingContext, info: SeqInfo, hq, hkv, d, scale):
        me = rc.rank
        Tl, W = qkv.shape
        qw, kvw = hq * d, 2 * hkv * d
        buf = rc.publish(qkv)
        side = _Side(qkv.device)
        out, lse = _block_fwd(qkv, info, hq, hkv, d, True, scale)        # own chunk: causal
        nxt = None
        for s in range(1, me + 1):
            if nxt is None:
                nxt = _fetch(rc, buf, qkv, me - s, Tl, W, qw, kvw, side)
            blk, ev = nxt
            _Side.wait(ev)
            nxt = _fetch(rc, buf, qkv, me - s - 1, Tl, W, qw, kvw, side) if s < me else None
            o_s, lse_s = _block_fwd(blk, info, hq, hkv, d, False, scale)  # earlier chunk: every key is visible
            out, lse = _merge(out, lse, o_s, lse_s)
        ctx.save_for_backward(qkv, out, lse)
        ctx.meta = (rc, info, hq, hkv, d, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        rc, info, hq, hkv, d, scale = ctx.meta
        me, n = rc.rank, rc.cp
        Tl, W = qkv.shape
        qw, kvw = hq * d, 2 * hkv * d
        dout = dout.contiguous()
        buf = rc.publish(qkv)
        side = _Side(qkv.device)
        g = _block_bwd(qkv, out, lse, dout, info, hq, hkv, d, True, scale)
        dq = g[:, :qw].float()
        dkv = g[:, qw:].float()
        gs = rc.return_slots(qkv)
        nxt = None
        for s in range(1, me + 1):
            if nxt is None:
                nxt = _fetch(rc, buf, qkv, me - s, Tl, W, qw, kvw, side)
            blk, ev = nxt
            _Side.wait(ev)
            nxt = _fetch(rc, buf, qkv, me - s - 1, Tl, W, qw, kvw, side) if s < me else None
            g = _block_bwd(blk, out, lse, dout, info, hq, hkv, d, False, scale)
            dq += g[:, :qw].float()
            gs[s, : Tl * kvw].copy_(g[:, qw:].reshape(-1))               # slot s: gradient for the chunk of rank me - s
        rc.returns_written()
        tmp = torch.empty(Tl, kvw, dtype=qkv.dtype, device=qkv.device)
        for s in range(1, n - me):                                       # rank me + s used my chunk at its step s
            rc.pull_cols(rc.gstage, me + s, tmp, s * gs.shape[1], 0, kvw, kvw, Tl, kvw)
            dkv += tmp.float()
        rc.returns_read()
        return torch.cat([dq, dkv], dim=1).to(qkv.dtype), None, None, None, None, None, None


def _halves(info: SeqInfo, device):
    """Zig-zag layout: a rank's rows of sequence i are its low chunk then its high chunk (``c_i`` rows each).
    Returns (row indices of the low halves, of the high halves, the ``SeqInfo`` of the ``c_i, c_i, ...`` half
    blocks, per-sequence (first row, c_i))."""
    lo, hi, lens, spans, at = [], [], [], [], 0
    for n in info.seqlens:
        assert n % 2 == 0, "zig-zag chunks come in pairs"
        c = n // 2
        lo.append(torch.arange(at, at + c))
        hi.append(torch.arange(at + c, at + n))
        lens += [c, c]
        spans.append((at, c))
        at += n
    cat = lambda xs: (torch.cat(xs) if xs else torch.zeros(0, dtype=torch.int64)).to(device)  # noqa: E731
    return cat(lo), cat(hi), SeqInfo(lens, device=device), spans


def _fetch_zigzag(rc: RingContext, buf, qkv, src: int, lo, hi, spans, W: int, qw: int, kvw: int, side):
    """Block against rank ``src`` in the zig-zag layout (on a side stream).  ``src`` below this rank: the local
    queries, with ``src``'s low-chunk K/V under both halves.  ``src`` above: the high queries under both halves, with
    ``src``'s K/V as they lie."""
    def fill():
        if src < rc.rank:
            blk = qkv.detach().clone()
            blocks = []
            for at, c in spans:
                if c:
                    blocks.append((src, at * W + qw, at * W + qw, W, W, c, kvw))
                    blocks.append((src, at * W + qw, (at + c) * W + qw, W, W, c, kvw))
            rc.pull_blocks(buf, blk, blocks)
        else:
            dup = torch.empty(qkv.shape[0], dtype=torch.int64, device=qkv.device)
            dup[lo] = hi
            dup[hi] = hi
            blk = qkv.detach().index_select(0, dup)
            rc.pull_blocks(buf, blk, [(src, qw, qw, W, W, qkv.shape[0], kvw)])
        return blk
    return side.run(fill)


class _RingAttnZigzag(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, rc: RingContext, info: SeqInfo, hq, hkv, d, scale):
        me, n = rc.rank, rc.cp
        Tl, W = qkv.shape
        qw, kvw = hq * d, 2 * hkv * d
        lo, hi, info_h, spans = _halves(info, qkv.device)
        buf = rc.publish(qkv)
        side = _Side(qkv.device)
        out, lse = _block_fwd(qkv, info, hq, hkv, d, True, scale)        # own pair of chunks: one causal block
        order = [(me - s) % n for s in range(1, n)]
        nxt = _fetch_zigzag(rc, buf, qkv, order[0], lo, hi, spans, W, qw, kvw, side) if order else None
        for k, j in enumerate(order):
            blk, ev = nxt
            _Side.wait(ev)
            nxt = (_fetch_zigzag(rc, buf, qkv, order[k + 1], lo, hi, spans, W, qw, kvw, side)
                   if k + 1 < len(order) else None)
            o_s, lse_s = _block_fwd(blk, info_h, hq, hkv, d, False, scale)
            if j < me:
                out, lse = _merge(out, lse, o_s, lse_s)
            else:                                                        # both halves hold partials of the high queries
                o_h, l_h = _merge(out[hi], lse[:, hi], o_s[lo], lse_s[:, lo])
                o_h, l_h = _merge(o_h, l_h, o_s[hi], lse_s[:, hi])
                out = out.index_copy(0, hi, o_h)
                lse = lse.index_copy(1, hi, l_h)
        ctx.save_for_backward(qkv, out, lse)
        ctx.meta = (rc, info, hq, hkv, d, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        rc, info, hq, hkv, d, scale = ctx.meta
        me, n = rc.rank, rc.cp
        Tl, W = qkv.shape
        qw, kvw = hq * d, 2 * hkv * d
        lo, hi, info_h, spans = _halves(info, qkv.device)
        dout = dout.contiguous()
        buf = rc.publish(qkv)
        side = _Side(qkv.device)
        g = _block_bwd(qkv, out, lse, dout, info, hq, hkv, d, True, scale)
        dq = g[:, :qw].float()
        dkv = g[:, qw:].float()
        gs = rc.return_slots(qkv)
        dup = torch.empty(Tl, dtype=torch.int64, device=qkv.device)
        dup[lo] = hi
        dup[hi] = hi
        out_h = lse_h = dout_h = None
        order = [(me - s) % n for s in range(1, n)]
        nxt = _fetch_zigzag(rc, buf, qkv, order[0], lo, hi, spans, W, qw, kvw, side) if order else None
        for k, j in enumerate(order):
            blk, ev = nxt
            _Side.wait(ev)
            nxt = (_fetch_zigzag(rc, buf, qkv, order[k + 1], lo, hi, spans, W, qw, kvw, side)
                   if k + 1 < len(order) else None)
            if j < me:
                g = _block_bwd(blk, out, lse, dout, info_h, hq, hkv, d, False, scale)
                dq += g[:, :qw].float()
                gk = g[:, qw:].float()
                ret = torch.zeros(Tl, kvw, dtype=qkv.dtype, device=qkv.device)
                ret[lo] = (gk[lo] + gk[hi]).to(qkv.dtype)                # both halves attended j's low chunk
            else:
                if out_h is None:
                    out_h = out.index_select(0, dup)
                    lse_h = lse.index_select(1, dup).contiguous()
                    dout_h = dout.index_select(0, dup)
                g = _block_bwd(blk, out_h, lse_h, dout_h, info_h, hq, hkv, d, False, scale)
                dq.index_add_(0, hi, g[lo, :qw].float() + g[hi, :qw].float())
                ret = g[:, qw:]
            gs[k + 1, : Tl * kvw].copy_(ret.reshape(-1))                 # slot s: gradient for the chunks of rank me - s
        rc.returns_written()
        tmp = torch.empty(Tl, kvw, dtype=qkv.dtype, device=qkv.device)
        for s in range(1, n):                                            # rank me + s used my chunks at its step s
            rc.pull_cols(rc.gstage, (me + s) % n, tmp, s * gs.shape[1], 0, kvw, kvw, Tl, kvw)
            dkv += tmp.float()
        rc.returns_read()
        return torch.cat([dq, dkv], dim=1).to(qkv.dtype), None, None, None, None, None, None


def _fetch(rc: RingContext, buf, qkv, src: int, Tl: int, W: int, qw: int, kvw: int, side):
    """Block for chunk ``src``: local queries next to the K/V columns pulled from rank ``src`` (on a side stream)."""
    def fill():
        blk = qkv.detach().clone()
        rc.pull_cols(buf, src, blk, qw, qw, W, W, Tl, kvw)
        return blk
    return side.run(fill)


def ring_attention(qkv: torch.Tensor, rc: Optional[RingContext], info: SeqInfo, n_heads: int, n_kv_heads: int,
                   head_dim: int, scale: Optional[float] = None) -> torch.Tensor:
    """Causal attention of this rank's chunk(s) ``qkv [Tl, (hq + 2 hkv) d]`` against every chunk at lower positions
    (``rc.zigzag`` selects the chunk assignment; ``info`` holds the local length of every sequence)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    from ..ops.attention import attention_packed
    if rc is None or rc.cp == 1:
        return attention_packed(qkv, info, n_heads, n_kv_heads, head_dim, causal=True, scale=scale)
    if rc.stage is not None:
        assert not qkv.is_cuda or head_dim in (64, 128), "ring attention uses the 64/128-wide attention kernels"
        fn = _RingAttnZigzag if rc.zigzag else _RingAttn
        return fn.apply(qkv.contiguous(), rc, info, n_heads, n_kv_heads, head_dim, scale)
    return _ring_attention_gathered(qkv, rc, info, n_heads, n_kv_heads, head_dim, scale)


class _GatherRows(torch.autograd.Function):
    """all_gather along dim 0 whose backward returns every rank the summed gradient of its own rows."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = dist.get_world_size(group)
        out = torch.empty(n * x.numel(), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous().reshape(-1), group=group)
        return out.view(n, *x.shape)

    @staticmethod
    def backward(ctx, dy):
        g = dy.contiguous().clone()
        dist.all_reduce(g, group=ctx.group)
        return g[dist.get_rank(ctx.group)], None


def chunk_positions(local_lens, cp: int, rank: int, zigzag: bool) -> torch.Tensor:
    """Position inside its sequence of every local row of rank ``rank`` (``local_lens``: that rank's row count per
    sequence, the same on every rank)."""
    pos = []
    for n in local_lens:
        if zigzag:
            c = n // 2
            pos.append(torch.arange(rank * c, (rank + 1) * c))
            pos.append(torch.arange((2 * cp - 1 - rank) * c, (2 * cp - rank) * c))
        else:
            pos.append(torch.arange(rank * n, (rank + 1) * n))
    return torch.cat(pos) if pos else torch.zeros(0, dtype=torch.int64)


def _ring_attention_gathered(qkv, rc: RingContext, info: SeqInfo, hq, hkv, d, scale):
    """Library-collective path (CPU / gloo): gather all chunks, attend under a mask built from the rows' positions."""
    Tl = qkv.shape[0]
    allq = _GatherRows.apply(qkv, rc.group)                              # [cp, Tl, W]
    q = qkv[:, : hq * d].reshape(Tl, hq, d).float()
    out = torch.zeros(Tl, hq, d, dtype=torch.float32, device=qkv.device)
    cu = info.cu_seqlens_cpu
    rep = hq // hkv
    pos = [chunk_positions(info.seqlens, rc.cp, r, rc.zigzag).to(qkv.device) for r in range(rc.cp)]
    for i in range(len(cu) - 1):
        a, b = cu[i], cu[i + 1]
        if b == a:
            continue
        kv = allq[:, a:b, hq * d:].float().reshape(rc.cp * (b - a), 2, hkv, d)
        k = kv[:, 0].repeat_interleave(rep, dim=1)
        v = kv[:, 1].repeat_interleave(rep, dim=1)
        kpos = torch.cat([p[a:b] for p in pos])
        mask = pos[rc.rank][a:b, None] >= kpos[None, :]
        sc = torch.einsum("qhd,khd->hqk", q[a:b], k) * scale
        sc = sc.masked_fill(~mask[None], float("-inf"))
        out[a:b] = torch.einsum("hqk,khd->qhd", torch.softmax(sc, dim=-1), v)
    return out.reshape(Tl, hq * d).to(qkv.dtype)


def split_for_context_parallel(seqlens, cp: int, rank: int, device=None, zigzag: bool = False):
    """Row indices (into the packed stream), positions and the local ``SeqInfo`` of rank ``rank`` when every sequence
    is cut into ``cp`` contiguous chunks (length divisible by ``cp``) or, with ``zigzag``, into ``2 cp`` chunks of
    which the rank takes chunk ``rank`` and chunk ``2 cp - 1 - rank`` (length divisible by ``2 cp``)."""
    parts = cp * (2 if zigzag else 1)
    idx, lens, start = [], [], 0
    for n in seqlens:
        assert n % parts == 0, "context parallelism needs sequence lengths divisible by the number of chunks"
        lens.append(n // cp)
        idx.append(chunk_positions([n // cp], cp, rank, zigzag) + start)
        start += n
    pos = chunk_positions(lens, cp, rank, zigzag)
    return torch.cat(idx).to(device), pos.to(device), SeqInfo(lens, device=device)
