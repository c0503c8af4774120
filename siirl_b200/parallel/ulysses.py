"""Ulysses sequence parallelism: the packed token stream is split over ``sp`` ranks everywhere except inside
attention, where every rank holds ALL tokens of ``heads / sp`` heads.

The reference switches layouts with NCCL all-to-alls around flash-attention
(siirl/utils/model_utils/ulysses.py, gather_seq_scatter_heads / gather_heads_scatter_seq, wired in by
siirl/models/transformers/monkey_patch.py:143-244).  Here each switch is ONE kernel that pulls the strided
``[tokens x head-columns]`` blocks it needs straight out of the peers' buffers (``sb_block_pull`` in
``csrc/comm.cu``): no pack / unpack copies around a collective, the permutation is the transfer.  The backward of
each switch is the other pull.  Without peer memory (CPU / gloo) the same block tables are applied to an
all-gathered copy.
"""
from __future__ import annotations

import ctypes
from typing import List, Tuple

import torch
import torch.distributed as dist

from ..ops import lib as _lib


class _PullBlock(ctypes.Structure):
    _fields_ = [("src_off", ctypes.c_longlong), ("dst_off", ctypes.c_longlong), ("src_pitch", ctypes.c_longlong),
                ("dst_pitch", ctypes.c_longlong), ("rows", ctypes.c_int), ("col_bytes", ctypes.c_int),
                ("src_rank", ctypes.c_int), ("pad", ctypes.c_int)]


Block = Tuple[int, int, int, int, int, int, int]   # src_rank, src_off, dst_off, src_pitch, dst_pitch, rows, col_bytes


class UlyssesSP:
    def __init__(self, group, comm=None, max_elems: int = 0):
        """``max_elems``: largest tensor (elements, bf16) that passes through a layout switch."""
        self.group, self.comm = group, comm
        self.sp = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.stage = None
        if comm is not None and self.sp > 1:
            self.stage = [comm.alloc(max_elems, torch.bfloat16), comm.alloc(max_elems, torch.bfloat16)]
            self._turn = 0
            comm.barrier()

    # ---- generic pull ----------------------------------------------------------------------------------
    def _pull(self, src: torch.Tensor, blocks: List[Block], out_shape) -> torch.Tensor:
        out = torch.empty(out_shape, dtype=src.dtype, device=src.device)
        if self.stage is None or not src.is_cuda:
            full = torch.empty(self.sp * src.numel(), dtype=src.dtype, device=src.device)
            dist.all_gather_into_tensor(full, src.contiguous().reshape(-1), group=self.group)
            full = full.view(self.sp, -1)
            es = src.element_size()
            flat_out = out.view(-1)
            for r, so, do, sp_, dp_, rows, cb in blocks:
                w = cb // es
                s2 = torch.as_strided(full, (rows, w), (sp_ // es, 1), r * src.numel() + so // es)
                torch.as_strided(flat_out, (rows, w), (dp_ // es, 1), do // es).copy_(s2)
            return out
        # alternate two staging buffers: a rank may start the next switch while a peer still reads this one
        buf = self.stage[self._turn]
        self._turn ^= 1
        n = src.numel()
        assert n <= buf.numel(), "sequence-parallel staging buffer too small"
        buf[:n].copy_(src.reshape(-1))
        self.comm.barrier()
        arr = (_PullBlock * len(blocks))()
        for i, (r, so, do, sp_, dp_, rows, cb) in enumerate(blocks):
            arr[i] = _PullBlock(so, do, sp_, dp_, rows, cb, r, 0)
        L = _lib.get_lib()
        _lib.check(L.sb_block_pull(self.comm.peers_of(buf).ptr_array, self.sp, arr, len(blocks), _lib.ptr(out),
                                   _lib.stream()), "sb_block_pull")
        return out

    # ---- block tables -------------------------------------------------------------------------------------
    def _tables(self, Tl: int, parts: List[Tuple[int, int]], es: int = 2):
        """``parts``: (first column, width) of every column group of the sequence-sharded matrix whose width is split
        over the ranks (q, k, v heads; or the attention output).  Returns (to_heads, to_seq, W, Wl)."""
        sp, me = self.sp, self.rank
        W = sum(w for _, w in parts)
        Wl = W // sp
        to_heads, to_seq = [], []
        dcol = 0
        for c0, w in parts:
            wl = w // sp
            for r in range(sp):
                # head layout [sp*Tl, Wl] <- rank r's sequence shard [Tl, W]
                to_heads.append((r, (c0 + me * wl) * es, (r * Tl * Wl + dcol) * es, W * es, Wl * es, Tl, wl * es))
                # sequence layout [Tl, W] <- rank r's head shard [sp*Tl, Wl]
                to_seq.append((r, (me * Tl * Wl + dcol) * es, (c0 + r * wl) * es, Wl * es, W * es, Tl, wl * es))
            dcol += wl
        return to_heads, to_seq, W, Wl

    # ---- public ops ------------------------------------------------------------------------------------------
    def seq_to_heads(self, x: torch.Tensor, parts: List[Tuple[int, int]]) -> torch.Tensor:
        """``x [T/sp, W]`` (this rank's tokens, all heads) -> ``[T, W/sp]`` (all tokens, this rank's heads)."""
        if self.sp == 1:
            return x
        return _Switch.apply(x.contiguous(), self, tuple(parts), True)

    def heads_to_seq(self, x: torch.Tensor, parts: List[Tuple[int, int]]) -> torch.Tensor:
        """``x [T, W/sp]`` -> ``[T/sp, W]``; ``parts`` describe the columns of the sequence-sharded result."""
        if self.sp == 1:
            return x
        return _Switch.apply(x.contiguous(), self, tuple(parts), False)


class _Switch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, sp: UlyssesSP, parts, to_heads: bool):
        ctx.sp, ctx.parts, ctx.to_heads = sp, parts, to_heads
        return _switch(x, sp, parts, to_heads)

    @staticmethod
    def backward(ctx, dy):
        return _switch(dy.contiguous(), ctx.sp, ctx.parts, not ctx.to_heads), None, None, None


def _switch(x: torch.Tensor, sp: UlyssesSP, parts, to_heads: bool) -> torch.Tensor:
    es = x.element_size()
    if to_heads:
        Tl = x.shape[0]
        th, _, W, Wl = sp._tables(Tl, list(parts), es)
        assert x.shape[1] == W and all(w % sp.sp == 0 for _, w in parts)
        return sp._pull(x, th, (sp.sp * Tl, Wl))
    Tl = x.shape[0] // sp.sp
    _, ts, W, Wl = sp._tables(Tl, list(parts), es)
    assert x.shape[1] == Wl
    return sp._pull(x, ts, (Tl, W))

