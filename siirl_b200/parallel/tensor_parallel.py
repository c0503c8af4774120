"""Tensor parallelism for the rollout engine: row-parallel GEMM fused with its all-reduce over peer memory.

The reference gets rollout tensor parallelism from vLLM / SGLang (``rollout.tensor_model_parallel_size``,
siirl/engine/rollout/vllm_rollout/vllm_rollout_spmd.py:92-157), whose row-parallel layers run a cuBLAS GEMM followed
by an NCCL all-reduce.  Here the two are ONE launch per rank (``sb_gemm_ar_bf16`` in ``csrc/gemm_tcgen05.cu``): the
tcgen05 GEMM's epilogue hands each finished output tile to the tile's owner rank through symmetric peer memory, the
owner sums the partial tiles of all ranks and stores the bf16 result into every rank's output, tile by tile while
the other tiles are still being multiplied.  On CPU (gloo ranks) the same API falls back to ``F.linear`` +
``all_reduce`` so the host-side logic is testable without GPUs.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..ops import lib as _lib

_MAX_RANKS = 16


class _ArParams(ctypes.Structure):
    _fields_ = [("partial", ctypes.c_void_p * _MAX_RANKS), ("out", ctypes.c_void_p * _MAX_RANKS),
                ("ready", ctypes.c_void_p * _MAX_RANKS), ("done", ctypes.c_void_p * _MAX_RANKS),
                ("local", ctypes.c_void_p), ("ldo", ctypes.c_longlong), ("world", ctypes.c_int),
                ("rank", ctypes.c_int), ("recv", ctypes.c_void_p * _MAX_RANKS), ("recv_slab", ctypes.c_longlong),
                ("one_shot", ctypes.c_int)]


class TPContext:
    """Buffers and flags of one tensor-parallel group.  ``max_rows x max_cols`` bounds the output of a
    row-parallel layer (tokens per forward x hidden size)."""

    def __init__(self, group, comm=None, max_rows: int = 8192, max_cols: int = 8192, max_tiles: int = 8192,
                 fused_max_rows: int = 128, one_shot_rows: int = 0):
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.comm = comm
        self.max_rows, self.max_cols, self.max_tiles = max_rows, max_cols, max_tiles
        # Two protocols (csrc/gemm_ar.cuh).  Push ("one shot"): every rank stores its fp32 partial tile into every
        # peer's receive slab and each rank sums locally; (world - 1) x M x N x 4 bytes leave each GPU, which for two
        # ranks is all an all-reduce can do anyway, so a group of two uses it at every size; larger groups use it up
        # to 512 rows (decode batches).  Owner pull ("two shot") moves 2 x (world - 1) / world x M x N x 4 bytes but
        # measured 0.4-0.8x of GEMM + NCCL all-reduce at prefill sizes, so beyond ``fused_max_rows`` rows such groups
        # take the library collective.
        self.fused_max_rows = fused_max_rows
        self.one_shot_rows = min(max_rows, one_shot_rows or (max_rows if self.world == 2 else 512))
        self._params: Dict[tuple, torch.Tensor] = {}
        self._slabs: Optional[torch.Tensor] = None
        if comm is not None and self.world > 1:
            n = max_rows * max_cols
            self.partial = comm.alloc(n, torch.float32)
            self.out = comm.alloc(n, torch.bfloat16)
            self.ready = comm.alloc(max_tiles * _MAX_RANKS, torch.int32)
            self.done = comm.alloc(max_tiles, torch.int32)
            self.recv = comm.alloc(2 * self.world * self.one_shot_rows * max_cols, torch.float32)
            self.local = torch.zeros(2 + max_tiles, dtype=torch.int32, device=comm.device)
            # split-K slabs of the decode path: at most one 128 x 128 tile per SM
            self._slabs = torch.empty(160 * 128 * 128, dtype=torch.float32, device=comm.device)
            comm.barrier()

    @property
    def fused(self) -> bool:
        return self.comm is not None and self.world > 1

    def _ar_params(self, N: int, one_shot: bool) -> torch.Tensor:
        t = self._params.get((N, one_shot))
        if t is None:
            c = self.comm
            s = _ArParams()
            for name, buf in (("partial", self.partial), ("out", self.out), ("ready", self.ready),
                              ("done", self.done), ("recv", self.recv)):
                arr = getattr(s, name)
                for r, p in enumerate(c.peers_of(buf).peer_ptrs):
                    arr[r] = p
            s.local = self.local.data_ptr()
            s.ldo, s.world, s.rank = N, self.world, self.rank
            s.recv_slab, s.one_shot = self.one_shot_rows * self.max_cols, int(one_shot)
            raw = bytes(s)
            t = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(c.device)
            self._params[(N, one_shot)] = t
        return t

    # ---- row-parallel linear ------------------------------------------------------------------------
    def row_parallel_linear(self, x: torch.Tensor, w_shard: torch.Tensor, bias: Optional[torch.Tensor] = None
                            ) -> torch.Tensor:
        """``sum_r x_r @ w_r^T + bias`` on every rank.  ``x [M, K/tp]`` contiguous, ``w_shard [N, K/tp]`` (a column
        slice of the full weight is fine: only the inner dimension must be contiguous).  The CUDA result is a view
        of the group's output buffer: valid until the next call on this context."""
        if self.world == 1:
            return F.linear(x, w_shard, bias) if not x.is_cuda else __import__(
                "siirl_b200.ops.dense", fromlist=["linear"]).linear(x, w_shard, bias)
        if not self.fused or not x.is_cuda:
            y = F.linear(x.float(), w_shard.float())
            dist.all_reduce(y, group=self.group)
            if bias is not None:
                y = y + bias.float()
            return y.to(x.dtype)
        from ..ops.dense import _best_splits, linear
        M, K = x.shape
        N = w_shard.shape[0]
        one_shot = M <= self.one_shot_rows
        if not one_shot and M > self.fused_max_rows:
            y = linear(x, w_shard)
            dist.all_reduce(y, group=self.group)
            return y + bias if bias is not None else y
        assert M * N <= self.max_rows * self.max_cols and N % 8 == 0 and w_shard.stride(1) == 1
        x = x.contiguous()
        tile_n = 128
        tiles_mn = (M + 127) // 128 * ((N + tile_n - 1) // tile_n)
        # split-K only while every (tile, slice) item gets its own CTA: a tile's finisher waits for peers in the kernel
        splits = min(_best_splits(tiles_mn, (K + 63) // 64), max(1, 148 // tiles_mn))
        L = _lib.get_lib()
        ll = ctypes.c_longlong
        if splits > 1:
            need = splits * M * N
            if self._slabs is None or self._slabs.numel() < need:
                self._slabs = torch.empty(need, dtype=torch.float32, device=x.device)
            c_local, stride = self._slabs, M * N
        else:
            c_local, stride = self.partial, 0
        _lib.check(L.sb_gemm_ar_bf16(_lib.ptr(x), _lib.ptr(w_shard), _lib.ptr(bias), M, N, K, ll(x.stride(0)),
                                     ll(w_shard.stride(0)), _lib.ptr(self._ar_params(N, one_shot)), _lib.ptr(c_local), tile_n,
                                     splits, ll(stride), self.max_tiles, _lib.ptr(_lib.status_word(x.device)),
                                     _lib.stream()), "sb_gemm_ar_bf16")
        return self.out[: M * N].view(M, N)
