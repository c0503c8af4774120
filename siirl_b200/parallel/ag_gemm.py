"""All-gather -> GEMM in one launch, for weights sharded by output rows over the ranks (ZeRO-3 / FSDP layout).

The reference's FSDP unshards a layer's weight with an NCCL all-gather and then runs the cuBLAS GEMM
(torch FSDP under siirl/engine/fsdp_workers.py:631-744).  ``AgLinear`` keeps each rank's row shard in symmetric
memory; ``sb_ag_gemm_bf16`` (``csrc/gemm_tcgen05.cu``) dedicates a few CTAs to pulling the peers' shards chunk by
chunk into a local staging matrix with plain peer loads while the remaining CTAs run the tcgen05 GEMM on the
chunks that have arrived, starting with the rank's own rows.  The training engine's default layout keeps a bf16
replica of the weights on every rank (only optimizer state is sharded) and therefore needs no gather at all; this
op serves the sharded-weight layout of models whose replica would not fit.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..ops import lib as _lib

_MAX_RANKS = 16


class _AgParams(ctypes.Structure):
    _fields_ = [("shard", ctypes.c_void_p * _MAX_RANKS), ("staging", ctypes.c_void_p), ("flags", ctypes.c_void_p),
                ("local", ctypes.c_void_p), ("ld", ctypes.c_longlong), ("world", ctypes.c_int),
                ("rank", ctypes.c_int), ("rows_per_rank", ctypes.c_int), ("copiers", ctypes.c_int)]


class AgLinear:
    """``y = x @ W^T + b`` with ``W [N, K]`` stored as ``N / world`` rows per rank."""

    def __init__(self, group, comm, N: int, K: int, copiers: int = 8, device=None, dtype=torch.bfloat16):
        self.group, self.comm = group, comm
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        assert N % self.world == 0 and K % 8 == 0
        self.N, self.K, self.rows = N, K, N // self.world
        self.copiers = copiers
        # a 128-row chunk of the gathered matrix must come from one owner
        self.fused = comm is not None and self.world > 1 and self.rows % 128 == 0
        self.tile_n = 256 if self.rows % 256 == 0 else 128
        if self.fused:
            dev = comm.device
            self.shard = comm.alloc(self.rows * K, torch.bfloat16).view(self.rows, K)
            self._shard_flat = self.shard.view(-1)
            self.staging = torch.empty(N, K, dtype=torch.bfloat16, device=dev)
            self.flags = torch.zeros((N + 127) // 128, dtype=torch.int32, device=dev)
            self.local = torch.zeros(2, dtype=torch.int32, device=dev)
            s = _AgParams()
            peers = comm.buffers[self._shard_flat.data_ptr()].peer_ptrs
            for r, p in enumerate(peers):
                s.shard[r] = p
            s.staging, s.flags, s.local = self.staging.data_ptr(), self.flags.data_ptr(), self.local.data_ptr()
            s.ld, s.world, s.rank, s.rows_per_rank, s.copiers = K, self.world, self.rank, self.rows, copiers
            self._params = torch.frombuffer(bytearray(bytes(s)), dtype=torch.uint8).to(dev)
        else:
            self.shard = torch.zeros(self.rows, K, dtype=dtype, device=device or "cpu")

    def load_shard(self, w_rows: torch.Tensor) -> None:
        """Install this rank's rows; collective on the peer-memory path (peers must see them before the next call)."""
        self.shard.copy_(w_rows)
        if self.fused:
            self.comm.barrier()

    def __call__(self, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        if not self.fused:
            if self.world > 1:
                full = torch.empty(self.N * self.K, dtype=self.shard.dtype, device=self.shard.device)
                dist.all_gather_into_tensor(full, self.shard.reshape(-1).contiguous(), group=self.group)
                full = full.view(self.N, self.K)
            else:
                full = self.shard
            return F.linear(x, full.to(x.dtype), bias)
        M = x.shape[0]
        x = x.contiguous()
        out = torch.empty(M, self.N, dtype=torch.bfloat16, device=x.device)
        L = _lib.get_lib()
        ll = ctypes.c_longlong
        _lib.check(L.sb_ag_gemm_bf16(_lib.ptr(x), _lib.ptr(self.staging), _lib.ptr(out), _lib.ptr(bias), M, self.N,
                                     self.K, ll(x.stride(0)), ll(self.K), ll(self.N), _lib.ptr(self._params),
                                     self.copiers, self.tile_n, _lib.ptr(_lib.status_word(x.device)),
                                     _lib.stream()),
                   "sb_ag_gemm_bf16")
        return out
