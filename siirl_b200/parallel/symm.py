"""Symmetric peer memory over NVLink / NVSwitch and the collectives fused with their neighbouring compute.

``SymmComm.create(group)`` gives every rank of a single-node process group a communicator whose ``alloc`` returns
buffers that all peers have mapped (``cudaMalloc`` + CUDA IPC handles exchanged through the process group).  Kernels
of ``csrc/comm.cu`` then read or write peer HBM directly:

* ``fused_rs_adamw_ag``  — the optimizer step of :class:`FlatParamStore`: gradient reduce-scatter by pulling the
  owned shard from every peer (+ ||g||^2), a 4-byte all-reduce of the norm, then AdamW on the shard whose epilogue
  stores the new bf16 parameters into every peer's replica (all-gather).  Two kernels move all the bytes; NCCL only
  carries one float and orders the phases.
* ``pull_segments``      — variable-length all-to-all-v / re-shard from a table of (peer, offset, bytes) segments in
  one launch (Data-Coordinator sample redistribution, weight re-layout).
* ``barrier``            — flag barrier with bounded device-side waits.

The reference has no counterpart: its collectives are NCCL calls inside torch FSDP / Megatron and per-sample Ray
object transfers (siirl/engine/fsdp_workers.py:897-1020, siirl/dag_worker/dagworker.py:1117-1239).  The NCCL path of
:class:`FlatParamStore` (``comm=None``) is kept as the measured baseline.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..ops import lib as _lib


class _RawCudaBuffer:
    """Exposes a raw device pointer to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class SymmBuffer:
    def __init__(self, local_ptr: int, nbytes: int, peer_ptrs: List[int], tensor_u8: torch.Tensor):
        self.local_ptr, self.nbytes, self.peer_ptrs, self.u8 = local_ptr, nbytes, peer_ptrs, tensor_u8
        self.ptr_array = (ctypes.c_void_p * len(peer_ptrs))(*peer_ptrs)


class SymmComm:
    def __init__(self, group, device: torch.device):
        self.group = group
        self.device = device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.L = _lib.get_lib()
        self.buffers: Dict[int, SymmBuffer] = {}
        self._epoch = 0
        self._flags: Optional[SymmBuffer] = None
        self._shard_grad: Optional[torch.Tensor] = None
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=device)
        self._norm = torch.zeros(1, dtype=torch.float32, device=device)
        self._sync_word = torch.zeros(1, dtype=torch.float32, device=device)

    @classmethod
    def create(cls, group=None) -> "SymmComm":
        if not torch.cuda.is_available():
            raise RuntimeError("peer memory needs CUDA")
        group = group if group is not None else dist.group.WORLD
        dev = torch.device("cuda", torch.cuda.current_device())
        world = dist.get_world_size(group)
        if world > 16:
            raise RuntimeError("peer-memory communicator supports up to 16 ranks of one NVSwitch domain")
        comm = cls(group, dev)
        comm._flags = comm._alloc_raw(4096)
        comm._flags.u8.zero_()
        torch.cuda.synchronize()
        dist.barrier(group)
        return comm

    # ---- allocation ---------------------------------------------------------------------------------
    def _alloc_raw(self, nbytes: int) -> SymmBuffer:
        nbytes = (nbytes + 255) // 256 * 256
        p = ctypes.c_void_p()
        _lib.check(self.L.sb_symm_alloc(ctypes.byref(p), ctypes.c_longlong(nbytes)), "sb_symm_alloc")
        handle = (ctypes.c_ubyte * 64)()
        _lib.check(self.L.sb_ipc_get_handle(p, handle), "sb_ipc_get_handle")
        gathered: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(gathered, bytes(handle), group=self.group)
        peers: List[int] = []
        for r, h in enumerate(gathered):
            if r == self.rank:
                peers.append(p.value)
                continue
            q = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            _lib.check(self.L.sb_ipc_open_handle(buf, ctypes.byref(q)), "sb_ipc_open_handle")
            peers.append(q.value)
        t = torch.as_tensor(_RawCudaBuffer(p.value, nbytes), device=self.device)
        sb = SymmBuffer(p.value, nbytes, peers, t)
        self.buffers[p.value] = sb
        return sb

    def alloc(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        """Zero-initialised symmetric 1-D tensor; every rank must call with the same arguments in the same order."""
        item = torch.empty(0, dtype=dtype).element_size()
        sb = self._alloc_raw(numel * item)
        sb.u8.zero_()
        return sb.u8[: numel * item].view(dtype)

    def peers_of(self, t: torch.Tensor) -> SymmBuffer:
        sb = self.buffers.get(t.data_ptr())
        if sb is None:
            raise KeyError("tensor was not allocated by this communicator (or is an offset view)")
        return sb

    # ---- synchronisation ------------------------------------------------------------------------------
    barrier_limit_ms = 30000    # bound of the device-side wait of one barrier

    def barrier(self, use_flags: bool = True, resync: bool = False) -> None:
        """Stream-ordered barrier across the ranks: flag kernel with a bounded wait, or a 1-element all-reduce.
        ``resync=True`` puts the all-reduce in front of the flags: use it where ranks arrive after long independent
        work (rollout, a whole backward pass), so that the bounded device-side wait only ever sees a small skew."""
        if resync or not use_flags:
            dist.all_reduce(self._sync_word, group=self.group)
        if use_flags:
            self._epoch += 1
            _lib.check(self.L.sb_flag_barrier(self._flags.ptr_array, self.world, self.rank, self._epoch,
                                              _lib.ptr(_lib.status_word(self.device)),
                                              ctypes.c_longlong(self.barrier_limit_ms), _lib.stream()),
                       "sb_flag_barrier")

    # ---- fused optimizer step ---------------------------------------------------------------------------
    def fused_rs_adamw_ag(self, store, lr: float, betas, eps: float, weight_decay: float,
                          max_grad_norm: float, extra_sumsq: Optional[torch.Tensor] = None,
                          grad_scale: Optional[float] = None) -> torch.Tensor:
        grads, params = self.peers_of(store.flat_grad), self.peers_of(store.flat_param)
        if self._shard_grad is None or self._shard_grad.numel() != store.shard_size:
            self._shard_grad = torch.empty(store.shard_size, dtype=torch.float32, device=self.device)
        f, ll = ctypes.c_float, ctypes.c_longlong
        self.barrier(resync=True)                       # every rank's backward has finished writing its gradients
        self._sumsq.zero_()
        _lib.check(self.L.sb_rs_reduce(grads.ptr_array, self.world, self.rank, ll(store.lo), ll(store.shard_size),
                                       _lib.ptr(self._shard_grad), _lib.ptr(self._sumsq),
                                       _lib.ptr(_lib.status_word(self.device)), _lib.stream()),
                   "sb_rs_reduce")
        if extra_sumsq is not None:
            self._sumsq += extra_sumsq
        dist.all_reduce(self._sumsq, group=self.group)  # 4 bytes; also orders "all peers have read my gradients"
        _lib.check(self.L.sb_adamw_allgather(
            _lib.ptr(store.master), _lib.ptr(store.exp_avg), _lib.ptr(store.exp_avg_sq), _lib.ptr(self._shard_grad),
            params.ptr_array, self.world, _lib.ptr(self._sumsq), _lib.ptr(self._norm), ll(store.lo),
            ll(store.shard_size), f(lr), f(betas[0]), f(betas[1]), f(eps), f(weight_decay), store.step_count,
            f(max_grad_norm if max_grad_norm else 0.0), f(grad_scale if grad_scale is not None else 1.0 / self.world),
            _lib.stream()), "sb_adamw_allgather")
        self.barrier()                                  # every peer's stores into my replica have landed
        return self._norm[0]

    # ---- segment pull (all-to-all-v) -----------------------------------------------------------------------
    def pull_segments(self, src: torch.Tensor, segments: Sequence[Tuple[int, int, int, int]],
                      out: torch.Tensor) -> None:
        """``segments`` = (src_rank, src_byte_offset, dst_byte_offset, nbytes) with 16-byte granularity; copies
        from the peers' instances of the symmetric tensor ``src`` into the local tensor ``out``."""
        if not segments:
            return
        import numpy as np
        table = np.zeros((len(segments), 4), dtype=np.int64)
        for i, (r, so, do, nb) in enumerate(segments):
            assert so % 16 == 0 and do % 16 == 0 and nb % 16 == 0
            table[i] = (so, do, nb, r)  # last 8 bytes: src_rank (low int32), pad
        dev_table = torch.from_numpy(table).to(self.device)
        _lib.check(self.L.sb_segment_pull(self.peers_of(src).ptr_array, self.world, _lib.ptr(dev_table), len(segments),
                                          _lib.ptr(out), _lib.stream()), "sb_segment_pull")

    def alltoallv_rows(self, send: torch.Tensor, send_counts: Sequence[int], staging: torch.Tensor,
                       all_counts: Sequence[Sequence[int]]) -> torch.Tensor:
        """Row-wise all-to-all-v: ``send`` holds this rank's rows grouped by destination (``send_counts[d]`` rows
        for rank d); ``all_counts[s][d]`` is the same table of every rank.  Rows are staged in the symmetric buffer
        ``staging`` and every rank pulls what is addressed to it.  Returns ``[sum_s all_counts[s][me], row]``."""
        row_bytes = send[0].numel() * send.element_size() if send.numel() else 16
        assert row_bytes % 16 == 0, "rows must be multiples of 16 bytes"
        n_send = int(sum(send_counts))
        flat = staging.view(torch.uint8)
        flat[: n_send * row_bytes].copy_(send.reshape(-1).view(torch.uint8)[: n_send * row_bytes])
        self.barrier()
        segs, dst = [], 0
        for s in range(self.world):
            off = sum(all_counts[s][: self.rank]) * row_bytes
            nb = all_counts[s][self.rank] * row_bytes
            if nb:
                segs.append((s, off, dst, nb))
            dst += nb
        out = torch.empty(dst // row_bytes, *send.shape[1:], dtype=send.dtype, device=self.device)
        self.pull_segments(staging, segs, out)
        self.barrier()
        return out

    # ---- sample redistribution (Data Coordinator) -------------------------------------------------------------
    def alltoall_samples(self, send):
        """All-to-all of per-destination sample lists ``send[dst] = [(pos, Sample), ...]`` whose tensors live on this
        GPU: tensor bytes are packed once into a symmetric staging buffer and every rank pulls the rows addressed to it
        in ONE kernel (``sb_segment_pull``); only the small descriptors (shapes, dtypes, offsets, non-tensor fields)
        travel through an object collective.  Replaces the per-sample object-store transfers of the reference
        (siirl/dag_worker/dagworker.py:1117-1239).  Returns ``recv[src] = [(pos, Sample), ...]``."""
        from ..data_coordinator.sample import Sample
        descs = [[] for _ in range(self.world)]
        chunks, off = [], 0
        for dst, part in enumerate(send):
            for pos, s in part:
                fields = []
                for k in sorted(s.tensors):
                    t = s.tensors[k].to(self.device).contiguous()
                    nb = t.numel() * t.element_size()
                    pad = (-nb) % 16
                    raw = t.reshape(-1).view(torch.uint8)
                    chunks.append(raw if not pad else torch.cat([raw, raw.new_zeros(pad)]))
                    fields.append((k, str(t.dtype).replace("torch.", ""), tuple(t.shape), off, nb))
                    off += nb + pad
                descs[dst].append((pos, fields, s.non_tensors, s.meta))
        gathered: List[Optional[list]] = [None] * self.world
        dist.all_gather_object(gathered, (descs, off), group=self.group)
        need = max(g[1] for g in gathered)
        stage = getattr(self, "_sample_stage", None)
        if stage is None or stage.numel() < need:      # same decision on every rank (need is global): collective alloc
            self._sample_stage = stage = self.alloc(max(need, 1 << 26), torch.uint8)
        if chunks:
            stage[:off].copy_(torch.cat(chunks))
        self.barrier()
        segs, out_off, plan = [], 0, []
        for src in range(self.world):
            for pos, fields, non_t, meta in gathered[src][0][self.rank]:
                placed = []
                for k, dt, shape, so, nb in fields:
                    nb16 = nb + ((-nb) % 16)
                    segs.append((src, so, out_off, nb16))
                    placed.append((k, dt, shape, out_off, nb))
                    out_off += nb16
                plan.append((src, pos, placed, non_t, meta))
        out = torch.empty(max(out_off, 16), dtype=torch.uint8, device=self.device)
        self.pull_segments(stage, segs, out)
        self.barrier()                                   # peers are done reading my staging buffer
        recv = [[] for _ in range(self.world)]
        for src, pos, placed, non_t, meta in plan:
            tensors = {}
            for k, dt, shape, o, nb in placed:
                tensors[k] = out[o:o + nb].view(getattr(torch, dt)).reshape(shape)
            recv[src].append((pos, Sample(tensors, non_t, meta)))
        return recv
