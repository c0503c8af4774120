"""Parameter-sharded training state ("ZeRO-3" / FSDP FULL_SHARD) for the packed decoder.

The reference shards parameters, gradients and optimizer state with torch FSDP (FULL_SHARD / HYBRID_SHARD,
siirl/engine/fsdp_workers.py:151-156, 897-1020) and regathers them for the rollout engine in its sharding managers
(siirl/engine/sharding_manager/fsdp_vllm.py:86-226).  Here the same memory layout is built on peer memory:

* A *unit* is one decoder layer.  Its parameters form one flat bf16 range; every rank keeps a contiguous ``1 / world``
  piece of every unit in symmetric memory (``param_shard [L, piece]``), plus the fp32 master copy, Adam moments and the
  accumulated gradient of those pieces.  Everything outside the layers (embedding, final norm, LM head, vision tower)
  stays in a replicated :class:`FlatParamStore` -- 14 % of a 7B model.
* Forward / recompute of layer ``i`` calls ``fetch(i)``: the unit is assembled in one of two gather slots by ONE
  kernel that pulls the pieces from the peers' shards (``sb_segment_pull``) on a side stream, one layer ahead of the
  compute stream, in the direction the pass is walking; the layer's parameters are re-pointed at the slot.  Parameter
  shards only change in the optimizer step (which ends in a barrier), so a gather needs no cross-rank handshake.
* Backward of layer ``i`` accumulates its weight gradients into one of two symmetric fp32 gradient slots
  (``main_grad`` views); when the layer's input gradient is ready ``reduce(i)`` runs: flag barrier, then one kernel in
  which each rank pulls its piece of the unit from every peer's slot and adds the sum to its gradient shard
  (``sb_rs_reduce_acc``).  The slot is cleared under the protection of the next barrier.
* ``step``: one squared-norm all-reduce for units and replicated part together, AdamW on the owned pieces (bf16
  results go straight into the owner's shard, which is what the peers gather from), barrier.
* ``materialize_full()`` regathers every unit into one full replica for consumers that need whole weights (the rollout
  engine and its tensor-parallel slicing, HF export); ``release_full()`` frees it again.

Training needs per-layer activation checkpointing: a layer's weights are re-fetched for its backward, and only the
recomputation inside the backward pass sees the re-fetched slot.

On CPU (gloo ranks) the gathers and reductions use the library collectives, so the bookkeeping is testable without
GPUs.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import lib as _lib
from .flat_params import FlatParamStore, _round_up

_ALIGN = 128


class _ShardHolder(nn.Module):
    """Wraps this rank's pieces of all units as one parameter so that a rank-local FlatParamStore manages their
    master copy, Adam moments, gradient buffer, host offload and checkpoint state."""

    def __init__(self, numel: int, dtype, device):
        super().__init__()
        self.pieces = nn.Parameter(torch.zeros(numel, dtype=dtype, device=device))


class ShardedParamStore:
    def __init__(self, module: nn.Module, group: Optional[dist.ProcessGroup] = None, comm=None,
                 optimizer_state: bool = True, trainable: bool = True, layers_attr: str = "layers",
                 replica_group: Optional[dist.ProcessGroup] = None):
        self.module = module
        # hybrid sharding: pieces are sharded over ``group`` and replicated over ``replica_group``, whose members
        # hold the same pieces and sum their gradients before the optimizer step
        self.replica_group = replica_group
        self.replicas = dist.get_world_size(replica_group) if replica_group is not None else 1
        self.group = group
        self.comm = comm
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.trainable = trainable
        layers = list(getattr(module, layers_attr))
        if not layers:
            raise ValueError("module has no layers to shard")
        self.layers = layers
        self.L = len(layers)
        first = next(layers[0].parameters())
        self.device, self.dtype = first.device, first.dtype
        self._cuda = self.device.type == "cuda"
        if self._cuda and self.world > 1 and comm is None:
            raise ValueError("parameter sharding on GPUs needs the peer-memory communicator")

        # ---- unit layout (identical for every layer of a decoder) -------------------------------------------------
        self.unit_params: List[List[Tuple[str, nn.Parameter]]] = [list(l.named_parameters()) for l in layers]
        self.unit_offsets: List[Dict[str, Tuple[int, int, torch.Size]]] = []
        unit_len = 0
        for plist in self.unit_params:
            off, table = 0, {}
            for n, p in plist:
                assert p.dtype == self.dtype and p.device == self.device, f"{n}: mixed dtype/device"
                table[n] = (off, p.numel(), p.shape)
                off = _round_up(off + p.numel(), _ALIGN)
            self.unit_offsets.append(table)
            unit_len = max(unit_len, off)
        self.unit_len = _round_up(unit_len, _ALIGN * self.world)
        self.piece = self.unit_len // self.world

        # ---- replicated remainder ----------------------------------------------------------------------------------
        prefix = layers_attr + "."
        rest = [n for n, _ in module.named_parameters() if not n.startswith(prefix)]
        self.root: Optional[FlatParamStore] = None
        if rest:
            self.root = FlatParamStore(module, group=group, comm=comm, optimizer_state=optimizer_state and trainable,
                                       param_filter=lambda n: not n.startswith(prefix), with_grad=trainable,
                                       replica_group=replica_group)

        # ---- this rank's pieces ------------------------------------------------------------------------------------
        sym = (lambda n, dt: comm.alloc(n, dt)) if (self._cuda and comm is not None and self.world > 1) else None
        holder = _ShardHolder(self.L * self.piece, self.dtype, self.device)
        staging = torch.zeros(self.unit_len, dtype=self.dtype, device=self.device)
        lo = self.rank * self.piece
        with torch.no_grad():
            for i, plist in enumerate(self.unit_params):
                staging.zero_()
                for n, p in plist:
                    o, k, _ = self.unit_offsets[i][n]
                    staging[o:o + k].copy_(p.data.reshape(-1))
                holder.pieces.data[i * self.piece:(i + 1) * self.piece].copy_(staging[lo:lo + self.piece])
        del staging
        self.local = FlatParamStore(holder, group=None, comm=None, optimizer_state=optimizer_state and trainable,
                                    local_only=True, grad_scale=1.0 / (self.world * self.replicas), param_alloc=sym,
                                    with_grad=trainable)
        self._holder = holder
        self.param_shard = self.local.flat_param          # [L * piece], symmetric on GPUs
        self.grad_shard = self.local.flat_grad            # fp32 [L * piece]
        # the full parameters of the layers go away; they reappear as views of a gather slot / the full replica
        self._placeholder = torch.empty(0, dtype=self.dtype, device=self.device)
        for plist in self.unit_params:
            for _, p in plist:
                p.data = self._placeholder
                p.requires_grad_(trainable)
                if hasattr(p, "main_grad"):
                    del p.main_grad

        # ---- slots ---------------------------------------------------------------------------------------------------
        self.gather_slots = torch.zeros(2, self.unit_len, dtype=self.dtype, device=self.device)
        self.grad_slots = None
        if trainable:
            alloc = sym or (lambda n, dt: torch.zeros(n, dtype=dt, device=self.device))
            self.grad_slots = alloc(2 * self.unit_len, torch.float32).view(2, self.unit_len)
        self._resident: Dict[int, int] = {}               # slot -> unit held (or being gathered)
        self._last_unit: Optional[int] = None
        self._dir = 1
        self._full: Optional[torch.Tensor] = None
        self._grad_dirty = [False, False]
        self._side = torch.cuda.Stream(self.device) if self._cuda else None
        self._ready = [None, None]                        # gather finished (side stream)
        self._seg_tables: Dict[int, torch.Tensor] = {}
        for i, layer in enumerate(layers):
            layer.zero3 = self
            layer.zero3_index = i
        if self._cuda and comm is not None and self.world > 1:
            torch.cuda.synchronize(self.device)
            comm.barrier(use_flags=False)                 # every rank's pieces are in place before the first gather

    # ---- attributes shared with FlatParamStore users ------------------------------------------------------------------
    def __getattr__(self, name):
        # layout / state of the replicated remainder (checkpoint code written against FlatParamStore reads them)
        root = self.__dict__.get("root")
        if root is None or name.startswith("__"):
            raise AttributeError(name)
        return getattr(root, name)

    @property
    def expert(self) -> FlatParamStore:
        """The rank-local store of this rank's pieces: the checkpoint manager saves and restores it next to the
        replicated part, the way it handles the rank-local experts of an expert-parallel model (same world size on
        resume)."""
        return self.local

    def invalidate(self) -> None:
        """Forget gathered copies (after the shards were overwritten by a checkpoint load)."""
        self._resident.clear()
        self._last_unit = None
        if self.world > 1:
            if self._cuda:
                torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)

    def make_reduce_hook(self, unit: int):
        """Tensor hook for the input of layer ``unit``: its gradient is ready when the layer's backward is queued."""
        def hook(_grad):
            self.reduce(unit)
            return None
        return hook

    @property
    def flat_grad(self) -> torch.Tensor:
        """The largest idle fp32 buffer between an optimizer step and the next backward (lent to the KV arena)."""
        return self.grad_shard

    @property
    def master(self):
        return self.local.master

    @property
    def step_count(self) -> int:
        return self.local.step_count

    # ---- gather ---------------------------------------------------------------------------------------------------------
    def _segments(self, unit: int) -> torch.Tensor:
        """Device table of (src_off, dst_off, bytes, src_rank) rows: piece q of the unit from rank q's shard."""
        t = self._seg_tables.get(unit)
        if t is None:
            import numpy as np
            es = torch.empty(0, dtype=self.dtype).element_size()
            tab = np.zeros((self.world, 4), dtype=np.int64)
            for q in range(self.world):
                tab[q] = (unit * self.piece * es, q * self.piece * es, self.piece * es, q)
            t = torch.from_numpy(tab).to(self.device)
            self._seg_tables[unit] = t
        return t

    def _gather_into(self, unit: int, out: torch.Tensor) -> None:
        """Assemble unit ``unit`` (``unit_len`` elements) in ``out`` from all ranks' pieces, on the current stream."""
        mine = self.param_shard[unit * self.piece:(unit + 1) * self.piece]
        if self.world == 1:
            out.copy_(mine)
            return
        if self._cuda:
            L = _lib.get_lib()
            _lib.check(L.sb_segment_pull(self.comm.peers_of(self.param_shard).ptr_array, self.world,
                                         _lib.ptr(self._segments(unit)), self.world, _lib.ptr(out), _lib.stream()),
                       "sb_segment_pull")
            return
        parts = [torch.empty_like(mine) for _ in range(self.world)]
        dist.all_gather(parts, mine.contiguous(), group=self.group)
        out.copy_(torch.cat(parts))

    def _issue_gather(self, unit: int, slot: int) -> None:
        self._resident[slot] = unit
        if not self._cuda:
            self._gather_into(unit, self.gather_slots[slot])
            return
        main = torch.cuda.current_stream(self.device)
        free = torch.cuda.Event()
        free.record(main)                                  # everything queued so far (the slot's last reader) is done
        self._side.wait_event(free)
        with torch.cuda.stream(self._side):
            self._gather_into(unit, self.gather_slots[slot])
            ev = torch.cuda.Event()
            ev.record(self._side)
        self._ready[slot] = ev

    def _point(self, unit: int, base: torch.Tensor, grad_base: Optional[torch.Tensor]) -> None:
        for n, p in self.unit_params[unit]:
            o, k, shp = self.unit_offsets[unit][n]
            p.data = base[o:o + k].view(shp)
            if grad_base is not None:
                p.main_grad = grad_base[o:o + k].view(shp)
                if self.dtype == torch.float32:
                    p.grad = p.main_grad                   # plain autograd accumulates in place

    def fetch(self, unit: int) -> None:
        """Make layer ``unit``'s parameters usable on the current stream and start gathering its neighbour in the
        direction of travel.  Called at the top of every layer forward (also the recomputation inside backward)."""
        if self._full is not None:
            return
        if unit == 0:
            d = 1
        elif unit == self._last_unit:
            d = -self._dir                                 # the pass turns around (last layer: forward -> backward)
        else:
            d = 1 if (self._last_unit is None or unit > self._last_unit) else -1
        self._dir, self._last_unit = d, unit
        slot = unit % 2
        if self._resident.get(slot) != unit:
            self._issue_gather(unit, slot)
        if self._cuda and self._ready[slot] is not None:
            torch.cuda.current_stream(self.device).wait_event(self._ready[slot])
        self._point(unit, self.gather_slots[slot], self.grad_slots[slot] if self.trainable else None)
        nxt = unit + d
        if 0 <= nxt < self.L and self._resident.get(nxt % 2) != nxt and self.world > 1:
            self._issue_gather(nxt, nxt % 2)

    # ---- gradient reduce-scatter -------------------------------------------------------------------------------------------
    def _barrier(self) -> None:
        if self.world == 1:
            return
        if self._cuda:
            self.comm.barrier()
        # gloo collectives below are synchronous: no extra barrier needed on CPU

    def reduce(self, unit: int) -> None:
        """Layer ``unit``'s backward is queued: add the ranks' gradients of the unit into the owners' shards."""
        if not self.trainable:
            return
        slot, other = unit % 2, (unit + 1) % 2
        mine = self.grad_shard[unit * self.piece:(unit + 1) * self.piece]
        lo = self.rank * self.piece
        # gradients that arrived through plain autograd (CPU ops; a backward that did not find ``main_grad``) instead
        # of being accumulated by the kernels: fold them into the slot
        for _, p in self.unit_params[unit]:
            if p.grad is not None and p.grad.data_ptr() != p.main_grad.data_ptr():
                p.main_grad.add_(p.grad.to(p.main_grad.dtype))
                p.grad = p.main_grad if self.dtype == torch.float32 else None
        self._barrier()                                    # all ranks wrote this unit and finished reading the other slot
        if self._grad_dirty[other]:
            self.grad_slots[other].zero_()
            self._grad_dirty[other] = False
        if self.world == 1:
            mine.add_(self.grad_slots[slot][lo:lo + self.piece])
        elif self._cuda:
            L = _lib.get_lib()
            ll = ctypes.c_longlong
            base = self.comm.peers_of(self.grad_slots.view(-1)).ptr_array
            _lib.check(L.sb_rs_reduce_acc(base, self.world, self.rank, ll(slot * self.unit_len + lo), ll(self.piece),
                                          _lib.ptr(mine), _lib.stream()), "sb_rs_reduce_acc")
        else:
            full = self.grad_slots[slot].clone()
            dist.all_reduce(full, group=self.group)
            mine.add_(full[lo:lo + self.piece])
        self._grad_dirty[slot] = True
        if unit == 0:
            # end of a backward pass: clear the last slot too, once every peer has read it
            self._barrier()
            self.grad_slots[slot].zero_()
            self._grad_dirty[slot] = False
        if self.dtype == torch.float32:
            for _, p in self.unit_params[unit]:
                p.grad = None

    # ---- optimizer -----------------------------------------------------------------------------------------------------------
    def zero_grad(self) -> None:
        if self.trainable:
            self.grad_shard.zero_()
        if self.root is not None and self.trainable:
            self.root.zero_grad()

    def offload_state(self) -> None:
        self.local.offload_state()
        if self.root is not None:
            self.root.offload_state()

    def reload_state(self, wait: bool = True) -> None:
        self.local.reload_state(wait)
        if self.root is not None:
            self.root.reload_state(wait)

    def step(self, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
             max_grad_norm: float = 1.0) -> torch.Tensor:
        """AdamW on the owned pieces and on the replicated remainder under one global gradient norm."""
        assert self.trainable and self.local.master is not None
        # squared norm of the (summed, unscaled) unit gradients this rank owns; the pieces partition the units, so
        # the sum over ranks is the units' squared norm
        if self.replicas > 1:
            dist.all_reduce(self.local.flat_grad, group=self.replica_group)
        mine = self.local.local_sumsq()
        if self.root is not None:
            norm = self.root.step(lr, betas, eps, weight_decay, max_grad_norm, extra_sumsq=mine)
            r = self.root
            total = r.comm._sumsq if (r.world > 1 and r.comm is not None and self._cuda) else r._sumsq
        else:
            total = mine.clone()
            if self.world > 1:
                dist.all_reduce(total, group=self.group)
            norm = total.sqrt()[0] / (self.world * self.replicas)
        self.local.step(lr, betas, eps, weight_decay, max_grad_norm, global_sumsq=total)
        self._resident.clear()                             # gathered copies are stale now
        self._last_unit = None
        if self.world > 1:
            if self._cuda:
                self.comm.barrier(resync=True)             # no peer gathers before every owner has written its pieces
            else:
                dist.barrier(group=self.group)
        return norm

    # ---- whole-model views -----------------------------------------------------------------------------------------------------
    def materialize_full(self) -> torch.Tensor:
        """Regather every unit into one full replica ``[L, unit_len]`` and point the layers' parameters at it (rollout
        engine, tensor-parallel slicing, export).  Idempotent; ``release_full`` undoes it."""
        if self._full is None:
            full = torch.empty(self.L, self.unit_len, dtype=self.dtype, device=self.device)
            for i in range(self.L):
                self._gather_into(i, full[i])
            self._full = full
            for i in range(self.L):
                self._point(i, full[i], None)
            self._resident.clear()
        return self._full

    def release_full(self) -> None:
        if self._full is None:
            return
        for plist in self.unit_params:
            for _, p in plist:
                p.data = self._placeholder
        self._full = None
        self._last_unit = None
        if self._cuda:
            torch.cuda.empty_cache()

    def named_tensors(self):
        """(name, full tensor) of every parameter; materialises the layers first."""
        self.materialize_full()
        for n, p in self.module.named_parameters():
            yield n, p.data

    def sync_master_from_params(self) -> None:
        """After loading whole weights into the module (``materialize_full`` views): take this rank's pieces back
        into the shard and the fp32 master copies."""
        assert self._full is not None, "load weights into the materialised replica first"
        lo = self.rank * self.piece
        with torch.no_grad():
            for i in range(self.L):
                self.param_shard[i * self.piece:(i + 1) * self.piece].copy_(self._full[i, lo:lo + self.piece])
        self.local.sync_master_from_params()
        if self.root is not None:
            self.root.sync_master_from_params()
        if self.world > 1:
            if self._cuda:
                torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
