"""Flat parameter / gradient store with a sharded AdamW ("ZeRO-2" layout).

Replaces torch FSDP + ``torch.optim.AdamW`` + ``clip_grad_norm_`` of the reference
(siirl/engine/fsdp_workers.py:897-1088, siirl/engine/actor/dp_actor.py:265-283) and Megatron's distributed
optimizer (siirl/utils/megatron/optimizer.py).  Design for 180 GB HBM parts on one NVSwitch domain:

* every parameter of a module is a view into ONE flat buffer in the compute dtype (bf16 on GPU), and has a
  ``main_grad`` view into ONE flat fp32 gradient buffer that the backward kernels accumulate into;
* the working copy of the parameters is replicated on the data-parallel ranks, so forward and backward need no
  communication at all;
* each rank owns a contiguous ``1/world`` shard of the fp32 master weights and Adam moments.  ``step()`` is
  reduce-scatter(grad) -> global norm -> AdamW on the shard -> all-gather(param); with the peer-memory backend
  (``siirl_b200.parallel.symm``) those three are a single kernel that pulls gradient shards from the peers'
  buffers, updates, and stores the new bf16 parameters into every peer's replica.

Communication therefore happens once per optimizer step (2 x model size), not once per layer per micro-batch.
"""
from __future__ import annotations

import ctypes
import math
from typing import Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import lib as _lib

_ALIGN = 128  # elements; keeps every parameter 256-byte aligned (TMA needs 16 bytes)


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class FlatParamStore:
    def __init__(self, module: nn.Module, group: Optional[dist.ProcessGroup] = None, comm=None,
                 optimizer_state: bool = True, param_filter=None, local_only: bool = False,
                 grad_scale: Optional[float] = None, param_alloc=None, with_grad: bool = True,
                 replica_group: Optional[dist.ProcessGroup] = None):
        """``param_filter(name) -> bool`` restricts the store to some parameters.  ``local_only`` makes a store
        whose parameters exist on this rank alone (expert-parallel experts): no reduce-scatter / all-gather, the
        whole state lives here, ``grad_scale`` (1 / data-parallel width) keeps their update on the same loss
        scale as the replicated parameters, and the clipping norm comes from the caller (``global_sumsq``).
        ``replica_group`` (hybrid sharding, FSDP's HYBRID_SHARD): the state is sharded over ``group`` and replicated
        over ``replica_group``; gradients are summed across the replicas before the shard group's reduce-scatter.
        ``param_alloc(numel, dtype)`` allocates the flat parameter buffer (a rank-local store whose parameters the
        peers read: symmetric memory); ``with_grad=False`` builds no gradient buffer (frozen models)."""
        params = [(n, p) for n, p in module.named_parameters() if param_filter is None or param_filter(n)]
        if not params:
            raise ValueError("module has no parameters")
        self.module = module
        self.group = group if not local_only else None
        self.comm = comm if not local_only else None  # peer-memory communicator (siirl_b200.parallel.symm.SymmComm)
        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.local_only = local_only
        self.replica_group = replica_group if not local_only else None
        self.replicas = dist.get_world_size(replica_group) if self.replica_group is not None else 1
        self.grad_scale = grad_scale
        if local_only:
            self.world, self.rank = 1, 0
        first = params[0][1]
        self.device, self.dtype = first.device, first.dtype
        self.names: List[str] = []
        self.offsets: Dict[str, Tuple[int, int, torch.Size]] = {}
        off = 0
        for n, p in params:
            assert p.dtype == self.dtype and p.device == self.device, f"{n}: mixed dtype/device"
            self.names.append(n)
            self.offsets[n] = (off, p.numel(), p.shape)
            off = _round_up(off + p.numel(), _ALIGN)
        self.total = _round_up(off, _ALIGN * max(self.world, 1))
        self.shard_size = self.total // self.world
        self.lo, self.hi = self.rank * self.shard_size, (self.rank + 1) * self.shard_size

        alloc = self.comm.alloc if (self.comm is not None and self.device.type == "cuda") else (
            lambda n, dt: torch.zeros(n, dtype=dt, device=self.device))
        self.flat_param = (param_alloc or alloc)(self.total, self.dtype)
        self.flat_grad = alloc(self.total, torch.float32) if with_grad else torch.zeros(0, device=self.device)
        for n, p in params:
            o, k, shp = self.offsets[n]
            view = self.flat_param[o:o + k].view(shp)
            view.copy_(p.data)
            p.data = view
            if not with_grad:
                continue
            g = self.flat_grad[o:o + k].view(shp)
            p.main_grad = g
            if self.dtype == torch.float32:
                p.grad = g  # plain autograd accumulates in place into the flat buffer
        self.params = [p for _, p in params]
        self.step_count = 0
        self.master = self.exp_avg = self.exp_avg_sq = None
        if optimizer_state:
            self.master = self.flat_param[self.lo:self.hi].float().clone()
            self.exp_avg = torch.zeros_like(self.master)
            self.exp_avg_sq = torch.zeros_like(self.master)
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._norm = torch.zeros(1, dtype=torch.float32, device=self.device)

    # ---- optimizer-state offload ------------------------------------------------------------------
    def offload_state(self) -> None:
        """Move the Adam moments of the owned shard to pinned host memory and release their device memory (the
        reference's ``fsdp_config.optimizer_offload``).  They are idle from the end of an optimizer step to the
        next one; on a single GPU they are 8 bytes per parameter that the rollout's KV arena can use."""
        if self.master is None or getattr(self, "_offloaded", False) or self.device.type != "cuda":
            return
        host = self.__dict__.setdefault("_host_state", {})
        for name in ("exp_avg", "exp_avg_sq"):
            t = getattr(self, name)
            if name not in host:
                host[name] = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
            host[name].copy_(t, non_blocking=True)
        torch.cuda.synchronize(self.device)
        self.exp_avg = self.exp_avg_sq = None
        self._offloaded = True
        torch.cuda.empty_cache()

    def reload_state(self, wait: bool = True) -> None:
        """Bring the moments back.  ``wait=False`` starts the copies on a side stream (call it when the backward
        passes begin); the optimizer step, or any later call with ``wait=True``, joins them."""
        if getattr(self, "_offloaded", False):
            side = self.__dict__.setdefault("_side_stream", torch.cuda.Stream(self.device))
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                self.exp_avg = self._host_state["exp_avg"].to(self.device, non_blocking=True)
                self.exp_avg_sq = self._host_state["exp_avg_sq"].to(self.device, non_blocking=True)
                self._reload_event = torch.cuda.Event()
                self._reload_event.record(side)
            self._offloaded = False
        ev = getattr(self, "_reload_event", None)
        if wait and ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)
            self.exp_avg.record_stream(torch.cuda.current_stream(self.device))
            self.exp_avg_sq.record_stream(torch.cuda.current_stream(self.device))
            self._reload_event = None

    # ---- gradients ----------------------------------------------------------------------------
    def zero_grad(self) -> None:
        self.flat_grad.zero_()
        if self.dtype != torch.float32:
            for p in self.params:
                p.grad = None

    def collect_grads(self) -> None:
        """Fold gradients that arrived through plain autograd (``p.grad``) into the flat fp32 buffer."""
        if self.dtype == torch.float32:
            for p in self.params:
                if p.grad is not None and p.grad.data_ptr() != p.main_grad.data_ptr():
                    p.main_grad.add_(p.grad)
                    p.grad = p.main_grad
            return
        for p in self.params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.float())
                p.grad = None

    # ---- optimizer step -----------------------------------------------------------------------
    def local_sumsq(self) -> torch.Tensor:
        """Sum of squares of this store's (unscaled) gradients, 1-element fp32 tensor."""
        self.collect_grads()
        out = torch.zeros(1, dtype=torch.float32, device=self.device)
        if self.device.type == "cuda":
            L = _lib.get_lib()
            _lib.check(L.sb_sumsq_accumulate(_lib.ptr(self.flat_grad), ctypes.c_longlong(self.flat_grad.numel()),
                                             _lib.ptr(out), _lib.stream()), "sb_sumsq_accumulate")
        else:
            out += self.flat_grad.double().pow(2).sum().float()
        return out

    def step(self, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
             max_grad_norm: float = 1.0, extra_sumsq: Optional[torch.Tensor] = None,
             global_sumsq: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One AdamW step on the owned shard; returns the global gradient norm (0-d tensor, no host sync).
        A non-finite norm leaves parameters and moments untouched.  ``extra_sumsq`` (this rank's share of
        gradients held by another store) is added to the squared norm before the ranks sum it;
        ``global_sumsq`` replaces the norm computation altogether (stores of rank-local parameters)."""
        assert self.master is not None, "store was built without optimizer state"
        self.reload_state()
        self.collect_grads()
        self.step_count += 1
        if self.replicas > 1:
            dist.all_reduce(self.flat_grad, group=self.replica_group)     # every shard group now holds the total
        grad_scale = self.grad_scale if self.grad_scale is not None else 1.0 / (self.world * self.replicas)
        if self.world > 1 and self.comm is not None and self.device.type == "cuda":
            norm = self.comm.fused_rs_adamw_ag(self, lr, betas, eps, weight_decay, max_grad_norm, extra_sumsq,
                                               grad_scale=grad_scale)
            return norm
        if self.world > 1:
            shard_grad = self._reduce_scatter()
        else:
            shard_grad = self.flat_grad
        self._sumsq.zero_()
        if self.device.type == "cuda":
            L = _lib.get_lib()
            _lib.check(L.sb_sumsq_accumulate(_lib.ptr(shard_grad), ctypes.c_longlong(shard_grad.numel()),
                                             _lib.ptr(self._sumsq), _lib.stream()), "sb_sumsq_accumulate")
        else:
            self._sumsq += shard_grad.double().pow(2).sum().float()
        if extra_sumsq is not None:
            self._sumsq += extra_sumsq
        if self.world > 1:
            dist.all_reduce(self._sumsq, group=self.group)
        if global_sumsq is not None:
            self._sumsq.copy_(global_sumsq)
        if self.device.type == "cuda":
            L = _lib.get_lib()
            f = ctypes.c_float
            _lib.check(L.sb_adamw_step(
                _lib.ptr(self.master), _lib.ptr(self.exp_avg), _lib.ptr(self.exp_avg_sq), _lib.ptr(shard_grad),
                _lib.ptr(self.flat_param[self.lo:self.hi]), _lib.ptr(self._sumsq), _lib.ptr(self._norm),
                ctypes.c_longlong(self.shard_size), f(lr), f(betas[0]), f(betas[1]), f(eps), f(weight_decay),
                self.step_count, f(max_grad_norm if max_grad_norm else 0.0), f(grad_scale), _lib.stream()),
                "sb_adamw_step")
        else:
            self._adamw_cpu(shard_grad, lr, betas, eps, weight_decay, max_grad_norm, grad_scale)
        if self.world > 1:
            self._all_gather_params()
        return self._norm[0]

    def _adamw_cpu(self, g, lr, betas, eps, wd, max_norm, grad_scale) -> None:
        norm = self._sumsq.sqrt() * grad_scale
        self._norm.copy_(norm)
        if not torch.isfinite(norm).all():
            return
        clip = 1.0
        if max_norm and max_norm > 0:
            clip = min(1.0, max_norm / (norm.item() + 1e-6))
        g = g.float() * (grad_scale * clip)
        b1, b2 = betas
        self.exp_avg.mul_(b1).add_(g, alpha=1 - b1)
        self.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1 - b2)
        bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
        self.master.mul_(1 - lr * wd)
        self.master.addcdiv_(self.exp_avg / bc1, (self.exp_avg_sq / bc2).sqrt_().add_(eps), value=-lr)
        self.flat_param[self.lo:self.hi].copy_(self.master)

    def _reduce_scatter(self) -> torch.Tensor:
        """Sum of the data-parallel ranks' gradients for the owned shard (library collective path)."""
        out = torch.empty(self.shard_size, dtype=torch.float32, device=self.device)
        try:
            dist.reduce_scatter_tensor(out, self.flat_grad, group=self.group)
        except (RuntimeError, NotImplementedError):
            dist.all_reduce(self.flat_grad, group=self.group)  # gloo has no reduce_scatter
            out.copy_(self.flat_grad[self.lo:self.hi])
        return out

    def _all_gather_params(self) -> None:
        shard = self.flat_param[self.lo:self.hi].clone()
        try:
            dist.all_gather_into_tensor(self.flat_param, shard, group=self.group)
        except (RuntimeError, NotImplementedError):
            parts = [torch.empty_like(shard) for _ in range(self.world)]
            dist.all_gather(parts, shard, group=self.group)
            self.flat_param.copy_(torch.cat(parts))

    # ---- state (sharded checkpoints) ----------------------------------------------------------
    def shard_state_dict(self) -> Dict[str, object]:
        self.reload_state()
        return {"layout": {"total": self.total, "world": self.world, "rank": self.rank,
                           "offsets": {n: (o, k, list(s)) for n, (o, k, s) in self.offsets.items()}},
                "master": self.master.cpu() if self.master is not None else None,
                "exp_avg": self.exp_avg.cpu() if self.exp_avg is not None else None,
                "exp_avg_sq": self.exp_avg_sq.cpu() if self.exp_avg_sq is not None else None,
                "step": self.step_count}

    def load_shard_state_dict(self, state: Dict[str, object]) -> None:
        self.reload_state()
        lay = state["layout"]
        if lay["total"] != self.total or lay["world"] != self.world:
            raise ValueError("shard layout differs (world size changed?): use load_full_state")
        for k in ("master", "exp_avg", "exp_avg_sq"):
            if state.get(k) is not None and getattr(self, k) is not None:
                getattr(self, k).copy_(state[k].to(self.device))
        self.step_count = int(state.get("step", 0))
        if self.master is not None:
            self.flat_param[self.lo:self.hi].copy_(self.master)
            if self.world > 1:
                self._all_gather_params()

    def load_full_state(self, master: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor,
                        step: int) -> None:
        """Elastic resume: load from unsharded state tensors and keep this rank's shard."""
        self.reload_state()
        self.master.copy_(master[self.lo:self.hi].to(self.device))
        self.exp_avg.copy_(exp_avg[self.lo:self.hi].to(self.device))
        self.exp_avg_sq.copy_(exp_avg_sq[self.lo:self.hi].to(self.device))
        self.step_count = step
        self.flat_param.copy_(master.to(self.device, self.dtype))

    def sync_master_from_params(self) -> None:
        """Call after loading model weights into the module (e.g. from safetensors)."""
        if self.master is not None:
            self.master.copy_(self.flat_param[self.lo:self.hi].float())

    def named_tensors(self) -> Iterable[Tuple[str, torch.Tensor]]:
        for n in self.names:
            o, k, shp = self.offsets[n]
            yield n, self.flat_param[o:o + k].view(shp)


def lr_at_step(optim_cfg, step: int, total_steps: int, megatron: bool = False) -> float:
    """Learning-rate schedule of the reference's optimizer config.

    FSDP-style keys (siirl/utils/model_utils/torch_functional.py:518-702): linear warm-up from 0 over
    ``lr_warmup_steps`` (or ``lr_warmup_steps_ratio``), then ``warmup_style`` constant / cosine / wsd down to
    ``min_lr_ratio * lr``.

    ``megatron=True`` reads the keys the reference hands to Megatron-core's parameter scheduler
    (siirl/utils/megatron/optimizer.py:40-75): warm-up from ``lr_warmup_init``, then ``lr_decay_style`` constant /
    linear / cosine / inverse-square-root over ``lr_decay_steps`` (default: the whole run) down to ``min_lr``."""
    base = optim_cfg.lr
    warm = optim_cfg.lr_warmup_steps
    if megatron:
        decay_steps = int(optim_cfg.lr_decay_steps or total_steps or 0)
        if warm is None or warm <= 0:
            warm = int((optim_cfg.lr_warmup_steps_ratio or 0.0) * max(decay_steps, 0))
        init, floor = float(optim_cfg.lr_warmup_init or 0.0), float(optim_cfg.min_lr or 0.0)
        if warm > 0 and step < warm:
            return init + (base - init) * (step + 1) / warm
        style = optim_cfg.lr_decay_style or "constant"
        if style == "constant" or decay_steps <= warm:
            return base
        if step >= decay_steps:
            return floor
        prog = (step - warm) / max(1, decay_steps - warm)
        if style == "linear":
            return floor + (base - floor) * (1.0 - prog)
        if style == "cosine":
            return floor + (base - floor) * 0.5 * (1.0 + math.cos(math.pi * prog))
        if style == "inverse-square-root":
            return max(floor, base * math.sqrt(max(warm, 1)) / math.sqrt(max(step, 1)))
        raise ValueError(f"unknown lr_decay_style {style!r}")
    if warm is None or warm < 0:
        warm = int(optim_cfg.lr_warmup_steps_ratio * max(total_steps, 0))
    if warm > 0 and step < warm:
        return base * (step + 1) / warm
    style = optim_cfg.warmup_style
    if style == "constant" or total_steps <= warm:
        return base
    prog = min(1.0, (step - warm) / max(1, total_steps - warm))
    min_ratio = optim_cfg.min_lr_ratio or 0.0
    if style == "cosine":
        c = 0.5 * (1 + math.cos(math.pi * 2 * optim_cfg.num_cycles * prog))
        return base * (min_ratio + (1 - min_ratio) * c)
    if style == "wsd":
        stable_end = 0.9
        if prog < stable_end:
            return base
        d = (prog - stable_end) / (1 - stable_end)
        return base * (min_ratio + (1 - min_ratio) * 0.5 * (1 + math.cos(math.pi * d)))
    return base


class ExpertSplitStore:
    """Optimizer store of an expert-parallel model: replicated (dense) parameters in a sharded-state
    :class:`FlatParamStore` over the data-parallel group, this rank's experts in a rank-local store.  One gradient
    norm over both clips both.  Attribute access falls through to the dense store, so code written against
    ``FlatParamStore`` (checkpointing, tests) keeps working; the expert store is ``.expert``."""

    def __init__(self, module: nn.Module, group=None, comm=None, is_expert=lambda n: ".experts_" in n):
        world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.dense = FlatParamStore(module, group, comm, param_filter=lambda n: not is_expert(n))
        self.expert = FlatParamStore(module, None, None, param_filter=is_expert, local_only=True,
                                     grad_scale=1.0 / world)

    def __getattr__(self, name):
        return getattr(self.__dict__["dense"], name)

    def zero_grad(self) -> None:
        self.dense.zero_grad()
        self.expert.zero_grad()

    def offload_state(self) -> None:
        self.dense.offload_state()
        self.expert.offload_state()

    def reload_state(self, wait: bool = True) -> None:
        self.dense.reload_state(wait)
        self.expert.reload_state(wait)

    def step(self, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
             max_grad_norm: float = 1.0) -> torch.Tensor:
        es = self.expert.local_sumsq()
        norm = self.dense.step(lr, betas, eps, weight_decay, max_grad_norm, extra_sumsq=es)
        d = self.dense
        total = d.comm._sumsq if (d.world > 1 and d.comm is not None and d.device.type == "cuda") else d._sumsq
        self.expert.step(lr, betas, eps, weight_decay, max_grad_norm, global_sumsq=total)
        return norm
