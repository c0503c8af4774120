"""Pipeline parallelism over NCCL / gloo point-to-point transfers.

The reference gets pipeline parallelism from Megatron-core's schedules (siirl/engine/actor/megatron_actor.py:307-510,
siirl/utils/megatron/pipeline_parallel.py).  Here a pipeline group of ``pp`` consecutive ranks splits the decoder
layers; a rank runs only its stage's layers and keeps gradients and optimizer state only for them, while the bf16
weights stay replicated (they are re-broadcast from their owning stage after every optimizer step), so the rollout
engine on every rank still sees the whole model without a resharding step.

Activations travel forward and their gradients backward with ``dist.send`` / ``dist.recv`` inside two autograd
functions, so an ordinary ``loss.backward()`` on every rank drives the whole pipeline:

* ``recv_from_prev``  forward: receive ``h`` from the previous stage; backward: send ``dL/dh`` to it;
* ``send_to_next``    forward: send ``h`` to the next stage and return a 0-d "handle"; backward: ignore the
  handle's (zero) incoming gradient, receive ``dL/dh`` from the next stage and return it.

A non-last stage adds ``0 * handle`` to the values it reports, which ties its autograd graph to the transfer.  One
micro-batch crosses the stages at a time (no interleaving of micro-batches): the schedule is the simplest correct
one, meant for capability parity, not for throughput.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


class PipelineContext:
    def __init__(self, group, num_layers: int):
        self.group = group
        self.pp = dist.get_world_size(group)
        self.stage = dist.get_rank(group)
        ranks = dist.get_process_group_ranks(group)
        self.prev = ranks[self.stage - 1] if self.stage > 0 else None
        self.next = ranks[self.stage + 1] if self.stage < self.pp - 1 else None
        self.last_global = ranks[-1]
        per = (num_layers + self.pp - 1) // self.pp
        self.layer_lo = min(num_layers, self.stage * per)
        self.layer_hi = min(num_layers, (self.stage + 1) * per)

    @property
    def is_first(self) -> bool:
        return self.stage == 0

    @property
    def is_last(self) -> bool:
        return self.stage == self.pp - 1

    def owns_param(self, name: str) -> bool:
        """Stage that trains a parameter: layers by index, embedding on the first stage, final norm / heads on the
        last (a tied embedding is trained by the first stage only)."""
        if name.startswith("layers."):
            return self.layer_lo <= int(name.split(".")[1]) < self.layer_hi
        if name.startswith("embed_tokens") or name.startswith("vision."):
            return self.is_first
        return self.is_last

    def owner_stage(self, name: str, num_layers: int) -> int:
        per = (num_layers + self.pp - 1) // self.pp
        if name.startswith("layers."):
            return min(self.pp - 1, int(name.split(".")[1]) // per)
        if name.startswith("embed_tokens") or name.startswith("vision."):
            return 0
        return self.pp - 1


class _RecvFromPrev(torch.autograd.Function):
    @staticmethod
    def forward(ctx, anchor: torch.Tensor, pc: PipelineContext, shape: Tuple[int, ...], dtype, device):
        ctx.pc = pc
        buf = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(buf, src=pc.prev)
        return buf

    @staticmethod
    def backward(ctx, grad):
        dist.send(grad.contiguous(), dst=ctx.pc.prev)
        return None, None, None, None, None


class _SendToNext(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h: torch.Tensor, pc: PipelineContext):
        ctx.pc, ctx.meta = pc, (h.shape, h.dtype, h.device)
        dist.send(h.contiguous(), dst=pc.next)
        return h.new_zeros(())

    @staticmethod
    def backward(ctx, _zero):
        shape, dtype, device = ctx.meta
        g = torch.empty(shape, dtype=dtype, device=device)
        dist.recv(g, src=ctx.pc.next)
        return g, None


def recv_from_prev(pc: PipelineContext, shape, dtype, device, needs_grad: bool) -> torch.Tensor:
    if needs_grad:
        anchor = torch.zeros((), device=device, requires_grad=True)
        return _RecvFromPrev.apply(anchor, pc, tuple(shape), dtype, device)
    buf = torch.empty(tuple(shape), dtype=dtype, device=device)
    dist.recv(buf, src=pc.prev)
    return buf


def send_to_next(pc: PipelineContext, h: torch.Tensor) -> Optional[torch.Tensor]:
    """Returns the 0-d handle when ``h`` carries gradient history, else ``None``."""
    if h.requires_grad and torch.is_grad_enabled():
        return _SendToNext.apply(h, pc)
    dist.send(h.contiguous(), dst=pc.next)
    return None


def broadcast_from_last(pc: PipelineContext, tensors: List[Optional[torch.Tensor]], shapes, dtypes, device):
    """Values computed by the last stage (log-probs, entropy) become available on every stage of the group."""
    out = []
    for t, shape, dt in zip(tensors, shapes, dtypes):
        buf = t.detach().contiguous() if pc.is_last else torch.empty(shape, dtype=dt, device=device)
        dist.broadcast(buf, src=pc.last_global, group=pc.group)
        out.append(buf)
    return out


@torch.no_grad()
def sync_stage_weights(model, pc: PipelineContext) -> None:
    """After an optimizer step every stage broadcasts the parameters it trains to the rest of its pipeline group, so
    all replicas (and the rollout engines that share them) hold the updated model."""
    ranks = dist.get_process_group_ranks(pc.group)
    n_layers = len(model.layers)
    for name, p in model.named_parameters():
        dist.broadcast(p.data, src=ranks[pc.owner_stage(name, n_layers)], group=pc.group)
