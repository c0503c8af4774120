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

A non-last stage adds ``0 * handle`` to the values it reports, which ties its autograd graph to the transfer.

Schedules.  Scoring passes run one micro-batch at a time.  Training runs Megatron's non-interleaved 1F1B order
(``schedule_1f1b``): stage ``s`` of ``P`` first runs ``P - s - 1`` warm-up forwards, then alternates one forward and
one backward, then drains its backwards, so up to ``P`` micro-batches are in flight and the stages work concurrently.
For that the sends are asynchronous (``isend``; buffers are kept until ``drain``) and the two directions use two
process groups of their own: a stage's "send activation of micro-batch k+1" and its neighbour's "send gradient of
micro-batch j" are then never queued behind one another (on NCCL each group has its own stream; on gloo the sends
return at once), which is what the combined send-forward / receive-backward calls of Megatron achieve with grouped
operations.  The interleaved (virtual-stage) schedule is not built.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def schedule_1f1b(stage: int, stages: int, micro_batches: int) -> List[Tuple[str, int]]:
    """Order of forward ("F", i) and backward ("B", i) passes of one stage under non-interleaved 1F1B."""
    warm = min(stages - stage - 1, micro_batches)
    order: List[Tuple[str, int]] = [("F", i) for i in range(warm)]
    for i in range(micro_batches - warm):
        order += [("F", warm + i), ("B", i)]
    order += [("B", i) for i in range(micro_batches - warm, micro_batches)]
    return order


class PipelineContext:
    def __init__(self, group, num_layers: int, fwd_group=None, bwd_group=None):
        self.group = group
        # groups of the same ranks that carry activations (forward) and their gradients (backward); None: the
        # default group carries both (sends are then only safe with one micro-batch in flight)
        self.fwd_group, self.bwd_group = fwd_group, bwd_group
        self._pending: list = []
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

    @property
    def pipelined(self) -> bool:
        return self.fwd_group is not None and self.bwd_group is not None

    def send(self, t: torch.Tensor, dst: int, forward: bool) -> None:
        """Asynchronous when the direction groups exist (the tensor is kept alive until ``drain``), else blocking."""
        t = t.contiguous()
        if not self.pipelined:
            dist.send(t, dst=dst)
            return
        self._pending.append((dist.isend(t, dst=dst, group=self.fwd_group if forward else self.bwd_group), t))
        if len(self._pending) > 4 * self.pp:
            self.drain(keep=2 * self.pp)

    def recv(self, buf: torch.Tensor, src: int, forward: bool) -> None:
        if not self.pipelined:
            dist.recv(buf, src=src)
        else:
            dist.recv(buf, src=src, group=self.fwd_group if forward else self.bwd_group)

    def drain(self, keep: int = 0) -> None:
        """Wait for the oldest outstanding sends (all of them by default)."""
        while len(self._pending) > keep:
            work, _ = self._pending.pop(0)
            work.wait()

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
        pc.recv(buf, pc.prev, forward=True)
        return buf

    @staticmethod
    def backward(ctx, grad):
        ctx.pc.send(grad, ctx.pc.prev, forward=False)
        return None, None, None, None, None


class _SendToNext(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h: torch.Tensor, pc: PipelineContext):
        ctx.pc, ctx.meta = pc, (h.shape, h.dtype, h.device)
        pc.send(h, pc.next, forward=True)
        return h.new_zeros(())

    @staticmethod
    def backward(ctx, _zero):
        shape, dtype, device = ctx.meta
        g = torch.empty(shape, dtype=dtype, device=device)
        ctx.pc.recv(g, ctx.pc.next, forward=False)
        return g, None


def recv_from_prev(pc: PipelineContext, shape, dtype, device, needs_grad: bool) -> torch.Tensor:
    if needs_grad:
        anchor = torch.zeros((), device=device, requires_grad=True)
        return _RecvFromPrev.apply(anchor, pc, tuple(shape), dtype, device)
    buf = torch.empty(tuple(shape), dtype=dtype, device=device)
    pc.recv(buf, pc.prev, forward=True)
    return buf


def send_to_next(pc: PipelineContext, h: torch.Tensor) -> Optional[torch.Tensor]:
    """Returns the 0-d handle when ``h`` carries gradient history, else ``None``."""
    if h.requires_grad and torch.is_grad_enabled():
        return _SendToNext.apply(h, pc)
    pc.send(h, pc.next, forward=True)
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
