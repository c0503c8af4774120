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
operations.

Interleaved (virtual-stage) schedule, ``virtual_pipeline_model_parallel_size = V > 1``: the layers are cut into
``P V`` model chunks and stage ``s`` holds chunks ``s, s + P, ..., s + (V - 1) P``, so a micro-batch goes round the
ring of stages ``V`` times (the last stage sends to the first).  ``schedule_interleaved`` gives Megatron's order: the
stage walks its "virtual micro-batches" k = 0 .. M V - 1 (groups of ``P`` micro-batches per chunk), with
``2 (P - s - 1) + (V - 1) P`` warm-up forwards, then one forward / one backward in turn, then the remaining backwards;
the pipeline bubble shrinks by the factor ``V``.  All stages walk k in the same order, so the k-th activation a stage
receives from its predecessor is the k-th one the predecessor sent: point-to-point order is the only tag needed.
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


def schedule_interleaved(stage: int, stages: int, micro_batches: int, chunks: int) -> List[Tuple[str, int, int]]:
    """Order of ("F" | "B", micro-batch, local chunk) of one stage under interleaved 1F1B with ``chunks`` model chunks
    per stage.  Megatron-core wants the number of micro-batches to be a multiple of ``stages``; here the largest such
    prefix runs interleaved and the ``micro_batches % stages`` left over follow as one group of all forwards (chunk
    by chunk), then all backwards."""
    P, V = stages, chunks
    if V == 1:
        return [(op, i, 0) for op, i in schedule_1f1b(stage, P, micro_batches)]
    rest = list(range(micro_batches - micro_batches % P, micro_batches))
    tail = [("F", i, c) for c in range(V) for i in rest] + [("B", i, c) for c in reversed(range(V)) for i in rest]
    M = micro_batches - len(rest)
    if M == 0:
        return tail
    total = M * V

    def unit(k: int, forward: bool) -> Tuple[int, int]:
        c = (k % (P * V)) // P
        return (k // (P * V)) * P + k % P, (c if forward else V - 1 - c)

    warm = total if M == P else min(2 * (P - stage - 1) + (V - 1) * P, total)
    order: List[Tuple[str, int, int]] = [("F",) + unit(k, True) for k in range(warm)]
    for i in range(total - warm):
        order += [("F",) + unit(warm + i, True), ("B",) + unit(i, False)]
    order += [("B",) + unit(i, False) for i in range(total - warm, total)]
    return order + tail


class PipelineContext:
    def __init__(self, group, num_layers: int, fwd_group=None, bwd_group=None, virtual: int = 1,
                 wrap_fwd_group=None, wrap_bwd_group=None):
        self.group = group
        self.virtual = max(1, int(virtual or 1))
        # the link last stage -> first stage of the interleaved schedule has process groups of its own: with two
        # stages it joins the same pair of ranks as the ordinary link, in the opposite direction, and on one NCCL
        # communicator a rank's queued send and its peer's queued send would each wait for a receive behind the other
        self.wrap_fwd_group = wrap_fwd_group if wrap_fwd_group is not None else fwd_group
        self.wrap_bwd_group = wrap_bwd_group if wrap_bwd_group is not None else bwd_group
        # groups of the same ranks that carry activations (forward) and their gradients (backward); None: the
        # default group carries both (sends are then only safe with one micro-batch in flight)
        self.fwd_group, self.bwd_group = fwd_group, bwd_group
        self._pending: list = []
        self.pp = dist.get_world_size(group)
        self.stage = dist.get_rank(group)
        ranks = dist.get_process_group_ranks(group)
        # with virtual stages the stages form a ring: the last one hands chunk c to the first one's chunk c + 1
        ring = self.virtual > 1
        self.prev = ranks[self.stage - 1] if (self.stage > 0 or ring) else None
        self.next = ranks[(self.stage + 1) % self.pp] if (self.stage < self.pp - 1 or ring) else None
        self.last_global = ranks[-1]
        self.num_layers = num_layers
        self.per_chunk = (num_layers + self.pp * self.virtual - 1) // (self.pp * self.virtual)
        self.layer_lo, self.layer_hi = self.chunk_layers(0)

    def chunk_layers(self, chunk: int) -> Tuple[int, int]:
        """Layer range of this stage's local chunk ``chunk`` (model chunk ``chunk * pp + stage``)."""
        m = chunk * self.pp + self.stage
        return min(self.num_layers, m * self.per_chunk), min(self.num_layers, (m + 1) * self.per_chunk)

    def chunk_is_first(self, chunk: int) -> bool:
        return self.stage == 0 and chunk == 0

    def chunk_is_last(self, chunk: int) -> bool:
        return self.stage == self.pp - 1 and chunk == self.virtual - 1

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
        wrap = self.stage == (self.pp - 1 if forward else 0)            # sender's side of the ring-closing link
        self._pending.append((dist.isend(t, dst=dst, group=self._link(forward, wrap)), t))
        if len(self._pending) > 4 * self.pp * self.virtual:
            self.drain(keep=2 * self.pp * self.virtual)

    def _link(self, forward: bool, wrap: bool):
        if forward:
            return self.wrap_fwd_group if wrap else self.fwd_group
        return self.wrap_bwd_group if wrap else self.bwd_group

    def recv(self, buf: torch.Tensor, src: int, forward: bool) -> None:
        if not self.pipelined:
            dist.recv(buf, src=src)
        else:
            wrap = self.stage == (0 if forward else self.pp - 1)        # receiver's side of the ring-closing link
            dist.recv(buf, src=src, group=self._link(forward, wrap))

    def drain(self, keep: int = 0) -> None:
        """Wait for the oldest outstanding sends (all of them by default)."""
        while len(self._pending) > keep:
            work, _ = self._pending.pop(0)
            work.wait()

    def owns_param(self, name: str) -> bool:
        """Stage that trains a parameter: layers by index, embedding on the first stage, final norm / heads on the
        last (a tied embedding is trained by the first stage only)."""
        if name.startswith("layers."):
            return self.owner_stage(name, self.num_layers) == self.stage
        if name.startswith("embed_tokens") or name.startswith("vision."):
            return self.is_first
        return self.is_last

    def owner_stage(self, name: str, num_layers: int) -> int:
        if name.startswith("layers."):
            return min(self.pp * self.virtual - 1, int(name.split(".")[1]) // self.per_chunk) % self.pp
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
