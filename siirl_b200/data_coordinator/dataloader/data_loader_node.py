"""Stateful, rank-partitioned dataloader DAG node.

Contract of the reference node (siirl/data_coordinator/dataloader/data_loader_node.py:117-433): the rollout
data-parallel width is ``group_world_size / rollout_tp``; each data-parallel rank draws
``train_batch_size // ddp_world`` prompts per step from its own partition with a seeded shuffle; TP peers of one
data-parallel rank see identical batches; ``auto_repeat`` wraps small datasets; ``state_dict`` /
``load_state_dict`` make resume continue with the next unseen batch.

``data.num_loader_workers > 0`` (the reference hands that number to ``torch.utils.data.DataLoader``): the next
training batch is tokenised / image-processed by a pool of threads while the current step runs on the GPU, one batch
ahead.  The checkpointed position only moves when a batch is handed out, so a prefetched batch that was never used is
drawn again after a resume."""
from __future__ import annotations

import random
from concurrent.futures import Future, ThreadPoolExecutor
from typing import Any, Dict, List, Optional, Tuple

from ..protocol import Batch
from .partitioned_dataset import PartitionedRLHFDataset, collate_fn


class DataLoaderNode:
    def __init__(self, config, tokenizer, processor=None, group_world_size: int = 1, group_rank: int = 0,
                 rollout_tp_size: int = 1, node_id: str = "data_loader"):
        self.node_id = node_id
        self.config = config
        data = config.data
        self.rollout_ddp_world_size = max(1, group_world_size // max(rollout_tp_size, 1))
        self.ddp_rank = group_rank // max(rollout_tp_size, 1)
        gen_bs = data.gen_batch_size or data.train_batch_size
        if gen_bs % self.rollout_ddp_world_size != 0:
            raise ValueError(f"batch size {gen_bs} is not divisible by the rollout data-parallel width "
                             f"{self.rollout_ddp_world_size}")
        self.batch_size = gen_bs // self.rollout_ddp_world_size
        self.train_dataset = PartitionedRLHFDataset(config, tokenizer, processor, self.ddp_rank,
                                                    self.rollout_ddp_world_size, is_eval=False)
        self.val_dataset = None
        if data.val_files or data.synthetic:
            self.val_dataset = PartitionedRLHFDataset(config, tokenizer, processor, self.ddp_rank,
                                                      self.rollout_ddp_world_size, is_eval=True, drop_last=False)
        n = len(self.train_dataset)
        if n < self.batch_size:
            if not data.auto_repeat:
                raise ValueError(f"rank partition holds {n} prompts < per-rank batch {self.batch_size}; "
                                 f"set data.auto_repeat=True to wrap around")
        self.shuffle = data.shuffle
        self.seed = int(getattr(config.trainer, "seed", 1))
        self.epoch = 0
        self.cursor = 0
        self._order = self._make_order(0)
        self.num_train_batches = max(1, n // self.batch_size) if n >= self.batch_size else 1
        self.num_val_batches = 0 if self.val_dataset is None else max(
            1, (len(self.val_dataset) + self.val_batch_size - 1) // self.val_batch_size)
        self._val_cursor = 0
        workers = int(getattr(data, "num_loader_workers", 0) or 0)
        self._pool = ThreadPoolExecutor(max_workers=workers, thread_name_prefix="loader") if workers > 0 else None
        self._ahead: Optional[Tuple[Future, int, int]] = None      # (batch being built, epoch and cursor after it)

    @property
    def val_batch_size(self) -> int:
        v = self.config.data.val_batch_size
        n = len(self.val_dataset) if self.val_dataset is not None else 0
        return max(1, min(v // self.rollout_ddp_world_size if v else n, max(n, 1)))

    def _make_order(self, epoch: int):
        idx = list(range(len(self.train_dataset)))
        if self.shuffle:
            random.Random(self.seed * 1000003 + epoch).shuffle(idx)
        return idx

    def _plan(self, epoch: int, cursor: int) -> Tuple[List[int], int, int]:
        """Indices of the batch that starts at ``(epoch, cursor)`` and the position after it."""
        out: List[int] = []
        order = self._order if epoch == self.epoch else self._make_order(epoch)
        while len(out) < self.batch_size:
            if cursor >= len(order):
                epoch, cursor = epoch + 1, 0
                order = self._make_order(epoch)
            take = min(self.batch_size - len(out), len(order) - cursor)
            out.extend(order[cursor:cursor + take])
            cursor += take
        return out, epoch, cursor

    def _advance(self, epoch: int, cursor: int) -> None:
        if epoch != self.epoch:
            self._order = self._make_order(epoch)
        self.epoch, self.cursor = epoch, cursor

    def _next_indices(self):
        out, epoch, cursor = self._plan(self.epoch, self.cursor)
        self._advance(epoch, cursor)
        return out

    def _build(self, indices: List[int]) -> Batch:
        items = list(self._pool.map(self.train_dataset.__getitem__, indices)) if self._pool is not None else \
            [self.train_dataset[i] for i in indices]
        return collate_fn(items)

    def _prefetch(self) -> None:
        indices, epoch, cursor = self._plan(self.epoch, self.cursor)
        workers = self._pool._max_workers

        def build() -> Batch:
            # the task itself holds one thread of the pool; the items go to the others
            if workers >= 2:
                return collate_fn(list(self._pool.map(self.train_dataset.__getitem__, indices)))
            return collate_fn([self.train_dataset[i] for i in indices])
        self._ahead = (self._pool.submit(build), epoch, cursor)

    def run(self, epoch: Optional[int] = None, is_validation_step: bool = False, **_) -> Batch:
        """Next training batch (or the next validation batch)."""
        if is_validation_step:
            if self.val_dataset is None:
                raise RuntimeError("no validation data configured")
            n = len(self.val_dataset)
            s = self._val_cursor
            e = min(s + self.val_batch_size, n)
            self._val_cursor = 0 if e >= n else e
            return collate_fn([self.val_dataset[i] for i in range(s, e)])
        if self._pool is None:
            return collate_fn([self.train_dataset[i] for i in self._next_indices()])
        if self._ahead is None:                       # first batch (or first after a resume): build it now, in parallel
            batch = self._build(self._next_indices())
        else:
            fut, epoch, cursor = self._ahead
            batch = fut.result()
            self._advance(epoch, cursor)
        self._prefetch()
        return batch

    def state_dict(self) -> Dict[str, Any]:
        return {"epoch": self.epoch, "cursor": self.cursor, "seed": self.seed, "batch_size": self.batch_size}

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        self.seed = int(state.get("seed", self.seed))
        self.epoch = int(state["epoch"])
        self.cursor = int(state["cursor"])
        self._order = self._make_order(self.epoch)
        self._ahead = None                            # whatever was being prefetched belonged to the old position
