"""Stateful, rank-partitioned dataloader DAG node.

Contract of the reference node (siirl/data_coordinator/dataloader/data_loader_node.py:117-433): the rollout
data-parallel width is ``group_world_size / rollout_tp``; each data-parallel rank draws
``train_batch_size // ddp_world`` prompts per step from its own partition with a seeded shuffle; TP peers of one
data-parallel rank see identical batches; ``auto_repeat`` wraps small datasets; ``state_dict`` /
``load_state_dict`` make resume continue with the next unseen batch."""
from __future__ import annotations

import random
from typing import Any, Dict, Optional

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

    def _next_indices(self):
        out = []
        while len(out) < self.batch_size:
            if self.cursor >= len(self._order):
                self.epoch += 1
                self.cursor = 0
                self._order = self._make_order(self.epoch)
            take = min(self.batch_size - len(out), len(self._order) - self.cursor)
            out.extend(self._order[self.cursor:self.cursor + take])
            self.cursor += take
        return out

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
        return collate_fn([self.train_dataset[i] for i in self._next_indices()])

    def state_dict(self) -> Dict[str, Any]:
        return {"epoch": self.epoch, "cursor": self.cursor, "seed": self.seed, "batch_size": self.batch_size}

    def load_state_dict(self, state: Dict[str, Any]) -> None:
        self.seed = int(state.get("seed", self.seed))
        self.epoch = int(state["epoch"])
        self.cursor = int(state["cursor"])
        self._order = self._make_order(self.epoch)
