"""Per-trajectory sample schema and batch <-> samples conversion.

Field contract of the reference (siirl/data_coordinator/sample.py:13-322): ``SampleInfo`` is the light metadata the
coordinator indexes (token counts, uid, the node the sample is destined for); ``Sample`` carries the tensors of one
trajectory; ``preprocess_dataloader`` repeats every prompt ``n`` times and assigns the integer group id ``uid``;
``Dict2Samples`` / ``Samples2Dict`` split and re-collate a :class:`Batch`; ``filter_batch`` (the reference's
``filter_tensordict``) keeps a subset of rows in tensor and non-tensor fields alike.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from .protocol import Batch


@dataclass
class SampleInfo:
    agent_group: int = 0
    sum_tokens: int = 0
    prompt_length: int = 0
    response_length: int = 0
    uid: Any = None
    node_id: Optional[str] = None
    dict_info: Dict[str, Any] = field(default_factory=dict)


@dataclass
class Sample:
    """Tensors and non-tensor fields of ONE trajectory (row of a batch)."""
    tensors: Dict[str, torch.Tensor] = field(default_factory=dict)
    non_tensors: Dict[str, Any] = field(default_factory=dict)
    meta: Dict[str, Any] = field(default_factory=dict)

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.tensors.values())


def preprocess_dataloader(batch: Batch, n: int, uid_offset: int = 0) -> Batch:
    """Repeat each prompt ``n`` times (interleaved) and attach the integer group id ``uid`` = ``uid_offset`` + index
    of the prompt inside this rank-local batch.  Callers that let samples travel between ranks (or accumulate
    several generation batches) pass offsets that do not overlap, so that two prompts never share an id when a rank
    computes group-relative advantages over the rows it holds."""
    bs = batch.batch_size
    uid = torch.arange(bs, dtype=torch.int64) + int(uid_offset)
    dev = next(iter(batch.tensors.values())).device if batch.tensors else torch.device("cpu")
    batch["uid"] = uid.to(dev)
    return batch.repeat(n, interleave=True) if n > 1 else batch


def Dict2Samples(batch: Batch, key: Optional[str] = None, node_id: Optional[str] = None,
                 agent_group: int = 0) -> (List[SampleInfo], List[Sample]):
    """Split a batch into per-row samples with their metadata."""
    infos, samples = [], []
    bs = batch.batch_size
    am = batch.get("attention_mask")
    rm = batch.get("response_mask")
    prompts = batch.get("prompts")
    uid = batch.get("uid")
    for i in range(bs):
        t = {k: v[i] for k, v in batch.tensors.items()}
        nt = {k: v[i] for k, v in batch.non_tensors.items()}
        s = Sample(t, nt, dict(batch.meta))
        total = int(am[i].sum()) if am is not None else 0
        resp = int(rm[i].sum()) if rm is not None else 0
        plen = int(prompts.shape[1]) if prompts is not None else max(total - resp, 0)
        u = uid[i].item() if isinstance(uid, torch.Tensor) else (uid[i] if uid is not None else None)
        infos.append(SampleInfo(agent_group=agent_group, sum_tokens=total, prompt_length=plen, response_length=resp,
                                uid=u, node_id=node_id, dict_info={"key": key} if key is not None else {}))
        samples.append(s)
    return infos, samples


def Samples2Dict(samples: Sequence[Sample]) -> Batch:
    """Re-collate samples into a batch; adds ``global_token_num`` (valid tokens per sample)."""
    if not samples:
        return Batch()
    tensors = {k: torch.stack([s.tensors[k] for s in samples], dim=0) for k in samples[0].tensors}
    non = {k: [s.non_tensors[k] for s in samples] for k in samples[0].non_tensors}
    meta: Dict[str, Any] = {}
    for s in samples:
        meta.update(s.meta)
    b = Batch(tensors, non, meta)
    if "attention_mask" in tensors:
        b.meta["global_token_num"] = tensors["attention_mask"].sum(-1).tolist()
    return b


def filter_batch(batch: Batch, mask_or_indices) -> Batch:
    """Keep the rows selected by a boolean mask or an index list/tensor (all per-sample fields follow)."""
    if isinstance(mask_or_indices, (list, tuple)):
        mask_or_indices = np.asarray(mask_or_indices)
    return batch.select_idxs(mask_or_indices)


filter_tensordict = filter_batch
