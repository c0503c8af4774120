"""``Batch``: the container that flows between DAG nodes.

It replaces the TensorDict/NonTensorData pair of the reference (siirl/data_coordinator/protocol.py,
sample.py) with one small class: per-sample tensors (leading dimension = batch size), per-sample
non-tensor columns (numpy object arrays) and step-level metadata.  Dict-style access
(``batch["advantages"]``, ``"uid" in batch``) covers all three stores, so node functions written
against the reference's field contract read the same.
"""
from __future__ import annotations

import copy
from typing import Any, Dict, Iterable, Iterator, List, Optional, Sequence, Union

import numpy as np
import torch


def _as_obj_array(values: Sequence[Any]) -> np.ndarray:
    arr = np.empty(len(values), dtype=object)
    for i, v in enumerate(values):
        arr[i] = v
    return arr


class Batch:
    def __init__(self, tensors: Optional[Dict[str, torch.Tensor]] = None,
                 non_tensors: Optional[Dict[str, Sequence[Any]]] = None, meta: Optional[Dict[str, Any]] = None):
        self.tensors: Dict[str, torch.Tensor] = {}
        self.non_tensors: Dict[str, np.ndarray] = {}
        self.meta: Dict[str, Any] = dict(meta or {})
        for k, v in (tensors or {}).items():
            self.tensors[k] = v
        for k, v in (non_tensors or {}).items():
            self.non_tensors[k] = v if isinstance(v, np.ndarray) and v.dtype == object else _as_obj_array(list(v))
        self._check()

    # ---- size ---------------------------------------------------------------------------------
    @property
    def batch_size(self) -> int:
        for v in self.tensors.values():
            return int(v.shape[0])
        for v in self.non_tensors.values():
            return len(v)
        return 0

    def __len__(self) -> int:
        return self.batch_size

    def _check(self) -> None:
        n = None
        for k, v in list(self.tensors.items()) + list(self.non_tensors.items()):
            m = int(v.shape[0]) if isinstance(v, torch.Tensor) else len(v)
            if n is None:
                n = m
            elif m != n:
                raise ValueError(f"field '{k}' has leading size {m}, expected {n}")

    # ---- dict-like access ---------------------------------------------------------------------
    def __contains__(self, key: str) -> bool:
        return key in self.tensors or key in self.non_tensors or key in self.meta

    def keys(self) -> List[str]:
        return list(self.tensors) + list(self.non_tensors) + list(self.meta)

    def __iter__(self) -> Iterator[str]:
        return iter(self.keys())

    def __getitem__(self, key: Union[str, slice, int, torch.Tensor, np.ndarray, list]):
        if isinstance(key, str):
            if key in self.tensors:
                return self.tensors[key]
            if key in self.non_tensors:
                return self.non_tensors[key]
            if key in self.meta:
                return self.meta[key]
            raise KeyError(key)
        if isinstance(key, int):
            key = [key]
        return self.select_idxs(key)

    def get(self, key: str, default: Any = None) -> Any:
        return self[key] if key in self else default

    def __setitem__(self, key: str, value: Any) -> None:
        n = self.batch_size
        empty = not self.tensors and not self.non_tensors
        if isinstance(value, torch.Tensor) and value.dim() >= 1 and (empty or value.shape[0] == n):
            self.non_tensors.pop(key, None)
            self.meta.pop(key, None)
            self.tensors[key] = value
        elif isinstance(value, np.ndarray) and value.dtype == object and (empty or len(value) == n):
            self.tensors.pop(key, None)
            self.meta.pop(key, None)
            self.non_tensors[key] = value
        elif isinstance(value, (list, tuple)) and not empty and len(value) == n and key not in self.meta:
            self.tensors.pop(key, None)
            self.non_tensors[key] = _as_obj_array(list(value))
        else:
            self.tensors.pop(key, None)
            self.non_tensors.pop(key, None)
            self.meta[key] = value

    def set_non_tensor(self, key: str, values: Sequence[Any]) -> None:
        self.non_tensors[key] = _as_obj_array(list(values))
        self._check()

    def pop(self, key: str, default: Any = None) -> Any:
        for store in (self.tensors, self.non_tensors, self.meta):
            if key in store:
                return store.pop(key)
        return default

    def update(self, other: Union["Batch", Dict[str, Any]]) -> "Batch":
        if isinstance(other, Batch):
            self.tensors.update(other.tensors)
            self.non_tensors.update(other.non_tensors)
            self.meta.update(other.meta)
        else:
            for k, v in other.items():
                self[k] = v
        self._check()
        return self

    union = update

    def select(self, keys: Iterable[str]) -> "Batch":
        keys = list(keys)
        return Batch({k: self.tensors[k] for k in keys if k in self.tensors},
                     {k: self.non_tensors[k] for k in keys if k in self.non_tensors},
                     {k: self.meta[k] for k in keys if k in self.meta} or dict(self.meta))

    # ---- row operations -----------------------------------------------------------------------
    def select_idxs(self, idx) -> "Batch":
        if isinstance(idx, slice):
            t = {k: v[idx] for k, v in self.tensors.items()}
            nt = {k: v[idx] for k, v in self.non_tensors.items()}
            return Batch(t, nt, self.meta)
        if isinstance(idx, torch.Tensor):
            if idx.dtype == torch.bool:
                idx = idx.nonzero(as_tuple=True)[0]
            idx_t = idx.long()
        else:
            arr = np.asarray(idx)
            if arr.dtype == bool:
                arr = np.nonzero(arr)[0]
            idx_t = torch.as_tensor(arr, dtype=torch.long)
        idx_np = idx_t.cpu().numpy()
        t = {k: v[idx_t.to(v.device)] for k, v in self.tensors.items()}
        nt = {k: v[idx_np] for k, v in self.non_tensors.items()}
        return Batch(t, nt, self.meta)

    def chunk(self, n: int) -> List["Batch"]:
        """Split into ``n`` nearly equal contiguous parts (first parts get the remainder)."""
        bs = self.batch_size
        base, extra = divmod(bs, n)
        out, start = [], 0
        for i in range(n):
            size = base + (1 if i < extra else 0)
            out.append(self.select_idxs(slice(start, start + size)))
            start += size
        return out

    def split(self, size: int) -> List["Batch"]:
        return [self.select_idxs(slice(s, min(s + size, self.batch_size))) for s in range(0, self.batch_size, size)]

    def repeat(self, n: int, interleave: bool = True) -> "Batch":
        if interleave:
            t = {k: v.repeat_interleave(n, dim=0) for k, v in self.tensors.items()}
            nt = {k: np.repeat(v, n, axis=0) for k, v in self.non_tensors.items()}
        else:
            t = {k: v.repeat(n, *([1] * (v.dim() - 1))) for k, v in self.tensors.items()}
            nt = {k: np.tile(v, n) for k, v in self.non_tensors.items()}
        return Batch(t, nt, self.meta)

    @staticmethod
    def concat(batches: Sequence["Batch"]) -> "Batch":
        batches = [b for b in batches if b is not None]
        if not batches:
            return Batch()
        first = batches[0]
        t = {k: torch.cat([b.tensors[k] for b in batches], dim=0) for k in first.tensors}
        nt = {k: np.concatenate([b.non_tensors[k] for b in batches], axis=0) for k in first.non_tensors}
        meta = {}
        for b in batches:
            meta.update(b.meta)
        return Batch(t, nt, meta)

    def to(self, device) -> "Batch":
        return Batch({k: v.to(device, non_blocking=True) for k, v in self.tensors.items()}, self.non_tensors,
                     self.meta)

    def pin_memory(self) -> "Batch":
        return Batch({k: (v.pin_memory() if not v.is_cuda else v) for k, v in self.tensors.items()}, self.non_tensors,
                     self.meta)

    def nbytes(self) -> int:
        return sum(v.numel() * v.element_size() for v in self.tensors.values())

    def clone(self) -> "Batch":
        return Batch({k: v.clone() for k, v in self.tensors.items()},
                     {k: v.copy() for k, v in self.non_tensors.items()}, copy.deepcopy(self.meta))

    def __repr__(self) -> str:
        t = {k: tuple(v.shape) for k, v in self.tensors.items()}
        return f"Batch(bs={self.batch_size}, tensors={t}, non_tensors={list(self.non_tensors)}, meta={list(self.meta)})"


def union_tensor_dict(a: Batch, b: Batch) -> Batch:
    """Merge ``b`` into ``a``; a tensor present in both must be identical."""
    for k, v in b.tensors.items():
        if k in a.tensors and not torch.equal(a.tensors[k], v):
            raise ValueError(f"field '{k}' differs between the two batches")
    return a.update(b)


def all_gather_batch(batch: Batch, group=None) -> Batch:
    """Concatenate the batches of all ranks of ``group`` in rank order
    (reference: ``all_gather_data_proto``, siirl/data_coordinator/protocol.py:114-122)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return batch
    world = dist.get_world_size(group)
    out_t = {}
    for k, v in batch.tensors.items():
        parts = [torch.empty_like(v) for _ in range(world)]
        dist.all_gather(parts, v.contiguous(), group=group)
        out_t[k] = torch.cat(parts, dim=0)
    out_nt = {}
    for k, v in batch.non_tensors.items():
        parts: List[Any] = [None] * world
        dist.all_gather_object(parts, list(v), group=group)
        out_nt[k] = _as_obj_array([x for p in parts for x in p])
    return Batch(out_t, out_nt, batch.meta)


def select_idxs(batch: Batch, idx) -> Batch:
    return batch.select_idxs(idx)
