"""Data Coordinator: the sample buffer between DAG stages whose data-parallel width differs.

API of the reference's Ray actor (siirl/data_coordinator/data_buffer.py:28-350) — ``put``, ``put_batch``,
``get_batch(batch_size, dp_rank, filter_plugin, balance_partitions)``, ``get_all_by_filter``, ``get_valid_size``,
``peek_source_dp_size``, ``reset_cache`` — without Ray: every GPU process owns a ``DataCoordinator`` holding the
samples it produced, and the *global* view the reference gets from one central actor is rebuilt collectively:

1. sample metadata (``SampleInfo`` + producer rank + sequence number) is all-gathered — a few bytes per sample;
2. every rank computes the same global FIFO selection and the same Karmarkar-Karp length-balanced equal-size
   partition (workload ``24576*s + s^2``, small-at-both-ends order inside a partition as the reference does for
   pipeline schedules);
3. payloads move producer -> consumer directly: through the peer-memory all-to-all-v kernel when a symmetric-memory
   communicator is attached (``siirl_b200.parallel.symm``), else through ``torch.distributed`` collectives.

With a single process (or no process group) the class degenerates to the reference's in-memory deque semantics.
"""
from __future__ import annotations

import threading
from collections import deque
from typing import Any, Callable, Deque, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..utils.model_utils.seqlen_balancing import calculate_workload, get_seqlen_balanced_partitions
from .sample import Sample, SampleInfo


def _small_at_both_ends(idxs: List[int], tokens: List[int]) -> List[int]:
    """Order one partition so that short samples sit at both ends and long ones in the middle."""
    s = sorted(idxs, key=lambda i: tokens[i])
    return s[::2] + s[1::2][::-1]


def balanced_plan(tokens: List[int], group_keys: List[Any], parts: int) -> List[List[int]]:
    """Length-balanced split of ``len(tokens)`` samples into ``parts`` equal-sized partitions (indices into the
    lists).  Samples that belong together -- entries with the same non-``None`` ``group_keys`` value: the
    responses to one prompt -- stay on one partition whenever all groups have the same size and that size divides
    the partition size, because group-relative advantages (GRPO, RLOO) are computed per rank on the rows it holds;
    otherwise single samples are balanced."""
    work = calculate_workload(tokens).tolist()
    n = len(tokens)
    by_key: Dict[Any, List[int]] = {}
    groups: List[List[int]] = []
    for i, k in enumerate(group_keys):
        if k is None:
            groups.append([i])
        elif k in by_key:
            by_key[k].append(i)
        else:
            by_key[k] = [i]
            groups.append(by_key[k])
    size = len(groups[0]) if groups else 1
    whole = (size > 1 and all(k is not None for k in group_keys) and all(len(g) == size for g in groups)
             and n % parts == 0 and (n // parts) % size == 0)
    if not whole:
        plan = get_seqlen_balanced_partitions(work, parts, equal_size=True)
        return [_small_at_both_ends(p, tokens) for p in plan]
    gwork = [sum(work[i] for i in g) for g in groups]
    gtok = [sum(tokens[i] for i in g) for g in groups]
    gplan = get_seqlen_balanced_partitions(gwork, parts, equal_size=True)
    return [[i for gi in _small_at_both_ends(part, gtok) for i in groups[gi]] for part in gplan]


class DataCoordinator:
    def __init__(self, nnodes: int = 1, ppo_mini_batch_size: int = 0, world_size: int = 1,
                 group: Optional[dist.ProcessGroup] = None, comm=None):
        self.nnodes = nnodes
        self.ppo_mini_batch_size = ppo_mini_batch_size
        self.world_size = world_size
        self.group = group
        self.comm = comm
        self._queue: Deque[Tuple[SampleInfo, Any, int]] = deque()
        self._lock = threading.Lock()
        self._seq = 0
        self._cache: Dict[int, List[Any]] = {}
        self._cache_key = None

    # ---- producer side --------------------------------------------------------------------------
    def put(self, sample_info: SampleInfo, sample_ref: Any, caller_node_id: Optional[str] = None) -> None:
        with self._lock:
            if caller_node_id is not None and sample_info.node_id is None:
                sample_info.node_id = caller_node_id
            self._queue.append((sample_info, sample_ref, self._seq))
            self._seq += 1

    def put_batch(self, sample_infos: Sequence[SampleInfo], sample_refs: Sequence[Any],
                  caller_node_id: Optional[str] = None) -> None:
        if len(sample_infos) != len(sample_refs):
            raise ValueError("sample_infos and sample_refs differ in length")
        for info, ref in zip(sample_infos, sample_refs):
            self.put(info, ref, caller_node_id)

    # ---- local (single-process) consumer side -------------------------------------------------------
    def get_valid_size(self) -> int:
        return len(self._queue)

    def _matching(self, filter_plugin: Optional[Callable[[SampleInfo], bool]]):
        return [(i, e) for i, e in enumerate(self._queue) if filter_plugin is None or filter_plugin(e[0])]

    def get_batch(self, batch_size: int, dp_rank: int = 0, filter_plugin: Optional[Callable] = None,
                  balance_partitions: Optional[int] = None) -> List[Any]:
        """Local semantics of the reference: the first caller selects ``batch_size * partitions`` samples FIFO
        (after ``filter_plugin``), balances them into equal-size partitions and caches one per ``dp_rank``;
        later callers read their partition from the cache.  Returns ``[]`` when not enough samples are buffered."""
        parts = balance_partitions or 1
        with self._lock:
            if dp_rank in self._cache:
                return self._cache.pop(dp_rank)
            if self._cache:
                return []
            cand = self._matching(filter_plugin)
            need = batch_size * parts
            if len(cand) < need:
                return []
            chosen = cand[:need]
            drop = {i for i, _ in chosen}
            self._queue = deque(e for i, e in enumerate(self._queue) if i not in drop)
            entries = [e for _, e in chosen]
            if parts > 1:
                plan = self._apply_length_balancing([e[0] for e in entries], parts)
            else:
                plan = [list(range(need))]
            for r, idxs in enumerate(plan):
                self._cache[r] = [entries[i][1] for i in idxs]
            return self._cache.pop(dp_rank, [])

    @staticmethod
    def _apply_length_balancing(infos: Sequence[SampleInfo], partitions: int) -> List[List[int]]:
        tokens = [max(int(i.sum_tokens), 1) for i in infos]
        return balanced_plan(tokens, [i.uid for i in infos], partitions)

    def get_all_by_filter(self, filter_plugin: Callable[[SampleInfo], bool]) -> List[Any]:
        with self._lock:
            hit = self._matching(filter_plugin)
            drop = {i for i, _ in hit}
            self._queue = deque(e for i, e in enumerate(self._queue) if i not in drop)
            return [e[1] for _, e in hit]

    def peek_source_dp_size(self, filter_plugin: Callable[[SampleInfo], bool]) -> Optional[int]:
        for info, _, _ in self._queue:
            if filter_plugin(info):
                return info.dict_info.get("source_dp_size")
        return None

    def reset_cache(self) -> None:
        with self._lock:
            self._cache.clear()

    def clear(self) -> None:
        with self._lock:
            self._queue.clear()
            self._cache.clear()

    # ---- collective consumer side --------------------------------------------------------------------
    def global_valid_size(self, filter_plugin: Optional[Callable] = None) -> int:
        n = len(self._matching(filter_plugin))
        if self._dist_ready():
            t = torch.tensor([n], dtype=torch.int64)
            objs: List[Any] = [None] * dist.get_world_size(self.group)
            dist.all_gather_object(objs, int(n), group=self.group)
            return int(sum(objs))
        return n

    def _dist_ready(self) -> bool:
        return dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1

    def get_batch_collective(self, batch_size: int, dp_rank: int, dp_size: int,
                             filter_plugin: Optional[Callable] = None, balance: bool = True,
                             rank_of_dp: Optional[Callable[[int], List[int]]] = None) -> List[Sample]:
        """Collective ``get_batch``: every rank of the group calls it with its own ``dp_rank``; the global batch
        of ``batch_size * dp_size`` samples is selected FIFO over all producers, length-balanced into ``dp_size``
        partitions and each rank receives its partition.  Ranks sharing a ``dp_rank`` (TP/SP peers) receive the
        same samples.  Returns ``[]`` on every rank when fewer samples than needed are buffered."""
        if not self._dist_ready():
            return self.get_batch(batch_size, dp_rank, filter_plugin, dp_size if balance else None)
        world = dist.get_world_size(self.group)
        me = dist.get_rank(self.group)
        mine = [(info, seq) for info, _, seq in self._queue if filter_plugin is None or filter_plugin(info)]
        meta_local = [(seq, int(info.sum_tokens), info.uid) for info, seq in mine]
        gathered: List[Any] = [None] * world
        dist.all_gather_object(gathered, (meta_local, dp_rank), group=self.group)
        flat = [(seq, r, tok, uid) for r, (metas, _) in enumerate(gathered) for (seq, tok, uid) in metas]
        need = batch_size * dp_size
        if len(flat) < need:
            return []
        flat.sort(key=lambda x: (x[0], x[1]))
        chosen = flat[:need]
        tokens = [max(t, 1) for _, _, t, _ in chosen]
        if balance and dp_size > 1:
            # a prompt's responses come from one producer: (producer, uid) names the group
            keys = [(src, uid) if uid is not None else None for _, src, _, uid in chosen]
            plan = balanced_plan(tokens, keys, dp_size)
        else:
            plan = [list(range(i * batch_size, (i + 1) * batch_size)) for i in range(dp_size)]
        dp_of_rank = [g[1] for g in gathered]
        # what this rank must send: for every destination rank, the chosen local samples of its partition
        local_by_seq = {seq: ref for _, ref, seq in self._queue}
        send: List[List[Tuple[int, Sample]]] = [[] for _ in range(world)]
        for dst in range(world):
            for pos, ci in enumerate(plan[dp_of_rank[dst]]):
                seq, src = chosen[ci][0], chosen[ci][1]
                if src == me:
                    send[dst].append((pos, local_by_seq[seq]))
        recv = self._exchange(send)
        got: List[Optional[Sample]] = [None] * batch_size
        for part in recv:
            for pos, s in part:
                got[pos] = s
        taken = {c[0] for c in chosen if c[1] == me}
        with self._lock:
            self._queue = deque(e for e in self._queue if e[2] not in taken)
        assert all(s is not None for s in got), "redistribution lost a sample"
        return got  # type: ignore[return-value]

    def _exchange(self, send: List[List[Tuple[int, Sample]]]) -> List[List[Tuple[int, Sample]]]:
        """All-to-all of sample lists.  Tensor payloads go through the attached peer-memory communicator when
        there is one; this generic path uses object collectives (CPU / gloo and the library baseline)."""
        world = dist.get_world_size(self.group)
        if self.comm is not None and hasattr(self.comm, "alltoall_samples"):
            return self.comm.alltoall_samples(send)
        cpu_send = [[(pos, _to_cpu(s)) for pos, s in part] for part in send]
        out: List[Any] = [None] * world
        try:
            dist.all_to_all_object_list(out, cpu_send, group=self.group)  # type: ignore[attr-defined]
        except (AttributeError, RuntimeError, NotImplementedError):
            gathered: List[Any] = [None] * world
            dist.all_gather_object(gathered, cpu_send, group=self.group)
            me = dist.get_rank(self.group)
            out = [gathered[src][me] for src in range(world)]
        return out


def _to_cpu(s: Sample) -> Sample:
    return Sample({k: v.cpu() for k, v in s.tensors.items()}, s.non_tensors, s.meta)


_GLOBAL: Dict[str, DataCoordinator] = {}


def init_data_coordinator(nnodes: int = 1, ppo_mini_batch_size: int = 0, world_size: int = 1,
                          group: Optional[dist.ProcessGroup] = None, comm=None,
                          name: str = "global_data_coordinator") -> DataCoordinator:
    """Create (or fetch) the process-wide coordinator (the reference creates a named detached actor)."""
    if name not in _GLOBAL:
        _GLOBAL[name] = DataCoordinator(nnodes, ppo_mini_batch_size, world_size, group, comm)
    return _GLOBAL[name]


def reset_data_coordinators() -> None:
    _GLOBAL.clear()
