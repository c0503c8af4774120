"""Sequence-length load balancing (reference: siirl/utils/model_utils/seqlen_balancing.py:29-417).

* ``calculate_workload``: attention-aware cost of a sequence, ``24576 * s + s^2`` (linear FLOPs of a 7B layer
  dominate up to ~24k tokens, then the quadratic attention term).
* ``karmarkar_karp`` / ``get_seqlen_balanced_partitions``: k-way partition (C++ in ``csrc/host/kk_partition.cpp``
  when the native library is built, pure Python otherwise; both give the same partitions).
* ``rearrange_micro_batches``: token-budget dynamic micro-batches, with the number of micro-batches equalised
  across data-parallel ranks by a MAX all-reduce so every rank runs the same number of steps.
"""
from __future__ import annotations

import ctypes
import heapq
import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def calculate_workload(seqlens) -> torch.Tensor:
    s = torch.as_tensor(seqlens, dtype=torch.int64)
    return 24576 * s + s * s


def _kk_python(workloads: Sequence[int], k: int, equal_size: bool) -> List[List[int]]:
    order = sorted((int(w), i) for i, w in enumerate(workloads))

    def sort_sets(sets):
        sets.sort(key=lambda s: (s[0], len(s[1])), reverse=True)
        return sets

    states = []
    if equal_size:
        assert len(order) % k == 0, f"{len(order)} items cannot be split evenly into {k} parts"
        for off in range(0, len(order), k):
            states.append(sort_sets([[order[off + j][0], [order[off + j][1]]] for j in range(k)]))
    else:
        for w, i in order:
            states.append(sort_sets([[w, [i]]] + [[0, []] for _ in range(k - 1)]))
    if not states:
        return [[] for _ in range(k)]
    heap = [(-(st[0][0] - st[-1][0]), -st[0][0], n, st) for n, st in enumerate(states)]
    heapq.heapify(heap)
    counter = len(states)
    while len(heap) > 1:
        _, _, _, a = heapq.heappop(heap)
        _, _, _, b = heapq.heappop(heap)
        for j in range(k):
            a[j][0] += b[k - 1 - j][0]
            a[j][1].extend(b[k - 1 - j][1])
        sort_sets(a)
        heapq.heappush(heap, (-(a[0][0] - a[-1][0]), -a[0][0], counter, a))
        counter += 1
    final = heap[0][3]
    return [sorted(s[1]) for s in final]


def karmarkar_karp(seqlen_list: Sequence[int], k_partitions: int, equal_size: bool) -> List[List[int]]:
    """Partition item indices into ``k_partitions`` sets with near-equal sums."""
    n = len(seqlen_list)
    try:
        from ...ops import lib as _lib
        if _lib.available():
            L = _lib.get_lib()
            w = (ctypes.c_longlong * n)(*[int(x) for x in seqlen_list])
            out = (ctypes.c_int * n)()
            rc = L.sb_kk_partition(w, n, k_partitions, int(equal_size), out)
            if rc == 0:
                parts: List[List[int]] = [[] for _ in range(k_partitions)]
                for i in range(n):
                    parts[out[i]].append(i)
                return parts
    except Exception:  # noqa: BLE001  (fall back to the Python implementation)
        pass
    return _kk_python(seqlen_list, k_partitions, equal_size)


def get_seqlen_balanced_partitions(seqlen_list: Sequence[int], k_partitions: int, equal_size: bool) -> List[List[int]]:
    assert len(seqlen_list) >= k_partitions, f"{len(seqlen_list)} items < {k_partitions} partitions"
    parts = karmarkar_karp(seqlen_list, k_partitions, equal_size)
    seen = sorted(i for p in parts for i in p)
    assert seen == list(range(len(seqlen_list))), "partitioner lost or duplicated items"
    if equal_size:
        assert all(len(p) == len(seqlen_list) // k_partitions for p in parts)
    return [sorted(p) for p in parts]


def log_seqlen_unbalance(seqlen_list: Sequence[int], partitions: List[List[int]], prefix: str) -> dict:
    k = len(partitions)
    n = len(seqlen_list)
    chunk = max(1, n // k)
    naive = [sum(seqlen_list[i:i + chunk]) for i in range(0, n, chunk)][:k]
    bal = [sum(seqlen_list[i] for i in p) for p in partitions]
    return {f"{prefix}/min": min(naive), f"{prefix}/max": max(naive), f"{prefix}/minmax_diff": max(naive) - min(naive),
            f"{prefix}/balanced_min": min(bal), f"{prefix}/balanced_max": max(bal),
            f"{prefix}/mean": sum(seqlen_list) / max(k, 1)}


def rearrange_micro_batches(seqlens: Sequence[int], max_token_len: int, dp_group=None,
                            same_micro_num_in_dp: bool = True, min_num_micro_batch: Optional[int] = None,
                            use_workload: bool = False) -> List[List[int]]:
    """Index lists of dynamic micro-batches such that each holds at most ``max_token_len`` tokens."""
    seqlens = [int(x) for x in seqlens]
    assert max(seqlens, default=0) <= max_token_len, \
        f"max_token_len {max_token_len} is smaller than the longest sequence {max(seqlens)}"
    total = sum(seqlens)
    num = min(len(seqlens), max(1, math.ceil(total / max_token_len)))
    if min_num_micro_batch is not None:
        num = max(num, min(min_num_micro_batch, len(seqlens)))
    if same_micro_num_in_dp and dist.is_available() and dist.is_initialized():
        t = torch.tensor([num], dtype=torch.int64)
        if dist.get_backend(dp_group) == "nccl":
            t = t.cuda()
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=dp_group)
        num = min(int(t.item()), len(seqlens))
    costs = calculate_workload(seqlens).tolist() if use_workload else seqlens
    while True:
        parts = get_seqlen_balanced_partitions(costs, num, equal_size=False)
        if all(sum(seqlens[i] for i in p) <= max_token_len for p in parts) or num >= len(seqlens):
            break
        num += 1
    parts = [p for p in parts if p]
    parts.sort(key=lambda p: sum(seqlens[i] ** 2 for i in p), reverse=True)
    return parts


def get_reverse_idx(idx_map: Sequence[int]) -> List[int]:
    rev = [0] * len(idx_map)
    for i, j in enumerate(idx_map):
        rev[j] = i
    return rev


def prepare_dynamic_batch(batch, max_token_len: int, dp_group=None) -> Tuple[list, List[List[int]]]:
    seqlens = batch["attention_mask"].sum(-1).tolist()
    parts = rearrange_micro_batches(seqlens, max_token_len, dp_group)
    return [batch.select_idxs(p) for p in parts], parts


def restore_dynamic_batch(data: torch.Tensor, batch_idx_list: List[List[int]]) -> torch.Tensor:
    flat = [i for p in batch_idx_list for i in p]
    rev = get_reverse_idx(flat)
    return data[torch.tensor(rev, dtype=torch.long, device=data.device)]
