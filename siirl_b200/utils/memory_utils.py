"""Memory hygiene between phases of a step (reference: siirl/utils/memory_utils.py:1-135, ``aggressive_empty_cache``).

On a colocated worker the rollout engine's KV arena, the training activations and the optimizer state take turns in
the same HBM.  ``release_memory`` returns cached allocator blocks to the driver between phases so that the next phase's
large allocations do not fragment; ``memory_report`` gives the numbers the ``perf/`` metrics log."""
from __future__ import annotations

import gc
from typing import Dict, Optional

import torch


def memory_report(device: Optional[torch.device] = None) -> Dict[str, float]:
    """Allocator and device figures in GiB (zeros on a CPU-only process)."""
    if not torch.cuda.is_available():
        return {"allocated_gib": 0.0, "reserved_gib": 0.0, "max_allocated_gib": 0.0, "free_gib": 0.0, "total_gib": 0.0}
    free, total = torch.cuda.mem_get_info(device)
    gib = float(1 << 30)
    return {"allocated_gib": torch.cuda.memory_allocated(device) / gib,
            "reserved_gib": torch.cuda.memory_reserved(device) / gib,
            "max_allocated_gib": torch.cuda.max_memory_allocated(device) / gib,
            "free_gib": free / gib, "total_gib": total / gib}


def release_memory(force_sync: bool = True, rounds: int = 2, min_reclaim_gib: float = 0.25) -> float:
    """Collect Python garbage and return cached CUDA blocks; repeats while a round still frees at least
    ``min_reclaim_gib``.  Returns the GiB of reserved memory given back."""
    if not torch.cuda.is_available():
        gc.collect()
        return 0.0
    if force_sync:
        torch.cuda.synchronize()
    before = torch.cuda.memory_reserved()
    last = before
    for _ in range(max(1, rounds)):
        gc.collect()
        torch.cuda.empty_cache()
        now = torch.cuda.memory_reserved()
        if (last - now) / float(1 << 30) < min_reclaim_gib:
            last = now
            break
        last = now
    return (before - last) / float(1 << 30)


def reset_peak_stats() -> None:
    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats()
