"""Profiling helpers (reference: siirl/utils/debug/profile.py:26-176, performance.py:26-90).

* ``Profiler``: ``torch.profiler`` window driven by ``profiler.*`` (enable, ranks, profile_steps, save_path); one
  chrome trace per profiled rank.
* ``mark_start_range / mark_end_range / mark_annotate``: NVTX ranges.
* ``DistProfiler.annotate``: decorator used on the DAG worker's node handlers; opens an NVTX range named after the
  role when profiling is enabled (on CUDA the reference's version is a no-op).
* ``GPUMemoryLogger`` / ``log_gpu_memory_usage``: allocator statistics before/after a call.
* ``CudaTimer``: device-side timing with CUDA events (the rule for every number this repo reports)."""
from __future__ import annotations

import functools
import os
from contextlib import contextmanager
from typing import Callable, Optional

import torch


class Profiler:
    def __init__(self, cfg, rank: int = 0):
        self.cfg = cfg
        self.rank = rank
        self.enabled = bool(cfg.enable) and (cfg.all_ranks or rank in list(cfg.ranks))
        self.steps = set(int(s) for s in cfg.profile_steps)
        self.prof = None

    def _make(self):
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        return torch.profiler.profile(activities=acts, record_shapes=self.cfg.record_shapes,
                                      profile_memory=self.cfg.with_memory, with_stack=self.cfg.with_stack)

    def start_step(self, step: int) -> None:
        if self.enabled and step in self.steps and self.prof is None:
            self.prof = self._make()
            self.prof.__enter__()

    def stop_step(self, step: int) -> Optional[str]:
        if self.prof is None or step not in self.steps:
            return None
        self.prof.__exit__(None, None, None)
        os.makedirs(self.cfg.save_path, exist_ok=True)
        path = os.path.join(self.cfg.save_path, f"trace_rank{self.rank}_step{step}.json")
        self.prof.export_chrome_trace(path)
        self.prof = None
        return path


def mark_start_range(message: Optional[str] = None):
    if torch.cuda.is_available():
        return torch.cuda.nvtx.range_start(message or "range")
    return None


def mark_end_range(range_id) -> None:
    if range_id is not None and torch.cuda.is_available():
        torch.cuda.nvtx.range_end(range_id)


def mark_annotate(message: Optional[str] = None) -> Callable:
    def deco(fn):
        @functools.wraps(fn)
        def wrapper(*a, **kw):
            rid = mark_start_range(message or fn.__name__)
            try:
                return fn(*a, **kw)
            finally:
                mark_end_range(rid)
        return wrapper
    return deco


class DistProfiler:
    enabled = bool(os.environ.get("SIIRL_ENABLE_PERF"))

    @staticmethod
    def annotate(role: Optional[str] = None, **_):
        def deco(fn):
            @functools.wraps(fn)
            def wrapper(*a, **kw):
                if not DistProfiler.enabled:
                    return fn(*a, **kw)
                rid = mark_start_range(role or fn.__name__)
                try:
                    return fn(*a, **kw)
                finally:
                    mark_end_range(rid)
            return wrapper
        return deco


def log_gpu_memory_usage(head: str, logger=print, rank: int = 0) -> dict:
    if not torch.cuda.is_available():
        return {}
    stats = {"allocated_gb": torch.cuda.memory_allocated() / 2 ** 30, "reserved_gb": torch.cuda.memory_reserved() / 2 ** 30,
             "max_allocated_gb": torch.cuda.max_memory_allocated() / 2 ** 30}
    if logger is not None:
        logger(f"[rank {rank}] {head}: " + ", ".join(f"{k}={v:.2f}" for k, v in stats.items()))
    return stats


class GPUMemoryLogger:
    def __init__(self, role: str, logger=print):
        self.role, self.logger = role, logger

    def __call__(self, fn):
        @functools.wraps(fn)
        def wrapper(*a, **kw):
            log_gpu_memory_usage(f"before {self.role}.{fn.__name__}", self.logger)
            out = fn(*a, **kw)
            log_gpu_memory_usage(f"after {self.role}.{fn.__name__}", self.logger)
            return out
        return wrapper


@contextmanager
def CudaTimer(sink: dict, name: str):
    """Device-side duration (ms) of the enclosed region on the current stream."""
    if not torch.cuda.is_available():
        import time
        t0 = time.perf_counter()
        yield
        sink[name] = (time.perf_counter() - t0) * 1e3
        return
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    yield
    e1.record()
    torch.cuda.synchronize()
    sink[name] = e0.elapsed_time(e1)
