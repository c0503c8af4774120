"""Out-of-band metric aggregation: ranks post their step metrics and carry on; a collector thread on rank 0 merges them
and hands the result to the loggers.

The reference runs a ``MetricWorker`` Ray actor with an asyncio queue: every rank's ``MetricClient.submit_metric``
pushes its local scalars, the actor reduces a key once the expected number of submissions has arrived (by name:
``min`` / ``max`` / ``sum|total``, else mean) and ``wait_final_res`` returns the merged dict to rank 0
(siirl/execution/metric_worker/metric_worker.py:34-274, utils.py:29-62).  There is no actor system here; the transport
is the key-value store that ``torch.distributed`` already keeps for rendezvous (a TCP store served by rank 0):

* ``MetricClient.submit_metric(metrics, step)``: one ``store.set`` of a JSON blob: no collective, no device sync, so
  the training loop does not wait for the slowest rank's logging;
* ``MetricWorker`` (rank 0): a thread that waits for the ``world`` blobs of every announced step, merges them with the
  same name convention as the in-band reduction (``utils/metrics/metric_utils.py::reduce_kind``), adds the fields
  that are not reduced (step, epoch) and calls ``sink(merged, step)`` (the tracker).  ``wait_final_res`` blocks until
  a step (or everything announced) has been delivered.
"""
from __future__ import annotations

import json
import math
import queue
import threading
from datetime import timedelta
from typing import Any, Callable, Dict, List, Optional

from ...utils.metrics.metric_utils import reduce_kind

_PREFIX = "metric_worker"


def merge_rank_metrics(per_rank: List[Dict[str, float]]) -> Dict[str, float]:
    """Name-convention merge of the ranks' scalars; a key missing on some ranks is merged over those that have it."""
    out: Dict[str, float] = {}
    for k in sorted({k for d in per_rank for k in d}):
        vals = [float(d[k]) for d in per_rank if k in d and d[k] is not None and not math.isnan(float(d[k]))]
        if not vals:
            continue
        kind = reduce_kind(k)
        out[k] = max(vals) if kind == "max" else min(vals) if kind == "min" else sum(vals) if kind == "sum" \
            else sum(vals) / len(vals)
    return out


def default_store():
    """The process group's rendezvous store (``None`` outside an initialised job)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return None
    from torch.distributed.distributed_c10d import _get_default_store
    return dist.PrefixStore(_PREFIX, _get_default_store())


class MetricClient:
    def __init__(self, store, rank: int):
        self.store, self.rank = store, rank

    def submit_metric(self, metrics: Dict[str, Any], step: int) -> None:
        numeric = {k: float(v) for k, v in metrics.items() if isinstance(v, (int, float)) and not isinstance(v, bool)}
        self.store.set(f"{step}/{self.rank}", json.dumps(numeric))


class MetricWorker(threading.Thread):
    def __init__(self, store, world: int, sink: Optional[Callable[[Dict[str, float], int], None]] = None,
                 timeout_s: float = 600.0):
        super().__init__(daemon=True, name="metric-worker")
        self.store, self.world, self.sink, self.timeout_s = store, world, sink, timeout_s
        self._todo: "queue.Queue[Optional[tuple]]" = queue.Queue()
        self._done: Dict[int, Dict[str, float]] = {}
        self._errors: Dict[int, str] = {}
        self._cv = threading.Condition()
        self._announced = 0
        self.start()

    def expect(self, step: int, extra: Optional[Dict[str, float]] = None) -> None:
        """Announce that all ranks post metrics for ``step``; ``extra`` entries are added to the merged dict as is."""
        with self._cv:
            self._announced += 1
        self._todo.put((int(step), dict(extra or {})))

    def run(self) -> None:
        while True:
            item = self._todo.get()
            if item is None:
                return
            step, extra = item
            keys = [f"{step}/{r}" for r in range(self.world)]
            try:
                self.store.wait(keys, timedelta(seconds=self.timeout_s))
                merged = merge_rank_metrics([json.loads(self.store.get(k).decode()) for k in keys])
                merged.update(extra)
                for k in keys:
                    try:
                        self.store.delete_key(k)
                    except Exception:  # noqa: BLE001  (stores without deletion keep the blobs: a few KB per step)
                        break
                if self.sink is not None:
                    self.sink(merged, step)
                with self._cv:
                    self._done[step] = merged
                    self._cv.notify_all()
            except Exception as e:  # noqa: BLE001
                with self._cv:
                    self._errors[step] = f"{type(e).__name__}: {e}"
                    self._done[step] = {}
                    self._cv.notify_all()

    def wait_final_res(self, step: Optional[int] = None, timeout_s: Optional[float] = None) -> Dict[str, float]:
        """Merged metrics of ``step``; with ``step=None`` waits for everything announced and returns the last one."""
        with self._cv:
            ok = self._cv.wait_for(lambda: (step in self._done) if step is not None
                                   else len(self._done) >= self._announced, timeout=timeout_s or self.timeout_s)
            if not ok:
                raise TimeoutError(f"metric worker: step {step if step is not None else 'all'} not delivered")
            if step is None:
                return self._done[max(self._done)] if self._done else {}
            if step in self._errors:
                raise RuntimeError(f"metric worker failed on step {step}: {self._errors[step]}")
            return self._done[step]

    def close(self, timeout_s: Optional[float] = None) -> None:
        """Deliver what is outstanding, then stop the thread."""
        try:
            self.wait_final_res(None, timeout_s)
        finally:
            self._todo.put(None)
            self.join(timeout=5.0)
