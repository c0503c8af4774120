"""Out-of-band metric aggregation over a key-value store."""
import threading
import time

import pytest
import torch.distributed as dist

from siirl_b200.execution.metric_worker import MetricClient, MetricWorker, merge_rank_metrics


def test_merge_follows_the_name_convention():
    m = merge_rank_metrics([{"timing_s/step": 1.0, "perf/max_memory_gb": 3.0, "response_length/min": 5, "perf/total_num_tokens": 10},
                            {"timing_s/step": 3.0, "perf/max_memory_gb": 7.0, "response_length/min": 2, "perf/total_num_tokens": 20,
                             "actor/only_here": 4.0}])
    assert m == {"timing_s/step": 2.0, "perf/max_memory_gb": 7.0, "response_length/min": 2.0, "perf/total_num_tokens": 30.0,
                 "actor/only_here": 4.0}


def test_worker_collects_steps_posted_in_any_order():
    store = dist.HashStore()
    got = []
    worker = MetricWorker(store, world=3, sink=lambda m, s: got.append((s, m)), timeout_s=20.0)
    clients = [MetricClient(store, r) for r in range(3)]
    worker.expect(1, {"training/global_step": 1})
    worker.expect(2, {"training/global_step": 2})

    def late():
        time.sleep(0.2)
        clients[2].submit_metric({"a/x": 9.0, "a/x_max": 9.0, "flag": True, "name": "skip me"}, 1)
    t = threading.Thread(target=late)
    t.start()
    for r in (0, 1):
        clients[r].submit_metric({"a/x": float(r), "a/x_max": float(r)}, 1)
    for r in range(3):
        clients[r].submit_metric({"a/x": 10.0 * r}, 2)       # step 2 is complete before step 1
    assert worker.wait_final_res(1) == {"a/x": 10.0 / 3, "a/x_max": 9.0, "training/global_step": 1}
    assert worker.wait_final_res(None)["a/x"] == 10.0
    t.join()
    worker.close()
    assert [s for s, _ in got] == [1, 2]                     # delivered in the order the steps were announced


def test_missing_rank_times_out_with_a_message():
    store = dist.HashStore()
    worker = MetricWorker(store, world=2, timeout_s=0.5)
    MetricClient(store, 0).submit_metric({"a": 1.0}, 7)
    worker.expect(7)
    with pytest.raises(RuntimeError, match="step 7"):
        worker.wait_final_res(7, timeout_s=5.0)
    worker._todo.put(None)
