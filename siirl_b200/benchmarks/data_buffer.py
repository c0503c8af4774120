"""Put / get throughput of the Data Coordinator on one process (the reference's
tests/data_buffer/performance_test_data_buffer.py workload: 1600 samples of 1024 tokens with a 1024-wide float
feature, batches of 128).

    python -m siirl_b200.benchmarks.data_buffer [--samples 1600] [--seq 1024] [--embed 1024] [--batch 128]
"""
from __future__ import annotations

import argparse
import json
import time

import torch

from ..data_coordinator import DataCoordinator
from ..data_coordinator.sample import Sample, SampleInfo


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--samples", type=int, default=1600)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--embed", type=int, default=1024)
    ap.add_argument("--batch", type=int, default=128)
    a = ap.parse_args()
    dc = DataCoordinator(1, 0, 1)
    samples = [Sample({"input_ids": torch.randint(0, 32000, (a.seq,)), "feat": torch.randn(a.embed)}, {"i": i}, {})
               for i in range(a.samples)]
    infos = [SampleInfo(sum_tokens=a.seq, dict_info={"key": "k"}) for _ in range(a.samples)]
    t0 = time.perf_counter()
    for i in range(0, a.samples, a.batch):
        dc.put_batch(infos[i:i + a.batch], samples[i:i + a.batch], caller_node_id="k")
    t_put = time.perf_counter() - t0
    t0 = time.perf_counter()
    got = 0
    while True:
        b = dc.get_batch(a.batch, 0, lambda info: info.dict_info.get("key") == "k", None)
        if not b:
            break
        got += len(b)
    t_get = time.perf_counter() - t0
    nbytes = a.samples * (a.seq * 8 + a.embed * 4)
    print(json.dumps({"samples": a.samples, "put_samples_per_s": round(a.samples / t_put), "get_samples_per_s":
                      round(got / max(t_get, 1e-9)), "payload_mb": round(nbytes / 2 ** 20, 1), "got": got}))


if __name__ == "__main__":
    main()
