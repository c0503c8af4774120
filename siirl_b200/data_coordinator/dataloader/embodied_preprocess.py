"""Task-list dataset for embodied training (reference: siirl/data_coordinator/dataloader/embodied_preprocess.py):
one row per (task, trial) of a benchmark suite, written as parquet with the columns the dataset reads
(``task_id``, ``trial_id``, a text ``prompt`` and ``data_source``).

    python -m siirl_b200.data_coordinator.dataloader.embodied_preprocess --suite libero_10 --out data/libero_10
"""
from __future__ import annotations

import argparse
import os
from typing import Dict, List

SUITE_TASKS = {"libero_spatial": 10, "libero_object": 10, "libero_goal": 10, "libero_10": 10, "libero_90": 90,
               "synthetic": 10}


def build_rows(suite: str, num_trials_per_task: int, split: str = "train", val_fraction: float = 0.1) -> List[Dict]:
    n_tasks = SUITE_TASKS.get(suite)
    if n_tasks is None:
        raise ValueError(f"unknown suite '{suite}' (known: {sorted(SUITE_TASKS)})")
    n_val = max(1, int(round(num_trials_per_task * val_fraction)))
    trials = range(num_trials_per_task - n_val) if split == "train" else range(num_trials_per_task - n_val,
                                                                                num_trials_per_task)
    return [{"task_id": t, "trial_id": k, "prompt": f"{suite} task {t}", "data_source": f"embodied/{suite}",
             "reward_model": {"style": "rule", "ground_truth": ""}, "extra_info": {"index": t * num_trials_per_task + k,
                                                                                   "suite": suite, "split": split}}
            for t in range(n_tasks) for k in trials]


def write_parquet(rows: List[Dict], path: str) -> None:
    import pandas as pd
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    pd.DataFrame(rows).to_parquet(path)


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--suite", default="libero_10")
    ap.add_argument("--num-trials-per-task", type=int, default=50)
    ap.add_argument("--out", required=True)
    a = ap.parse_args(argv)
    for split in ("train", "val"):
        rows = build_rows(a.suite, a.num_trials_per_task, split)
        write_parquet(rows, os.path.join(a.out, f"{split}.parquet"))
        print(f"{split}: {len(rows)} rows -> {os.path.join(a.out, split + '.parquet')}")


if __name__ == "__main__":
    main()
