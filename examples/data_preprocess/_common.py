"""Shared helpers of the data-preparation scripts: read local json / json-lines / parquet, write the training
schema (``prompt`` chat messages, ``data_source``, ``reward_model.ground_truth``, ``extra_info``, optional
``images``).  Nothing is downloaded: ``--src`` points at files obtained beforehand."""
import json
import os

import pandas as pd


def read_rows(path):
    if path.endswith(".parquet"):
        return pd.read_parquet(path).to_dict("records")
    with open(path) as f:
        if path.endswith(".jsonl"):
            return [json.loads(line) for line in f if line.strip()]
        return json.load(f)


def write_split(rows, out_dir, split):
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, f"{split}.parquet")
    pd.DataFrame(rows).to_parquet(path)
    print(f"{split}: {len(rows)} rows -> {path}")


def row(data_source, question, truth, split, index, ability="math", images=None, extra=None):
    r = {"data_source": data_source, "prompt": [{"role": "user", "content": question}], "ability": ability,
         "reward_model": {"style": "rule", "ground_truth": str(truth)},
         "extra_info": {"split": split, "index": index, **(extra or {})}}
    if images is not None:
        r["images"] = images
    return r
