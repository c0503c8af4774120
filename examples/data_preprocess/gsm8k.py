"""GSM8K -> parquet rows in the training schema (prompt as chat messages, rule-based reward with the final number).
Reads the dataset's json-lines files (``question`` / ``answer`` fields) from ``--src``; no download is attempted.

    python examples/data_preprocess/gsm8k.py --src ~/raw/gsm8k --out ~/data/gsm8k
"""
import argparse
import json
import os
import re

import pandas as pd

SUFFIX = " Let's think step by step and output the final answer after \"####\"."


def rows(path, split):
    out = []
    with open(path) as f:
        for i, line in enumerate(f):
            ex = json.loads(line)
            m = re.search(r"#### (\-?[0-9\.\,]+)", ex["answer"])
            truth = m.group(1).replace(",", "") if m else ""
            out.append({"data_source": "openai/gsm8k", "prompt": [{"role": "user", "content": ex["question"] + SUFFIX}],
                        "ability": "math", "reward_model": {"style": "rule", "ground_truth": truth},
                        "extra_info": {"split": split, "index": i}})
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", required=True)
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    os.makedirs(a.out, exist_ok=True)
    for split in ("train", "test"):
        pd.DataFrame(rows(os.path.join(a.src, f"{split}.jsonl"), split)).to_parquet(os.path.join(a.out, f"{split}.parquet"))
