"""DeepScaleR preview set (json with ``problem``, ``answer``) -> training parquet scored by the math rule.

    python examples/data_preprocess/deepscaler.py --src ~/raw/deepscaler.json --out ~/data/deepscaler
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _common import read_rows, row, write_split  # noqa: E402

SUFFIX = " Let's think step by step and output the final answer within \\boxed{}."

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", required=True)
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    rows = [row("math_dapo", ex["problem"] + SUFFIX, ex["answer"], "train", i) for i, ex in enumerate(read_rows(a.src))]
    write_split(rows, a.out, "train")
