"""MATH (lighteval/MATH layout: ``problem``, ``solution`` with a final \\boxed{} answer) -> training parquet.

    python examples/data_preprocess/math_dataset.py --src ~/raw/math --out ~/data/math
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _common import read_rows, row, write_split  # noqa: E402

from siirl_b200.utils.reward_score.math import last_boxed_only_string, remove_boxed  # noqa: E402

SUFFIX = " Let's think step by step and output the final answer within \\boxed{}."

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", required=True)
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    for split in ("train", "test"):
        src = next(p for p in (os.path.join(a.src, f"{split}{e}") for e in (".jsonl", ".json", ".parquet")) if os.path.exists(p))
        out = []
        for i, ex in enumerate(read_rows(src)):
            boxed = last_boxed_only_string(ex["solution"])
            out.append(row("lighteval/MATH", ex["problem"] + SUFFIX, remove_boxed(boxed) if boxed else "", split, i))
        write_split(out, a.out, split)
