"""Geometry3K (``problem``, ``answer``, ``images``) -> training parquet with image prompts for the VL models.

    python examples/data_preprocess/geo3k.py --src ~/raw/geometry3k --out ~/data/geo3k
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _common import read_rows, row, write_split  # noqa: E402

SUFFIX = (" You FIRST think about the reasoning process as an internal monologue and then provide the final answer. "
          "The final answer MUST BE put in \\boxed{}.")

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", required=True)
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    for split in ("train", "test"):
        out = []
        for i, ex in enumerate(read_rows(os.path.join(a.src, f"{split}.parquet"))):
            out.append(row("hiyouga/geometry3k", ex["problem"] + SUFFIX, ex["answer"], split, i,
                           images=list(ex["images"])))
        write_split(out, a.out, split)
