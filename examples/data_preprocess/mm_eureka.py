"""MM-Eureka (json-lines with ``question``, ``answer``, ``image_urls`` pointing at local files) -> training parquet.

    python examples/data_preprocess/mm_eureka.py --src ~/raw/mm_eureka/dataset.jsonl --out ~/data/mm_eureka
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _common import read_rows, row, write_split  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--val-fraction", type=float, default=0.02)
    a = ap.parse_args()
    base = os.path.dirname(os.path.abspath(a.src))
    rows = []
    for i, ex in enumerate(read_rows(a.src)):
        imgs = []
        for p in ex.get("image_urls", []):
            with open(p if os.path.isabs(p) else os.path.join(base, p), "rb") as f:
                imgs.append({"bytes": f.read()})
        rows.append(row("mm_eureka", ex["question"], ex["answer"].replace("$", ""), "train", i, images=imgs))
    n_val = max(1, int(len(rows) * a.val_fraction))
    write_split(rows[n_val:], a.out, "train")
    write_split(rows[:n_val], a.out, "test")
