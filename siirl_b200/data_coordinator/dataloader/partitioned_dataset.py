"""Rank-partitioned RLHF prompt dataset.

Behaviour of the reference dataset (siirl/data_coordinator/dataloader/partitioned_dataset.py:37-456): each
data-parallel rank reads only its slice of the parquet rows; when the row count does not divide evenly the
trailing ranks are padded with duplicates flagged ``padded_duplicate`` (validation skips them); prompts longer than
``max_prompt_length`` are filtered or truncated according to ``data.truncation``; items are chat-templated,
tokenised and LEFT-padded to ``max_prompt_length``; ``collate_fn`` stacks tensors and keeps the rest as object
arrays.  Synthetic datasets (``data.synthetic``) produce the same item dictionary without files.
"""
from __future__ import annotations

import random
from typing import Any, Dict, List, Optional

import torch
from torch.utils.data import Dataset

from ..protocol import Batch


def left_pad(ids: List[int], length: int, pad_id: int, truncation: str = "error"):
    if len(ids) > length:
        if truncation == "left":
            ids = ids[-length:]
        elif truncation == "right":
            ids = ids[:length]
        elif truncation == "middle":
            half = length // 2
            ids = ids[:half] + ids[-(length - half):]
        else:
            raise ValueError(f"prompt of {len(ids)} tokens exceeds max_prompt_length {length}")
    pad = length - len(ids)
    input_ids = torch.tensor([pad_id] * pad + ids, dtype=torch.int64)
    mask = torch.tensor([0] * pad + [1] * len(ids), dtype=torch.int64)
    pos = torch.clamp(torch.cumsum(mask, 0) - 1, min=0)
    return input_ids, mask, pos


def collate_fn(items: List[Dict[str, Any]]) -> Batch:
    tensors: Dict[str, List[torch.Tensor]] = {}
    non: Dict[str, List[Any]] = {}
    for it in items:
        for k, v in it.items():
            (tensors if isinstance(v, torch.Tensor) else non).setdefault(k, []).append(v)
    return Batch({k: torch.stack(v, 0) for k, v in tensors.items()}, non)


class PartitionedRLHFDataset(Dataset):
    def __init__(self, config, tokenizer, processor=None, ddp_rank: int = 0, ddp_world_size: int = 1,
                 is_eval: bool = False, drop_last: Optional[bool] = None):
        self.cfg = config.data if hasattr(config, "data") else config
        self.tokenizer = tokenizer
        self.processor = processor
        self.rank, self.world = ddp_rank, ddp_world_size
        self.is_eval = is_eval
        self.max_prompt_length = self.cfg.max_prompt_length
        self._full_config = config if hasattr(config, "actor_rollout_ref") else None
        self._vl = None
        self.rows: List[Dict[str, Any]] = []
        files = self.cfg.val_files if is_eval else self.cfg.train_files
        if isinstance(files, str):
            files = [files]
        if self.cfg.synthetic:
            self.rows = _synthetic_rows(self.cfg, tokenizer, is_eval)
            self._partition_rows(drop_last if drop_last is not None else not is_eval)
        else:
            self._load_parquet(list(files), drop_last if drop_last is not None else not is_eval)
        if self.cfg.filter_overlong_prompts or self.cfg.filter_overlong_prompt:
            self.rows = [r for r in self.rows if len(self._prompt_ids(r)) <= self.max_prompt_length]

    # ---- loading --------------------------------------------------------------------------------
    def _load_parquet(self, files: List[str], drop_last: bool) -> None:
        import os
        import pyarrow.parquet as pq
        total_rows, metas = 0, []
        for f in files:
            pf = pq.ParquetFile(os.path.expanduser(f))
            metas.append((pf, total_rows))
            total_rows += pf.metadata.num_rows
        lo, hi, pad = self._slice(total_rows, drop_last)
        rows: List[Dict[str, Any]] = []
        for pf, base in metas:
            n = pf.metadata.num_rows
            a, b = max(lo, base), min(hi, base + n)
            if a >= b:
                continue
            # read only the row groups that intersect [a, b)
            start = base
            for rg in range(pf.num_row_groups):
                m = pf.metadata.row_group(rg).num_rows
                if start + m > a and start < b:
                    tbl = pf.read_row_group(rg).to_pylist()
                    s, e = max(a - start, 0), min(b - start, m)
                    rows.extend(tbl[s:e])
                start += m
        for r in rows:
            r["padded_duplicate"] = False
        for i in range(pad):
            dup = dict(rows[i % len(rows)]) if rows else {}
            dup["padded_duplicate"] = True
            rows.append(dup)
        self.rows = rows

    def _slice(self, total: int, drop_last: bool):
        if drop_last:
            per = total // self.world
            return self.rank * per, (self.rank + 1) * per, 0
        per = (total + self.world - 1) // self.world
        lo = min(self.rank * per, total)
        hi = min(lo + per, total)
        return lo, hi, per - (hi - lo)

    def _partition_rows(self, drop_last: bool) -> None:
        lo, hi, pad = self._slice(len(self.rows), drop_last)
        rows = self.rows[lo:hi]
        for r in rows:
            r["padded_duplicate"] = False
        for i in range(pad):
            dup = dict(rows[i % len(rows)]) if rows else {}
            dup["padded_duplicate"] = True
            rows.append(dup)
        self.rows = rows

    # ---- items ----------------------------------------------------------------------------------
    def _prompt_ids(self, row: Dict[str, Any]) -> List[int]:
        if "prompt_ids" in row:
            return list(row["prompt_ids"])
        prompt = row[self.cfg.prompt_key]
        if isinstance(prompt, str):
            return self.tokenizer.encode(prompt, add_special_tokens=False)
        text = self.tokenizer.apply_chat_template(list(prompt), add_generation_prompt=True, tokenize=False)
        return self.tokenizer.encode(text, add_special_tokens=False)

    def __len__(self) -> int:
        return len(self.rows)

    def _vl_processor(self):
        """Image processor of the policy's vision tower (built on first use from the model configuration)."""
        if self._vl is None:
            from ...models.config import get_config
            from ...models.vision_processor import make_vl_processor
            m = self._full_config.actor_rollout_ref.model
            mcfg = get_config(m.arch_preset or m.path, dict(m.override_config or {}))
            if mcfg.vision is None and mcfg.vit is None and mcfg.moonvit is None:
                raise ValueError("the dataset has images but the model has no vision tower")
            self._vl = make_vl_processor(mcfg, m.image_min_pixels, m.image_max_pixels)
        return self._vl

    def __getitem__(self, idx: int) -> Dict[str, Any]:
        row = self.rows[idx]
        ids = self._prompt_ids(row)
        mm_inputs = None
        images = row.get(self.cfg.image_key) if self.cfg.image_key in row else None
        videos = row.get(self.cfg.video_key) if self.cfg.video_key in row else None
        has_img = images is not None and len(images) > 0
        has_vid = videos is not None and len(videos) > 0
        if (has_img or has_vid) and self._full_config is not None:
            frames = []
            if has_vid:
                from .vision_utils import process_video
                m = self._full_config.actor_rollout_ref.model
                # videos have pixel limits and a frame budget of their own (the reference's processor keys,
                # siirl/data_coordinator/dataloader/partitioned_dataset.py:136-139, 355-358)
                frames = [v if isinstance(v, torch.Tensor) and v.dim() == 4 else
                          process_video(v if isinstance(v, dict) else {"video": v}, fps=m.video_fps,
                                        fps_max_frames=m.video_maxlen, max_pixels=m.video_max_pixels,
                                        min_pixels=m.video_min_pixels) for v in videos]
            out = self._vl_processor()(ids, list(images) if has_img else [], frames)
            ids = out["input_ids"]
            mm_inputs = {"pixel_values": out["pixel_values"], "image_grid_thw": out["image_grid_thw"]}
        input_ids, mask, pos = left_pad(ids, self.max_prompt_length, self.tokenizer.pad_token_id, self.cfg.truncation)
        item: Dict[str, Any] = {
            "input_ids": input_ids, "attention_mask": mask, "position_ids": pos,
            "raw_prompt_ids": ids[-self.max_prompt_length:],
            "data_source": row.get(self.cfg.reward_fn_key, row.get("data_source", "unknown")),
            "reward_model": row.get("reward_model", {}), "extra_info": row.get("extra_info", {}) or {},
            "index": (row.get("extra_info") or {}).get("index", idx),
            "padded_duplicate": bool(row.get("padded_duplicate", False)),
        }
        if mm_inputs is not None:
            item["multi_modal_inputs"] = mm_inputs       # per-sample dict: ragged, travels as a non-tensor field
        if "pixel_values" in row:
            item["pixel_values"] = row["pixel_values"]
            item["image_grid_thw"] = row["image_grid_thw"]
        for k in ("task_id", "trial_id"):          # embodied task-list rows
            if k in row:
                item[k] = torch.tensor(int(row[k]), dtype=torch.int64)
        if self.cfg.return_raw_chat:
            item["raw_prompt"] = row.get(self.cfg.prompt_key)
        for k in ("tools_kwargs", "interaction_kwargs"):
            if k in (row.get("extra_info") or {}):
                item[k] = row["extra_info"][k]
        return item


def _synthetic_rows(cfg, tokenizer, is_eval: bool) -> List[Dict[str, Any]]:
    """Seeded synthetic prompt sets.

    ``arith``  : "a+b=" digit prompts, ground truth = digits of the sum (exact-match reward);
    ``random`` : uniform random token ids of uniform random length (throughput benchmarks);
    ``parity`` : like ``random``; the reward function looks only at the last generated token."""
    rng = random.Random(1234 + (7 if is_eval else 0))
    kind = cfg.synthetic
    n = cfg.synthetic_size if not is_eval else max(8, cfg.synthetic_size // 16)
    lo, hi = cfg.synthetic_min_prompt, min(cfg.synthetic_max_prompt, cfg.max_prompt_length)
    rows = []
    vocab = len(tokenizer)
    for i in range(n):
        if kind == "arith":
            a, b = rng.randint(0, 10 ** 6), rng.randint(0, 10 ** 6)
            text = f"{a}+{b}="
            ids = tokenizer.encode(text)
            want = max(lo, len(ids))
            ids = [tokenizer.encode(" ")[0]] * (rng.randint(want, max(want, hi)) - len(ids)) + ids
            rows.append({"prompt_ids": ids, "data_source": "synthetic/arith",
                         "reward_model": {"style": "rule", "ground_truth": str(a + b)}, "extra_info": {"index": i}})
        elif kind in ("random", "parity", "bernoulli"):
            L = rng.randint(lo, hi)
            ids = [rng.randint(3, vocab - 1) for _ in range(L)]
            rows.append({"prompt_ids": ids, "data_source": f"synthetic/{kind}",
                         "reward_model": {"style": "rule", "ground_truth": ""},
                         "extra_info": {"index": i, "seed": rng.randint(0, 2 ** 31)}})
        elif kind == "vl":
            L = rng.randint(lo, hi)
            ids = [rng.randint(3, min(vocab, 1000) - 1) for _ in range(L)]
            side = cfg.synthetic_image_size
            img = torch.randint(0, 256, (side, side, 3), dtype=torch.uint8,
                                generator=torch.Generator().manual_seed(rng.randint(0, 2 ** 31)))
            rows.append({"prompt_ids": ids, "images": [img], "data_source": "synthetic/parity",
                         "reward_model": {"style": "rule", "ground_truth": ""},
                         "extra_info": {"index": i, "seed": rng.randint(0, 2 ** 31)}})
        elif kind == "embodied":
            ids = tokenizer.encode(f"task {i % 10}")
            rows.append({"prompt_ids": ids, "data_source": "embodied/synthetic", "task_id": i % 10,
                         "trial_id": i // 10, "reward_model": {"style": "rule", "ground_truth": ""},
                         "extra_info": {"index": i}})
        else:
            raise ValueError(f"unknown synthetic dataset '{kind}'")
    return rows

