"""Metric definitions (key names documented by the reference, docs/user_interface/metrics_interface.rst:132-242;
formulas of siirl/utils/metrics/metric_utils.py:70-258): data metrics (scores, rewards, advantages, returns,
values, response/prompt lengths and clip ratios), timing metrics (``timing_s/*``, ``timing_per_token_ms/*``) and
throughput (``perf/throughput`` = tokens / (step time * n_gpus)).  Reduction across ranks is chosen from the key
name: contains ``max`` -> MAX, ``min`` -> MIN, ``sum``/``total`` -> SUM, otherwise mean
(siirl/execution/metric_worker/utils.py:29-62)."""
from __future__ import annotations

from typing import Any, Dict, List

import numpy as np
import torch
import torch.distributed as dist


def _masked_mean(x, m):
    return (x * m).sum() / m.sum().clamp(min=1)


def compute_data_metric(batch, use_critic: bool = False) -> Dict[str, float]:
    m: Dict[str, float] = {}
    mask = batch["response_mask"].float()
    R = mask.shape[-1]
    valid = mask.bool()
    if "token_level_scores" in batch:
        s = batch["token_level_scores"].float().sum(-1)
        m.update({"critic/score/mean": s.mean().item(), "critic/score/max": s.max().item(),
                  "critic/score/min": s.min().item()})
    if "token_level_rewards" in batch:
        r = batch["token_level_rewards"].float().sum(-1)
        m.update({"critic/rewards/mean": r.mean().item(), "critic/rewards/max": r.max().item(),
                  "critic/rewards/min": r.min().item()})
    if "advantages" in batch and valid.any():
        a = batch["advantages"].float()[valid]
        m.update({"critic/advantages/mean": a.mean().item(), "critic/advantages/max": a.max().item(),
                  "critic/advantages/min": a.min().item()})
    if "returns" in batch and valid.any():
        rt = batch["returns"].float()[valid]
        m.update({"critic/returns/mean": rt.mean().item(), "critic/returns/max": rt.max().item(),
                  "critic/returns/min": rt.min().item()})
    if use_critic and "values" in batch and valid.any():
        v = batch["values"].float()[valid]
        rt = batch["returns"].float()[valid]
        m.update({"critic/values/mean": v.mean().item(), "critic/values/max": v.max().item(),
                  "critic/values/min": v.min().item(),
                  "critic/vf_explained_var": (1.0 - (rt - v).var() / (rt.var() + 1e-5)).item()})
    rl = mask.sum(-1)
    m.update({"response_length/mean": rl.mean().item(), "response_length/max": rl.max().item(),
              "response_length/min": rl.min().item(), "response_length/clip_ratio": (rl >= R).float().mean().item()})
    if "attention_mask" in batch:
        P = batch["attention_mask"].shape[-1] - R
        pl = batch["attention_mask"][:, :P].float().sum(-1)
        m.update({"prompt_length/mean": pl.mean().item(), "prompt_length/max": pl.max().item(),
                  "prompt_length/min": pl.min().item(), "prompt_length/clip_ratio": (pl >= P).float().mean().item()})
    return m


def compute_timing_metrics(batch, timing_raw: Dict[str, float]) -> Dict[str, float]:
    mask = batch["response_mask"]
    n_resp = float(mask.sum())
    n_all = float(batch["attention_mask"].sum()) if "attention_mask" in batch else n_resp
    tokens_of = {"gen": n_resp, "generate": n_resp}
    out = {f"timing_s/{k}": v for k, v in timing_raw.items()}
    for k, v in timing_raw.items():
        out[f"timing_per_token_ms/{k}"] = v * 1000.0 / max(tokens_of.get(k, n_all), 1.0)
    return out


def compute_throughput_metrics(batch, timing_raw: Dict[str, float], n_gpus: int) -> Dict[str, float]:
    total = float(sum(batch.meta.get("global_token_num", []))) if "global_token_num" in batch.meta else \
        float(batch["attention_mask"].sum())
    t = timing_raw.get("step", 1e-9)
    return {"perf/total_num_tokens": total, "perf/time_per_step": t, "perf/throughput": total / (t * max(n_gpus, 1))}


def reduce_kind(key: str) -> str:
    k = key.lower()
    if "max" in k:
        return "max"
    if "min" in k:
        return "min"
    if "sum" in k or "total" in k:
        return "sum"
    return "mean"


def reduce_metrics_across_ranks(metrics: Dict[str, float], group=None) -> Dict[str, float]:
    """One packed all-reduce per reduction kind (reference: DistributedMetricAggregator,
    siirl/dag_worker/metric_aggregator.py:54-211).  Keys may differ between ranks: the union is used."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return dict(metrics)
    world = dist.get_world_size(group)
    all_keys: List[Any] = [None] * world
    dist.all_gather_object(all_keys, sorted(metrics), group=group)
    keys = sorted({k for ks in all_keys for k in ks})
    backend = dist.get_backend(group)
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    out: Dict[str, float] = {}
    for kind, op in (("mean", dist.ReduceOp.SUM), ("sum", dist.ReduceOp.SUM), ("max", dist.ReduceOp.MAX),
                     ("min", dist.ReduceOp.MIN)):
        ks = [k for k in keys if reduce_kind(k) == kind]
        if not ks:
            continue
        fill = {"mean": 0.0, "sum": 0.0, "max": -float("inf"), "min": float("inf")}[kind]
        vals = torch.tensor([float(metrics.get(k, fill)) for k in ks] +
                            ([float(k in metrics) for k in ks] if kind == "mean" else []), dtype=torch.float64,
                            device=dev)
        dist.all_reduce(vals, op=op, group=group)
        vals = vals.cpu().tolist()
        for i, k in enumerate(ks):
            out[k] = vals[i] / max(vals[len(ks) + i], 1.0) if kind == "mean" else vals[i]
    return out


def process_validation_metrics(data_sources: List[str], sample_inputs: List[str],
                               infos: Dict[str, List[Any]], seed: int = 42) -> Dict[str, Dict[str, Dict[str, float]]]:
    """Per data source and variable: mean@N, std@N, best@N / worst@N (bootstrap), maj@N when predictions exist
    (reference: metric_utils.py:461-598)."""
    from collections import defaultdict
    by = defaultdict(lambda: defaultdict(lambda: defaultdict(list)))
    for i, ds in enumerate(data_sources):
        for var, vals in infos.items():
            if i < len(vals) and isinstance(vals[i], (int, float, bool, np.floating, np.integer)):
                by[ds][sample_inputs[i]][var].append(float(vals[i]))
    rng = np.random.RandomState(seed)
    out: Dict[str, Dict[str, Dict[str, float]]] = {}
    for ds, prompts in by.items():
        agg = defaultdict(lambda: defaultdict(list))
        for _, var2vals in prompts.items():
            for var, vals in var2vals.items():
                n = len(vals)
                agg[var][f"mean@{n}"].append(float(np.mean(vals)))
                if n > 1:
                    agg[var][f"std@{n}"].append(float(np.std(vals)))
                    boots = [rng.choice(vals, size=n, replace=True) for _ in range(100)]
                    agg[var][f"best@{n}/mean"].append(float(np.mean([b.max() for b in boots])))
                    agg[var][f"worst@{n}/mean"].append(float(np.mean([b.min() for b in boots])))
        out[ds] = {var: {k: float(np.mean(v)) for k, v in d.items()} for var, d in agg.items()}
    return out
