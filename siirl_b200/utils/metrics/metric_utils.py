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
    """How a metric is merged over ranks, from the words of its name (split at ``/ _ @ . -``): ``max``, ``min``,
    ``sum`` / ``total``, else the mean.  Whole words only: ``timing_s/step`` is a mean although "timing" contains
    "min"."""
    import re
    words = set(re.split(r"[/_@.\-]+", key.lower()))
    if "max" in words:
        return "max"
    if "min" in words:
        return "min"
    if "sum" in words or "total" in words:
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


def bootstrap_metric(data: List[Any], subset_size: int, reduce_fns, n_bootstrap: int = 1000, seed: int = 42):
    """Mean and standard deviation of each ``reduce_fn`` over ``n_bootstrap`` resamples (with replacement) of
    ``subset_size`` items (reference: metric_utils.py:385-425; 1000 resamples, seed 42)."""
    rng = np.random.RandomState(seed)
    idx = rng.randint(0, len(data), size=(n_bootstrap, subset_size))
    out = []
    for fn in reduce_fns:
        vals = [fn([data[j] for j in row]) for row in idx]
        out.append((float(np.mean(vals)), float(np.std(vals))))
    return out


def calc_maj_val(data: List[Dict[str, Any]], vote_key: str, val_key: str) -> float:
    """Value of the first item that carries the most frequent ``vote_key`` (majority voting over the predictions of
    one prompt; reference: metric_utils.py:427-458)."""
    votes: Dict[Any, List[Any]] = {}
    for d in data:
        votes.setdefault(d[vote_key], []).append(d[val_key])
    best = max(votes, key=lambda k: len(votes[k]))
    return votes[best][0]


def process_validation_metrics(data_sources: List[str], sample_inputs: List[str],
                               infos: Dict[str, List[Any]], seed: int = 42,
                               n_bootstrap: int = 1000) -> Dict[str, Dict[str, Dict[str, float]]]:
    """Per data source and variable, averaged over prompts: ``mean@N``, ``std@N`` and, for N > 1 samples per prompt and
    subset sizes n = 2, 4, 8, ... , N, the bootstrap estimates ``best@n/mean|std``, ``worst@n/mean|std`` and, when
    ``infos`` has a ``pred`` column, ``maj@n/mean|std`` (majority vote over the predictions, scored with the variable
    of the winning prediction) -- reference: metric_utils.py:461-598."""
    from collections import defaultdict
    by = defaultdict(lambda: defaultdict(lambda: defaultdict(list)))
    preds = infos.get("pred")
    for i, ds in enumerate(data_sources):
        for var, vals in infos.items():
            if var == "pred":
                continue
            if i < len(vals) and isinstance(vals[i], (int, float, bool, np.floating, np.integer)):
                by[ds][sample_inputs[i]][var].append(float(vals[i]))
        if preds is not None and i < len(preds):
            by[ds][sample_inputs[i]]["__pred__"].append(preds[i])
    out: Dict[str, Dict[str, Dict[str, float]]] = {}
    for ds, prompts in by.items():
        agg = defaultdict(lambda: defaultdict(list))
        for _, var2vals in prompts.items():
            votes = var2vals.get("__pred__")
            for var, vals in var2vals.items():
                if var == "__pred__":
                    continue
                n = len(vals)
                agg[var][f"mean@{n}"].append(float(np.mean(vals)))
                if n <= 1:
                    continue
                agg[var][f"std@{n}"].append(float(np.std(vals)))
                sizes, k = [], 2
                while k < n:
                    sizes.append(k)
                    k *= 2
                sizes.append(n)
                for k in sizes:
                    (bm, bs), (wm, ws) = bootstrap_metric(vals, k, [np.max, np.min], n_bootstrap, seed)
                    agg[var][f"best@{k}/mean"].append(bm)
                    agg[var][f"best@{k}/std"].append(bs)
                    agg[var][f"worst@{k}/mean"].append(wm)
                    agg[var][f"worst@{k}/std"].append(ws)
                    if votes is not None and len(votes) == n:
                        pairs = [{"val": v, "pred": p} for v, p in zip(vals, votes)]
                        (mm, ms), = bootstrap_metric(pairs, k, [lambda d: calc_maj_val(d, "pred", "val")],
                                                     n_bootstrap, seed)
                        agg[var][f"maj@{k}/mean"].append(mm)
                        agg[var][f"maj@{k}/std"].append(ms)
        out[ds] = {var: {k: float(np.mean(v)) for k, v in d.items()} for var, d in agg.items()}
    return out


# ---------------------------------------------------------------------------------------------------------------
# per-rank performance records (reference: siirl/dag_worker/dag_utils.py:684-876)
# ---------------------------------------------------------------------------------------------------------------
def write_rank_performance_csv(metrics: Dict[str, Any], step: int, rank: int, world: int, out_dir: str,
                               group=None) -> str:
    """Gather every rank's (unreduced) metric dict on rank 0 and write one CSV per step: a row per metric key common
    to all ranks, a column per rank, then ``max, min, delta_max_min, delta_max_rank_0`` -- the table that shows which
    rank is the straggler of a node.  Returns the path on rank 0, "" elsewhere."""
    import csv
    import os
    numeric = {k: float(v) for k, v in metrics.items() if isinstance(v, (int, float, np.floating, np.integer))}
    gathered: List[Any] = [numeric]
    if dist.is_available() and dist.is_initialized() and world > 1:
        gathered = [None] * world if rank == 0 else None
        dist.gather_object(numeric, gathered, dst=dist.get_global_rank(group, 0) if group is not None else 0,
                           group=group)
    if rank != 0:
        return ""
    rows = [m for m in gathered if isinstance(m, dict)]
    if not rows:
        return ""
    common = set(rows[0])
    for m in rows[1:]:
        common &= set(m)
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, f"world_{world}_step_{step}_common_metrics.csv")
    with open(path, "w", newline="", encoding="utf-8") as f:
        w = csv.writer(f)
        w.writerow(["metric"] + [f"rank_{i}" for i in range(len(rows))] + ["max", "min", "delta_max_min",
                                                                         "delta_max_rank_0"])
        for k in sorted(common):
            vals = [m[k] for m in rows]
            w.writerow([k] + vals + [max(vals), min(vals), max(vals) - min(vals), max(vals) - vals[0]])
    return path


def format_core_performance_metrics(metrics: Dict[str, Any], step: int, enable_perf: bool = True) -> str:
    """Plain-text summary of one step for the console: step time and throughput, reward / score statistics, per-node
    timings, MFU, memory and sequence lengths."""
    def g(key, prec=3):
        v = metrics.get(key)
        if v is None:
            return "N/A"
        return f"{v:.{prec}f}" if isinstance(v, (float, np.floating)) else str(v)

    lines = [f"===== core performance metrics, step {step} =====",
             f"  step time (s)              : {g('perf/time_per_step')}",
             f"  throughput (tokens/s/GPU)  : {g('perf/throughput', 2)}",
             f"  tokens in step             : {g('perf/total_num_tokens', 0)}",
             f"  actor entropy              : {g('actor/entropy', 4)}",
             f"  rewards mean / min / max   : {g('critic/rewards/mean')} / {g('critic/rewards/min')} / "
             f"{g('critic/rewards/max')}",
             f"  scores mean / min / max    : {g('critic/score/mean')} / {g('critic/score/min')} / "
             f"{g('critic/score/max')}"]
    if enable_perf:
        lines.append("  node timings (s):")
        for k in sorted(k for k in metrics if k.startswith("timing_s/") and k != "timing_s/step"):
            lines.append(f"    {k[len('timing_s/'):]:<26}: {g(k)}")
    lines += [f"  MFU actor                  : {g('perf/mfu/actor')}",
              f"  max memory allocated (GB)  : {g('perf/max_memory_allocated_gb', 2)}",
              f"  max memory reserved (GB)   : {g('perf/max_memory_reserved_gb', 2)}",
              f"  prompt length mean / max   : {g('prompt_length/mean', 1)} / {g('prompt_length/max', 0)}",
              f"  response length mean / max : {g('response_length/mean', 1)} / {g('response_length/max', 0)}",
              f"  response clip ratio        : {g('response_length/clip_ratio', 4)}"]
    return "\n".join(lines)
