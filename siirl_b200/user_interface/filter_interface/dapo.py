"""DAPO dynamic sampling filter (reference: siirl/user_interface/filter_interface/dapo.py:24-107).

Groups trajectories by ``uid`` and keeps only the groups whose chosen metric (``acc | score | seq_reward |
seq_final_reward``) varies inside the group (std > 0) — or singleton groups; uniform groups give zero advantage and
only dilute the batch.  Emits ``dapo_sampling/{kept_trajectories_ratio, initial_trajectories,
final_trajectories}``.  Signature of every filter node: ``fn(config, batch, **kwargs) -> NodeOutput``."""
from __future__ import annotations

import torch

from ...dag_worker.data_structures import NodeOutput
from ...data_coordinator.sample import filter_batch


def dynamic_sampling(config=None, batch=None, **kwargs) -> NodeOutput:
    fg = config.algorithm.filter_groups
    n0 = batch.batch_size
    if not fg.enable:
        return NodeOutput(batch, {"dapo_sampling/kept_trajectories_ratio": 1.0,
                                  "dapo_sampling/initial_trajectories": float(n0),
                                  "dapo_sampling/final_trajectories": float(n0)})
    metric = fg.metric
    if metric == "score":
        vals = batch["token_level_scores"].sum(-1)
    elif metric in batch:
        vals = batch[metric]
        if not isinstance(vals, torch.Tensor):
            vals = torch.tensor([float(v) for v in vals])
    else:
        raise KeyError(f"filter metric '{metric}' not found in the batch")
    vals = vals.float().cpu()
    uid = batch["uid"].cpu() if isinstance(batch["uid"], torch.Tensor) else torch.tensor(list(batch["uid"]))
    _, inv = torch.unique(uid, return_inverse=True)
    G = int(inv.max()) + 1
    cnt = torch.zeros(G).index_add_(0, inv, torch.ones_like(vals))
    mean = torch.zeros(G).index_add_(0, inv, vals) / cnt
    var = torch.zeros(G).index_add_(0, inv, (vals - mean[inv]) ** 2)
    keep_group = (var > 0) | (cnt == 1)
    keep = keep_group[inv]
    kept = filter_batch(batch, keep)
    kept.meta["kept_indices"] = keep.nonzero(as_tuple=True)[0].tolist()
    n1 = kept.batch_size
    return NodeOutput(kept, {"dapo_sampling/kept_trajectories_ratio": n1 / max(n0, 1),
                             "dapo_sampling/initial_trajectories": float(n0),
                             "dapo_sampling/final_trajectories": float(n1)})
