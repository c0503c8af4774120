"""Embodied dynamic sampling (reference: siirl/user_interface/filter_interface/embodied.py:27-270): per prompt
group keep the group only if its success rate lies inside ``[accuracy_lower_bound, accuracy_upper_bound]`` and,
optionally, drop trajectories that hit the step limit without finishing."""
from __future__ import annotations

import torch

from ...dag_worker.data_structures import NodeOutput
from ...data_coordinator.sample import filter_batch


def embodied_local_rank_sampling(config=None, batch=None, **kwargs) -> NodeOutput:
    es = config.algorithm.embodied_sampling
    n0 = batch.batch_size
    keep = torch.ones(n0, dtype=torch.bool)
    if es.filter_accuracy and "complete" in batch and "uid" in batch:
        acc = batch["complete"].float().reshape(n0).cpu()
        uid = batch["uid"].cpu()
        _, inv = torch.unique(uid, return_inverse=True)
        G = int(inv.max()) + 1
        cnt = torch.zeros(G).index_add_(0, inv, torch.ones(n0))
        rate = torch.zeros(G).index_add_(0, inv, acc) / cnt
        ok = (rate >= es.accuracy_lower_bound) & (rate <= es.accuracy_upper_bound)
        keep &= ok[inv]
    if es.filter_truncated and "finish_step" in batch:
        max_steps = config.actor_rollout_ref.embodied.env.max_steps
        fs = batch["finish_step"].reshape(n0).cpu()
        done = batch["complete"].reshape(n0).cpu().bool() if "complete" in batch else torch.zeros(n0, dtype=torch.bool)
        keep &= ~((fs >= max_steps) & ~done)
    kept = filter_batch(batch, keep) if not bool(keep.all()) else batch
    return NodeOutput(kept, {"embodied_sampling/kept_ratio": kept.batch_size / max(n0, 1),
                             "embodied_sampling/initial_trajectories": float(n0),
                             "embodied_sampling/final_trajectories": float(kept.batch_size)})
