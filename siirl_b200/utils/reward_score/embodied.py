"""Embodied trajectory reward (reference: siirl/utils/reward_score/embodied.py:41-200).

Successful episodes score 1.  A failed episode is scored by how close its video embedding lies to the successful
episodes of the same task: success embeddings are clustered with DBSCAN, the distance ``d`` to the nearest cluster
centre is min-max normalised over the failed episodes of the batch to ``d_hat`` in [0, 1], and the score is
``0.6 * sigmoid(10 * (0.5 - d_hat))``.  Without any success in the task the failed episodes score 0."""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch


def dbscan(x: np.ndarray, eps: float, min_samples: int) -> np.ndarray:
    """Plain DBSCAN labels (-1 = noise); O(n^2) distances, n is a batch of episodes."""
    n = len(x)
    d = np.linalg.norm(x[:, None, :] - x[None, :, :], axis=-1)
    neigh = [np.flatnonzero(d[i] <= eps) for i in range(n)]
    core = np.array([len(nb) >= min_samples for nb in neigh])
    labels = np.full(n, -1, dtype=np.int64)
    c = 0
    for i in range(n):
        if labels[i] != -1 or not core[i]:
            continue
        labels[i] = c
        stack = list(neigh[i])
        while stack:
            j = stack.pop()
            if labels[j] == -1:
                labels[j] = c
                if core[j]:
                    stack.extend(k for k in neigh[j] if labels[k] == -1)
        c += 1
    return labels


def cluster_centers(success_emb: np.ndarray, eps: float = 0.5, min_samples: int = 2) -> np.ndarray:
    if len(success_emb) == 0:
        return success_emb
    labels = dbscan(success_emb, eps, min_samples)
    centers = [success_emb[labels == c].mean(0) for c in range(labels.max() + 1)]
    if not centers:                       # everything is noise: fall back to the mean of all successes
        centers = [success_emb.mean(0)]
    return np.stack(centers)


def compute_embodied_reward(batch_embeddings, complete, task_file_name: Optional[Sequence[str]] = None,
                            eps: float = 0.5, min_samples: int = 2, max_shaped: float = 0.6,
                            sharpness: float = 10.0, **_) -> List[float]:
    emb = torch.as_tensor(batch_embeddings).float().cpu().numpy()
    ok = torch.as_tensor(complete).float().cpu().numpy() > 0.5
    B = len(ok)
    tasks = list(task_file_name) if task_file_name is not None else ["_"] * B
    scores = np.where(ok, 1.0, 0.0).astype(np.float64)
    for t in set(tasks):
        idx = np.array([i for i in range(B) if tasks[i] == t])
        succ, fail = idx[ok[idx]], idx[~ok[idx]]
        if len(succ) == 0 or len(fail) == 0:
            continue
        centers = cluster_centers(emb[succ], eps, min_samples)
        d = np.linalg.norm(emb[fail][:, None, :] - centers[None, :, :], axis=-1).min(1)
        span = d.max() - d.min()
        d_hat = (d - d.min()) / span if span > 1e-8 else np.full_like(d, 0.5)
        scores[fail] = max_shaped / (1.0 + np.exp(-sharpness * (0.5 - d_hat)))
    return scores.tolist()
