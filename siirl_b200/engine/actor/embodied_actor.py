"""Trajectory <-> model-row views for embodied (VLA) policies.

An embodied batch holds whole trajectories: ``responses [B, L, A]`` (L model calls of A = chunk * action_token_len
action tokens), per-call prompts ``step_input_ids / step_attention_mask [B, L, P]``, per-call policy images
``images [B, L, S, S, 3]`` and ``finish_step [B]`` in environment steps.  Advantages, masks and log-probs live on
the flattened ``[B, L*A]`` token axis (reference: siirl/engine/actor/embodied_actor.py:40-573, which walks
``traj_mini_batch_size`` trajectories at a time and masks calls beyond ``finish_step``).  Here only the EXECUTED
calls become model rows — ``[N, P+A]`` rows of the ordinary packed log-prob path with their image attached — so
compute is proportional to the steps that happened, and results are scattered back to ``[B, L*A]``."""
from __future__ import annotations

from typing import Tuple

import torch

from ...data_coordinator.protocol import Batch

_TOKEN_KEYS = ("advantages", "returns", "old_log_probs", "ref_log_prob", "response_mask", "rollout_log_probs",
               "token_level_rewards", "token_level_scores")


def executed_calls(finish_step: torch.Tensor, L: int, actions_per_call: int) -> torch.Tensor:
    """``[B, L]`` bool: call l of trajectory b ran (its first action index is below ``finish_step``)."""
    first = torch.arange(L, device=finish_step.device)[None, :] * actions_per_call
    return first < finish_step.reshape(-1, 1)


def trajectory_response_mask(finish_step: torch.Tensor, L: int, actions_per_call: int,
                             action_token_len: int) -> torch.Tensor:
    """``[B, L*A]`` mask = token index < finish_step * action_token_len (tokens of executed actions)."""
    T = L * actions_per_call * action_token_len
    t = torch.arange(T, device=finish_step.device)[None, :]
    return (t < finish_step.reshape(-1, 1) * action_token_len).long()


def flatten_trajectories(data: Batch, actions_per_call: int) -> Tuple[Batch, torch.Tensor, torch.Tensor]:
    """Returns (rows batch, b index ``[N]``, l index ``[N]``)."""
    resp = data["responses"]
    B, L, A = resp.shape
    run = executed_calls(data["finish_step"].to(resp.device), L, actions_per_call)
    bi, li = run.nonzero(as_tuple=True)
    rows = Batch({}, {}, dict(data.meta))
    r = resp[bi, li]
    p_ids = data["step_input_ids"][bi, li]
    p_am = data["step_attention_mask"][bi, li]
    rows["responses"] = r
    rows["input_ids"] = torch.cat([p_ids, r], -1)
    tok_mask = torch.ones_like(r)
    if "response_mask" in data:
        tok_mask = data["response_mask"].reshape(B, L, A)[bi, li]
    # every token of an executed call is fed to the model; the loss mask may end inside the last call
    rows["attention_mask"] = torch.cat([p_am, torch.ones_like(r)], -1)
    rows["response_mask"] = tok_mask
    rows["images"] = data["images"][bi, li]
    for k in _TOKEN_KEYS:
        if k in data and k != "response_mask":
            rows[k] = data[k].reshape(B, L, A)[bi, li]
    return rows, bi, li


def scatter_steps(values: torch.Tensor, bi: torch.Tensor, li: torch.Tensor, B: int, L: int) -> torch.Tensor:
    """Per-row ``[N, A]`` values -> ``[B, L*A]`` (zeros where a call did not run)."""
    A = values.shape[1]
    out = torch.zeros(B, L, A, dtype=values.dtype, device=values.device)
    out[bi.to(values.device), li.to(values.device)] = values
    return out.reshape(B, L * A)
