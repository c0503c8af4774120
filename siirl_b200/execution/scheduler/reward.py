"""Reward plumbing: user reward function loading, manager construction, guarded scoring.

Reference: siirl/execution/scheduler/reward.py:44-229.  Priority when choosing the scorer: a custom function
(``custom_reward_function.path/.name``) wins over the default dispatch by ``data_source``.  A scorer that raises
does not kill the step: the batch gets zero rewards and the error is reported in the metrics."""
from __future__ import annotations

import importlib.util
import os
import sys
from functools import partial
from typing import Any, Callable, Dict, Optional, Tuple

import torch

from ...engine.reward_manager import REWARD_MANAGERS
from ...utils.reward_score import default_compute_score


def load_custom_reward_function(path: Optional[str], name: str = "compute_score",
                                reward_kwargs: Optional[Dict[str, Any]] = None) -> Optional[Callable]:
    if not path:
        return None
    path = os.path.expanduser(path)
    if not os.path.exists(path):
        raise FileNotFoundError(f"Reward function file '{path}' not found.")
    spec = importlib.util.spec_from_file_location("custom_reward_module", path)
    module = importlib.util.module_from_spec(spec)
    sys.modules["custom_reward_module"] = module
    spec.loader.exec_module(module)
    if not hasattr(module, name):
        raise AttributeError(f"Reward function '{name}' not found in '{path}'.")
    fn = getattr(module, name)
    return partial(fn, **reward_kwargs) if reward_kwargs else fn


def create_reward_manager(config, tokenizer, num_examine: int = 0, max_resp_len: Optional[int] = None, **kwargs):
    name = config.reward_model.reward_manager
    if name not in REWARD_MANAGERS:
        raise NotImplementedError(f"unknown reward manager '{name}' (have {sorted(REWARD_MANAGERS)})")
    crf = config.custom_reward_function
    score_fn = load_custom_reward_function(crf.path, crf.name, dict(crf.reward_kwargs or {})) or default_compute_score
    cls = REWARD_MANAGERS[name]
    extra: Dict[str, Any] = dict(config.reward_model.reward_kwargs or {})
    extra.update(kwargs)
    if name == "dapo":
        extra.update(max_resp_len=max_resp_len or config.data.max_response_length,
                     overlong_buffer_cfg=config.reward_model.overlong_buffer)
    if name == "embodied":
        extra.setdefault("action_token_len", config.actor_rollout_ref.embodied.action_token_len)
        if "embodied_score_fn" in kwargs:
            score_fn = kwargs.pop("embodied_score_fn")
        elif score_fn is default_compute_score:
            from ...utils.reward_score.embodied import compute_embodied_reward
            score_fn = compute_embodied_reward
    return cls(tokenizer=tokenizer, num_examine=num_examine, compute_score=score_fn,
               reward_fn_key=config.data.reward_fn_key, **extra)


def compute_reward(batch, reward_fn) -> Tuple[torch.Tensor, Dict[str, Any]]:
    """Returns ``(reward_tensor, extra_info)``; scorer exceptions yield zero rewards."""
    try:
        res = reward_fn(batch, return_dict=True)
        return res["reward_tensor"], res.get("reward_extra_info", {})
    except Exception as e:  # noqa: BLE001
        zeros = torch.zeros(batch["responses"].shape[:2], dtype=torch.float32, device=batch["responses"].device)
        return zeros, {"reward_error": [f"{type(e).__name__}: {e}"]}
