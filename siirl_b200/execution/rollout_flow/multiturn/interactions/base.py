"""Interaction interface: a simulated user/environment that answers the assistant between turns
(reference: siirl/execution/rollout_flow/multiturn/interactions/base.py)."""
from __future__ import annotations

import importlib
import uuid
from typing import Any, Dict, List, Optional, Tuple

import yaml

from .....utils.reward_score import gsm8k as gsm8k_score


class BaseInteraction:
    def __init__(self, config: Dict[str, Any]):
        self.config = config or {}
        self.name = self.config.get("name", "interaction")

    async def start_interaction(self, instance_id: Optional[str] = None, **kwargs) -> str:
        return instance_id or uuid.uuid4().hex

    async def generate_response(self, instance_id: str, messages: List[Dict[str, Any]], **kwargs
                                ) -> Tuple[bool, str, float, Dict[str, Any]]:
        """Returns ``(should_terminate, response text, turn score, extra)``."""
        return True, "", 0.0, {}

    async def calculate_score(self, instance_id: str, **kwargs) -> float:
        return 0.0

    async def finalize_interaction(self, instance_id: str, **kwargs) -> None:
        return None


class Gsm8kInteraction(BaseInteraction):
    """Checks the assistant's last message against the ground truth; asks to try again when it is wrong."""

    def __init__(self, config):
        super().__init__(config)
        self._state: Dict[str, Dict[str, Any]] = {}

    async def start_interaction(self, instance_id=None, ground_truth=None, **kw) -> str:
        iid = await super().start_interaction(instance_id)
        self._state[iid] = {"ground_truth": ground_truth, "response": "", "reward": 0.0}
        return iid

    async def generate_response(self, instance_id, messages, **kw):
        content = next((m["content"] for m in reversed(messages) if m.get("role") == "assistant"), "")
        self._state[instance_id]["response"] = content
        r = await self.calculate_score(instance_id)
        if r >= 1.0:
            return True, "Your response is correct!", 1.0, {}
        return False, "Your response is incorrect! You need to reflect on your answer and try again.", 0.0, {}

    async def calculate_score(self, instance_id, **kw) -> float:
        st = self._state[instance_id]
        return gsm8k_score.compute_score(st["response"], st["ground_truth"], method="flexible")

    async def finalize_interaction(self, instance_id, **kw) -> None:
        self._state.pop(instance_id, None)


def initialize_interactions_from_config(path_or_dict) -> Dict[str, BaseInteraction]:
    if isinstance(path_or_dict, str):
        with open(path_or_dict) as f:
            cfg = yaml.safe_load(f)
    else:
        cfg = path_or_dict
    out: Dict[str, BaseInteraction] = {}
    for it in (cfg or {}).get("interaction", []):
        mod, _, cls = it["class_name"].rpartition(".")
        klass = getattr(importlib.import_module(mod or __name__), cls)
        c = dict(it.get("config", {}))
        name = it.get("name") or c.get("name") or cls.lower().replace("interaction", "")
        c["name"] = name
        if name in out:
            raise ValueError(f"duplicate interaction name '{name}'")
        out[name] = klass(c)
    return out
