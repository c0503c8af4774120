"""Environment interface of the embodied (VLA) workflow (reference: siirl/environment/embodied/base.py)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional


class BaseVLAEnvironment:
    """Batched environment: ``reset`` returns one observation dict per environment, ``step`` applies one action
    (or a chunk of actions) per environment and returns per-environment dicts with ``obs``, ``reward``, ``done``,
    ``success`` and ``step``."""

    num_envs: int = 0

    async def reset(self, task_ids: Optional[List[int]] = None, trial_ids: Optional[List[int]] = None
                    ) -> List[Dict[str, Any]]:
        raise NotImplementedError

    async def step(self, action) -> List[Dict[str, Any]]:
        raise NotImplementedError

    def close(self) -> None:
        pass
