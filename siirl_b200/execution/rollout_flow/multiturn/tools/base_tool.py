"""Tool interface for multi-turn rollouts: async ``create / execute / calc_reward / release`` per trajectory
instance (reference: siirl/execution/rollout_flow/multiturn/tools/base_tool.py)."""
from __future__ import annotations

import uuid
from typing import Any, Dict, Optional, Tuple

from .schemas import OpenAIFunctionToolSchema


class BaseTool:
    def __init__(self, config: Dict[str, Any], tool_schema: OpenAIFunctionToolSchema):
        self.config = config or {}
        self.tool_schema = tool_schema
        self.name = tool_schema.function.name

    def get_openai_tool_schema(self) -> OpenAIFunctionToolSchema:
        return self.tool_schema

    async def create(self, instance_id: Optional[str] = None, **kwargs) -> str:
        return instance_id or uuid.uuid4().hex

    async def execute(self, instance_id: str, parameters: Dict[str, Any], **kwargs) -> Tuple[str, float, Dict[str, Any]]:
        """Returns ``(tool response text, step reward, metrics)``."""
        return "", 0.0, {}

    async def calc_reward(self, instance_id: str, **kwargs) -> float:
        return 0.0

    async def release(self, instance_id: str, **kwargs) -> None:
        return None
