"""Request / response schema of the asynchronous rollout path (reference: siirl/engine/rollout/schemas.py).  A
request tracks one multi-turn conversation: messages, tool schemas, token ids with their loss mask (model tokens 1,
tool / user tokens 0), log-probs and the finish state."""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional


class AsyncRolloutRequestStateEnum(str, Enum):
    PENDING = "pending"
    RUNNING = "running"
    TOOL_CALLING = "tool_calling"
    INTERACTING = "interacting"
    COMPLETED = "completed"
    FAILED = "failed"


class FinishReasonTypeEnum(str, Enum):
    LENGTH = "length"
    STOP = "stop"
    TOOL_CALL = "tool_calls"

    @classmethod
    def from_str(cls, v: str) -> "FinishReasonTypeEnum":
        return {"length": cls.LENGTH, "stop": cls.STOP, "tool_calls": cls.TOOL_CALL, "tool_call": cls.TOOL_CALL}[v]


@dataclass
class Message:
    role: str
    content: str
    tool_calls: Optional[List[Dict[str, Any]]] = None


@dataclass
class AsyncRolloutRequest:
    request_id: str
    batch_data_id: int = 0
    rollout_offset: int = 0
    state: AsyncRolloutRequestStateEnum = AsyncRolloutRequestStateEnum.PENDING
    messages: List[Message] = field(default_factory=list)
    tool_schemas: Optional[List[Dict[str, Any]]] = None
    tools_kwargs: Dict[str, Any] = field(default_factory=dict)
    interaction_kwargs: Dict[str, Any] = field(default_factory=dict)
    prompt_ids: List[int] = field(default_factory=list)
    response_ids: List[int] = field(default_factory=list)
    response_loss_mask: List[int] = field(default_factory=list)
    response_logprobs: List[float] = field(default_factory=list)
    reward_scores: Dict[str, Any] = field(default_factory=dict)
    max_response_len: int = 8192
    max_model_len: int = 32768
    metrics: Dict[str, Any] = field(default_factory=dict)

    def add_assistant_tokens(self, ids: List[int], logprobs: List[float]) -> None:
        self.response_ids += list(ids)
        self.response_loss_mask += [1] * len(ids)
        self.response_logprobs += list(logprobs)

    def add_observation_tokens(self, ids: List[int]) -> None:
        """Tool results / user turns: part of the context, excluded from the loss."""
        self.response_ids += list(ids)
        self.response_loss_mask += [0] * len(ids)
        self.response_logprobs += [0.0] * len(ids)

    @property
    def remaining(self) -> int:
        return max(0, min(self.max_response_len - len(self.response_ids),
                          self.max_model_len - len(self.prompt_ids) - len(self.response_ids)))

    def finalize(self, reward_scores: Optional[Dict[str, Any]] = None, finish: str = "stop") -> None:
        self.state = AsyncRolloutRequestStateEnum.COMPLETED
        self.reward_scores.update(reward_scores or {})
        self.metrics["finish_reason"] = FinishReasonTypeEnum.from_str(finish).value
        n = self.max_response_len
        self.response_ids, self.response_loss_mask = self.response_ids[:n], self.response_loss_mask[:n]
        self.response_logprobs = self.response_logprobs[:n]
