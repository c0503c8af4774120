"""Request / response schema of the asynchronous rollout path.

``AsyncRolloutRequest`` tracks one multi-turn conversation from its first prompt to the padded training row
(reference: siirl/engine/rollout/schemas.py:61-674).  It is a message-level state machine over token lists:

* the conversation is kept twice, as chat ``messages`` and as ``input_ids`` with a parallel ``loss_mask``
  (1 = token the policy generated, 0 = prompt / user / tool token) and ``position_ids``;
* every message that joins the conversation is tokenised *incrementally*: the chat template is applied to a fixed
  two-message base conversation plus the new message, and the tokens after the base conversation's end are the delta.
  Re-templating the whole history each turn would re-tokenise earlier turns (and could change their ids); the delta
  keeps the ids the engine actually saw;
* ``get_generation_prompt_ids`` returns what the engine is asked to continue (the incremental ids, or a fresh
  rendering of all messages when ``use_inference_chat_template``), appending the assistant header once;
* ``finalize`` strips a dangling assistant header, compares the incremental ids with one full rendering
  (``tokenization_sanity_check_mode``: strict / ignore_strippable / disable), truncates to the model and response
  limits and splits prompt / response parts.

The tokenizer ("processing class") only needs ``apply_chat_template(messages, tools=, add_generation_prompt=,
tokenize=)`` and ``decode`` -- HF tokenizers and the synthetic tokenizer both qualify.
"""
from __future__ import annotations

import difflib
import logging
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Dict, List, Optional, Sequence

logger = logging.getLogger(__name__)

# the fixed conversation in front of which single messages are rendered to get their token delta
BASE_CHAT_HISTORY = [{"role": "system", "content": "You are a helpful assistant."},
                     {"role": "user", "content": "I am a user."}]


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
        try:
            return {"length": cls.LENGTH, "stop": cls.STOP, "tool_calls": cls.TOOL_CALL, "tool_call": cls.TOOL_CALL}[v]
        except KeyError:
            raise ValueError(f"unsupported finish reason '{v}'") from None


class TokenizationSanityCheckModeEnum(str, Enum):
    DISABLE = "disable"
    STRICT = "strict"
    IGNORE_STRIPPABLE = "ignore_strippable"


@dataclass
class Message:
    role: str
    content: Any
    tool_calls: Optional[List[Dict[str, Any]]] = None

    def to_dict(self) -> Dict[str, Any]:
        d = {"role": self.role, "content": self.content}
        if self.tool_calls:
            d["tool_calls"] = self.tool_calls
        return d


def _as_id_list(x) -> List[int]:
    if isinstance(x, dict):
        x = x["input_ids"]
    if hasattr(x, "tolist"):
        x = x.tolist()
    if x and isinstance(x[0], (list, tuple)):
        x = x[0]
    return [int(t) for t in x]


def _template_ids(tok, messages: Sequence[Dict[str, Any]], tools, add_generation_prompt: bool) -> List[int]:
    kw = {"tools": tools} if tools else {}
    return _as_id_list(tok.apply_chat_template(list(messages), add_generation_prompt=add_generation_prompt,
                                               tokenize=True, **kw))


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
    multi_modal_data: Optional[Dict[str, Any]] = None
    # token-level state (filled by ``create`` or by the low-level ``add_*_tokens`` calls)
    input_ids: List[int] = field(default_factory=list)
    loss_mask: List[int] = field(default_factory=list)
    position_ids: List[int] = field(default_factory=list)
    prompt_ids: List[int] = field(default_factory=list)
    response_ids: List[int] = field(default_factory=list)
    response_loss_mask: List[int] = field(default_factory=list)
    response_logprobs: List[float] = field(default_factory=list)
    response_position_ids: List[int] = field(default_factory=list)
    reward_scores: Dict[str, Any] = field(default_factory=dict)
    max_prompt_len: int = 8192
    max_response_len: int = 8192
    max_model_len: int = 32768
    metrics: Dict[str, Any] = field(default_factory=dict)
    use_inference_chat_template: bool = False
    tokenization_sanity_check_mode: TokenizationSanityCheckModeEnum = TokenizationSanityCheckModeEnum.STRICT
    generation_prompt_ids: List[int] = field(default_factory=list)
    base_conv_wo_gen_prompt_end_pos: int = 0
    base_conv_with_gen_prompt_end_pos: int = 0

    # ---- construction ------------------------------------------------------------------------------------------------
    @classmethod
    def create(cls, request_id: str, messages: Sequence[Any], processing_class, *, tool_schemas=None,
               max_prompt_len: int = 8192, max_response_len: int = 8192, max_model_len: int = 32768,
               use_inference_chat_template: bool = False, tokenization_sanity_check_mode="strict", **kw
               ) -> "AsyncRolloutRequest":
        """Tokenise the opening messages (without the assistant header) and measure the base conversation, so that
        later messages can be added as token deltas."""
        if not messages:
            raise ValueError("messages is required to create a rollout request")
        msgs = [m if isinstance(m, Message) else Message(m["role"], m.get("content", ""), m.get("tool_calls"))
                for m in messages]
        tools = list(tool_schemas) if tool_schemas else None
        dicts = [m.to_dict() for m in msgs]
        ids = _template_ids(processing_class, dicts, tools, add_generation_prompt=False)
        with_gen = _template_ids(processing_class, dicts, tools, add_generation_prompt=True)
        gen_prompt = with_gen[len(ids):] if with_gen[:len(ids)] == ids else []
        base_wo = _template_ids(processing_class, BASE_CHAT_HISTORY, tools, add_generation_prompt=False)
        base_with = _template_ids(processing_class, BASE_CHAT_HISTORY, tools, add_generation_prompt=True)
        if len(ids) > max_prompt_len:
            logger.warning("request %s: prompt of %d tokens exceeds max_prompt_len %d", request_id, len(ids),
                           max_prompt_len)
        mode = tokenization_sanity_check_mode
        if not isinstance(mode, TokenizationSanityCheckModeEnum):
            mode = TokenizationSanityCheckModeEnum(str(mode))
        return cls(request_id=request_id, messages=msgs, tool_schemas=tools, input_ids=list(ids),
                   loss_mask=[0] * len(ids), position_ids=list(range(len(ids))), prompt_ids=list(ids),
                   max_prompt_len=max_prompt_len, max_response_len=max_response_len, max_model_len=max_model_len,
                   use_inference_chat_template=use_inference_chat_template, tokenization_sanity_check_mode=mode,
                   generation_prompt_ids=gen_prompt, base_conv_wo_gen_prompt_end_pos=len(base_wo),
                   base_conv_with_gen_prompt_end_pos=len(base_with), **kw)

    # ---- token bookkeeping ----------------------------------------------------------------------------------------------
    def _extend(self, ids: Sequence[int], in_loss: bool, logprobs: Optional[Sequence[float]] = None) -> None:
        ids = [int(t) for t in ids]
        start = (self.position_ids[-1] + 1) if self.position_ids else 0
        if not self.input_ids and self.prompt_ids:
            # requests built without ``create`` (prompt ids given directly): the conversation starts as the prompt
            self.input_ids = list(self.prompt_ids)
            self.loss_mask = [0] * len(self.prompt_ids)
            self.position_ids = list(range(len(self.prompt_ids)))
            start = len(self.prompt_ids)
        self.input_ids += ids
        self.loss_mask += [1 if in_loss else 0] * len(ids)
        self.position_ids += list(range(start, start + len(ids)))
        self.response_ids += ids
        self.response_loss_mask += [1 if in_loss else 0] * len(ids)
        self.response_logprobs += list(logprobs) if logprobs is not None else [0.0] * len(ids)
        assert len(self.input_ids) == len(self.loss_mask) == len(self.position_ids), self.request_id

    def add_assistant_tokens(self, ids: Sequence[int], logprobs: Sequence[float]) -> None:
        """Tokens the engine generated (in the loss), with their sampling log-probs."""
        self._extend(ids, True, logprobs)

    def add_observation_tokens(self, ids: Sequence[int]) -> None:
        """Tool results / user turns: part of the context, excluded from the loss."""
        self._extend(ids, False)

    @property
    def attention_mask(self) -> List[int]:
        return [1] * len(self.input_ids)

    @property
    def remaining(self) -> int:
        used = len(self.response_ids)
        return max(0, min(self.max_response_len - used, self.max_model_len - len(self.prompt_ids) - used))

    # ---- message-level transitions -------------------------------------------------------------------------------------
    def _ends_with_generation_prompt(self) -> bool:
        g = self.generation_prompt_ids
        return bool(g) and self.input_ids[-len(g):] == g

    def get_generation_prompt_ids(self, processing_class) -> List[int]:
        """Ids the engine continues from.  Appends the assistant header to the conversation once per turn."""
        if self.generation_prompt_ids and not self._ends_with_generation_prompt():
            self._extend(self.generation_prompt_ids, False)
        self.state = AsyncRolloutRequestStateEnum.RUNNING
        if self.use_inference_chat_template:
            return _template_ids(processing_class, [m.to_dict() for m in self.messages], self.tool_schemas,
                                 add_generation_prompt=True)
        return list(self.input_ids)

    def _delta(self, processing_class, message: Message, after_generation_prompt: bool) -> List[int]:
        ids = _template_ids(processing_class, [*BASE_CHAT_HISTORY, message.to_dict()], self.tool_schemas,
                            add_generation_prompt=False)
        cut = self.base_conv_with_gen_prompt_end_pos if after_generation_prompt else \
            self.base_conv_wo_gen_prompt_end_pos
        return ids[cut:]

    def add_user_message(self, processing_class, content: str) -> None:
        msg = Message("user", content)
        self.messages.append(msg)
        self._extend(self._delta(processing_class, msg, False), False)
        self.state = AsyncRolloutRequestStateEnum.INTERACTING

    def add_assistant_message(self, processing_class, content: str, tool_calls: Optional[List[Dict[str, Any]]] = None,
                              token_ids: Optional[Sequence[int]] = None,
                              logprobs: Optional[Sequence[float]] = None) -> None:
        """Append the assistant turn.  With ``token_ids`` (what the engine sampled, plus log-probs) those exact ids
        enter the conversation; otherwise the turn is re-tokenised from ``content`` after the assistant header."""
        msg = Message("assistant", content, tool_calls)
        self.messages.append(msg)
        if self.generation_prompt_ids and not self._ends_with_generation_prompt():
            self._extend(self.generation_prompt_ids, False)
        if token_ids is not None:
            self._extend(token_ids, True, logprobs)
        else:
            self._extend(self._delta(processing_class, msg, True), True)
        self.state = AsyncRolloutRequestStateEnum.TOOL_CALLING if tool_calls else AsyncRolloutRequestStateEnum.RUNNING

    def add_tool_response_messages(self, processing_class, contents: Sequence[Any]) -> None:
        """One ``tool`` message per result; dict contents (multi-modal parts) are kept as they are."""
        if not contents:
            return
        ids: List[int] = []
        for c in contents:
            msg = Message("tool", c)
            self.messages.append(msg)
            ids += self._delta(processing_class, msg, False)
        self._extend(ids, False)
        self.state = AsyncRolloutRequestStateEnum.RUNNING

    def update_metrics(self, metrics: Any, tool_id: str) -> None:
        self.metrics.setdefault(tool_id, []).append(metrics)

    # ---- end of the conversation ------------------------------------------------------------------------------------------
    def prompt_diffs(self, processing_class, full_ids: Sequence[int], context_chars: int = 10) -> List[Dict[str, Any]]:
        """Differences between one full rendering of the conversation and the incrementally built ids, as decoded
        text chunks (with a little context) and index ranges."""
        a, b = list(full_ids), list(self.input_ids)
        out = []
        for tag, i1, i2, j1, j2 in difflib.SequenceMatcher(None, a, b, autojunk=False).get_opcodes():
            if tag == "equal":
                continue
            out.append({"full_prompt_chunk": processing_class.decode(a[i1:i2]),
                        "current_prompt_chunk": processing_class.decode(b[j1:j2]), "indices": (i1, i2, j1, j2),
                        "context": processing_class.decode(a[max(0, i1 - context_chars):i2 + context_chars])})
        return out

    def finalize(self, processing_class=None, reward_scores: Optional[Dict[str, Any]] = None,
                 finish: Any = "stop") -> None:
        finish = finish if isinstance(finish, FinishReasonTypeEnum) else FinishReasonTypeEnum.from_str(str(finish))
        if finish == FinishReasonTypeEnum.TOOL_CALL:
            raise ValueError("a conversation cannot end in a tool call")
        self.state = AsyncRolloutRequestStateEnum.COMPLETED
        self.reward_scores.update(reward_scores or {})
        self.metrics["finish_reason"] = finish.value
        if self._ends_with_generation_prompt() and self.loss_mask[-1] == 0 and self.response_ids:
            # the assistant header was appended but no assistant tokens followed: take it back
            g = len(self.generation_prompt_ids)
            if len(self.response_ids) >= g:
                for name in ("input_ids", "loss_mask", "position_ids", "response_ids", "response_loss_mask",
                             "response_logprobs"):
                    setattr(self, name, getattr(self, name)[:-g])
        mode = self.tokenization_sanity_check_mode
        if processing_class is not None and mode != TokenizationSanityCheckModeEnum.DISABLE and self.messages \
                and self.input_ids:
            full = _template_ids(processing_class, [m.to_dict() for m in self.messages], self.tool_schemas, False)
            diffs = self.prompt_diffs(processing_class, full)
            if mode == TokenizationSanityCheckModeEnum.IGNORE_STRIPPABLE:
                diffs = [d for d in diffs if d["full_prompt_chunk"].strip() or d["current_prompt_chunk"].strip()]
            if diffs:
                self.metrics["tokenization_diffs"] = len(diffs)
                logger.warning("request %s: training and inference tokenisation differ (%s): %s", self.request_id,
                               mode.value, "; ".join(f"{d['indices']}: {d['full_prompt_chunk']!r} vs "
                                                     f"{d['current_prompt_chunk']!r}" for d in diffs[:4]))
        self.truncate_output_ids()

    def truncate_output_ids(self) -> None:
        m = self.max_model_len
        self.input_ids, self.loss_mask, self.position_ids = self.input_ids[:m], self.loss_mask[:m], \
            self.position_ids[:m]
        n = min(self.max_response_len, max(0, m - len(self.prompt_ids)))
        self.response_ids, self.response_loss_mask = self.response_ids[:n], self.response_loss_mask[:n]
        self.response_logprobs = self.response_logprobs[:n]
        p = len(self.prompt_ids)
        self.response_position_ids = self.position_ids[p:p + n] if self.position_ids else \
            list(range(p, p + len(self.response_ids)))
