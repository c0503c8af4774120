"""Multi-turn agent loops on top of the in-process async rollout server.

Protocol of the reference (siirl/execution/rollout_flow/multiturn/agent_loop/agent_loop.py:46-388,
tool_agent_loop.py): tokenise the chat with the tool schemas -> loop { generate (sticky session to one server so the
prefix stays cached) -> append response ids with ``response_mask = 1`` -> stop on response budget /
``max_assistant_turns`` / ``max_user_turns`` -> parse ``<tool_call>{json}</tool_call>`` blocks (Hermes format) ->
run up to ``max_parallel_calls`` tools concurrently (create -> execute -> release), truncating tool output to
``max_tool_response_length`` on the left / right / middle -> tokenise the tool messages and append them with
``response_mask = 0`` }.  The loss mask therefore excludes tool and user tokens.  ``AgentLoopManager`` spreads a
batch over the loops and collates the outputs into the padded batch layout of the rollout node.
"""
from __future__ import annotations

import asyncio
import json
import re
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch

from .....data_coordinator import Batch
from .....engine.packing import position_ids_from_mask
from ..tools.base_tool import BaseTool
from ..tools.schemas import OpenAIFunctionCallSchema


@dataclass
class AgentLoopOutput:
    prompt_ids: List[int]
    response_ids: List[int]
    response_mask: List[int]
    response_logprobs: List[float] = field(default_factory=list)
    num_turns: int = 0
    metrics: Dict[str, Any] = field(default_factory=dict)
    reward_score: Optional[float] = None


class AsyncLLMServerManager:
    """Least-loaded server choice with sticky sessions: turns of one request go to the same server."""

    def __init__(self, servers: List[Any], max_cache_size: int = 10000):
        self.servers = list(servers)
        self.load = [0] * len(servers)
        self.sticky: Dict[str, int] = {}
        self.max_cache_size = max_cache_size

    def _choose(self, request_id: str) -> int:
        if request_id in self.sticky:
            return self.sticky[request_id]
        i = min(range(len(self.servers)), key=lambda k: self.load[k])
        if len(self.sticky) >= self.max_cache_size:
            self.sticky.pop(next(iter(self.sticky)))
        self.sticky[request_id] = i
        return i

    async def generate(self, request_id: str, prompt_ids: List[int], sampling_params: Dict[str, Any]) -> Dict[str, Any]:
        i = self._choose(request_id)
        self.load[i] += 1
        try:
            return await self.servers[i].generate(request_id, prompt_ids, sampling_params)
        finally:
            self.load[i] -= 1


class AgentLoopBase:
    def __init__(self, config, server_manager: AsyncLLMServerManager, tokenizer, **kwargs):
        self.config = config
        self.server_manager = server_manager
        self.tokenizer = tokenizer
        r = config.actor_rollout_ref.rollout
        self.prompt_length = r.prompt_length
        self.response_length = r.response_length

    def _encode_chat(self, messages, tools=None, add_generation_prompt=True) -> List[int]:
        text = self.tokenizer.apply_chat_template(messages, add_generation_prompt=add_generation_prompt,
                                                  tokenize=False, tools=tools) \
            if tools else self.tokenizer.apply_chat_template(messages, add_generation_prompt=add_generation_prompt,
                                                             tokenize=False)
        return self.tokenizer.encode(text, add_special_tokens=False)

    async def run(self, messages: List[Dict[str, Any]], sampling_params: Dict[str, Any], **kwargs) -> AgentLoopOutput:
        raise NotImplementedError


class SingleTurnAgentLoop(AgentLoopBase):
    async def run(self, messages, sampling_params, raw_prompt_ids: Optional[List[int]] = None, **kwargs):
        prompt_ids = list(raw_prompt_ids) if raw_prompt_ids is not None else self._encode_chat(messages)
        sp = dict(sampling_params, max_new_tokens=self.response_length)
        out = await self.server_manager.generate(uuid.uuid4().hex, prompt_ids, sp)
        ids = out["token_ids"][: self.response_length]
        return AgentLoopOutput(prompt_ids, ids, [1] * len(ids), out["logprobs"][: len(ids)], num_turns=2)


_TOOL_CALL_RE = re.compile(r"<tool_call>(.*?)</tool_call>", re.DOTALL)


def parse_hermes_tool_calls(text: str) -> List[OpenAIFunctionCallSchema]:
    calls = []
    for m in _TOOL_CALL_RE.findall(text):
        try:
            d = json.loads(m)
            call, err = OpenAIFunctionCallSchema.from_raw(d["name"], d.get("arguments", {}))
            if not err:
                calls.append(call)
        except (json.JSONDecodeError, KeyError, TypeError):
            continue
    return calls


def truncate_text(text: str, limit: int, side: str) -> str:
    if limit is None or len(text) <= limit:
        return text
    if side == "left":
        return text[:limit] + "...(truncated)"
    if side == "right":
        return "(truncated)..." + text[-limit:]
    half = limit // 2
    return text[:half] + "...(truncated)..." + text[-half:]


class ToolAgentLoop(AgentLoopBase):
    def __init__(self, config, server_manager, tokenizer, tools: Optional[List[BaseTool]] = None,
                 interaction=None, **kwargs):
        super().__init__(config, server_manager, tokenizer)
        mt = config.actor_rollout_ref.rollout.multi_turn
        self.tools = {t.name: t for t in (tools or [])}
        self.tool_schemas = [t.get_openai_tool_schema().to_dict() for t in (tools or [])]
        self.max_assistant_turns = mt.max_assistant_turns
        self.max_user_turns = mt.max_user_turns
        self.max_parallel_calls = mt.max_parallel_calls
        self.max_tool_response_length = mt.max_tool_response_length
        self.truncate_side = mt.tool_response_truncate_side
        self.interaction = interaction

    async def _call_tool(self, call: OpenAIFunctionCallSchema, tools_kwargs: Dict[str, Any]) -> Dict[str, Any]:
        tool = self.tools.get(call.name)
        if tool is None:
            return {"role": "tool", "content": f"Error: unknown tool '{call.name}'", "reward": 0.0}
        kw = tools_kwargs.get(call.name, {})
        iid = None
        try:
            iid = await tool.create(**kw.get("create_kwargs", {}))
            text, reward, _ = await tool.execute(iid, call.arguments, **kw.get("execute_kwargs", {}))
        except Exception as e:  # noqa: BLE001  (a failing tool is reported to the model, not raised)
            text, reward = f"Error when executing tool: {e}", 0.0
        finally:
            if iid is not None:
                await tool.release(iid)
        return {"role": "tool", "content": truncate_text(str(text), self.max_tool_response_length, self.truncate_side),
                "reward": reward}

    async def run(self, messages, sampling_params, tools_kwargs: Optional[Dict[str, Any]] = None,
                  interaction_kwargs: Optional[Dict[str, Any]] = None, **kwargs) -> AgentLoopOutput:
        tools_kwargs = tools_kwargs or {}
        request_id = uuid.uuid4().hex
        prompt_ids = self._encode_chat(messages, tools=self.tool_schemas or None)
        # length of the system-prompt prefix a lone tool/user message gets from the chat template
        base = self.tokenizer.encode(self.tokenizer.apply_chat_template([{"role": "system", "content": ""}],
                                                                        add_generation_prompt=False, tokenize=False),
                                     add_special_tokens=False) if hasattr(self.tokenizer, "apply_chat_template") else []
        ids = list(prompt_ids)
        mask: List[int] = []
        logps: List[float] = []
        assistant_turns = user_turns = 0
        tool_reward = 0.0
        inter_id = None
        if self.interaction is not None:
            inter_id = await self.interaction.start_interaction(**(interaction_kwargs or {}))
        history = list(messages)
        while True:
            budget = self.response_length - len(mask)
            if budget <= 0:
                break
            out = await self.server_manager.generate(request_id, ids, dict(sampling_params, max_new_tokens=budget))
            new = out["token_ids"][:budget]
            ids += new
            mask += [1] * len(new)
            logps += out["logprobs"][: len(new)]
            assistant_turns += 1
            if len(mask) >= self.response_length:
                break
            if self.max_assistant_turns and assistant_turns >= self.max_assistant_turns:
                break
            if self.max_user_turns and user_turns >= self.max_user_turns:
                break
            text = self.tokenizer.decode(new, skip_special_tokens=True)
            history.append({"role": "assistant", "content": text})
            calls = parse_hermes_tool_calls(text)[: self.max_parallel_calls]
            if calls:
                replies = await asyncio.gather(*[self._call_tool(c, tools_kwargs) for c in calls])
                tool_reward += sum(r["reward"] for r in replies)
                extra_msgs = [{"role": "tool", "content": r["content"]} for r in replies]
            elif self.interaction is not None:
                stop, reply, score, _ = await self.interaction.generate_response(inter_id, history)
                tool_reward += score
                if stop:
                    break
                extra_msgs = [{"role": "user", "content": reply}]
            else:
                break
            history += extra_msgs
            enc = self._encode_chat(extra_msgs, add_generation_prompt=True)
            if base and enc[: len(base)] == base:
                enc = enc[len(base):]
            enc = enc[: self.response_length - len(mask)]
            ids += enc
            mask += [0] * len(enc)
            logps += [0.0] * len(enc)
            user_turns += 1
        if inter_id is not None:
            await self.interaction.finalize_interaction(inter_id)
        resp = ids[len(prompt_ids):][: self.response_length]
        return AgentLoopOutput(prompt_ids, resp, mask[: len(resp)], logps[: len(resp)],
                               num_turns=assistant_turns + user_turns + 1, metrics={"tool_reward": tool_reward})


AGENT_LOOPS = {"single_turn_agent": SingleTurnAgentLoop, "tool_agent": ToolAgentLoop}


class AgentLoopManager:
    """Runs one agent loop per sample concurrently and collates the results (reference ``AgentLoopManager`` +
    ``AgentLoopWorker`` post-processing, agent_loop.py:148-388)."""

    def __init__(self, config, servers: List[Any], tokenizer, tools=None, interactions=None):
        self.config = config
        self.tokenizer = tokenizer
        self.server_manager = AsyncLLMServerManager(servers)
        self.tools = tools or []
        self.interactions = interactions or {}

    def _loop_for(self, agent_name: str, interaction_name: Optional[str]):
        cls = AGENT_LOOPS.get(agent_name, SingleTurnAgentLoop)
        return cls(self.config, self.server_manager, self.tokenizer, tools=self.tools,
                   interaction=self.interactions.get(interaction_name) if interaction_name else None)

    async def _run_all(self, batch: Batch, sampling_params: Dict[str, Any]) -> List[AgentLoopOutput]:
        agent = self.config.actor_rollout_ref.rollout.agent.agent_name
        if self.config.actor_rollout_ref.rollout.multi_turn.enable and agent == "single_turn_agent":
            agent = "tool_agent"
        tasks = []
        for i in range(batch.batch_size):
            msgs = batch["raw_prompt"][i] if "raw_prompt" in batch else None
            raw_ids = batch["raw_prompt_ids"][i] if "raw_prompt_ids" in batch else None
            ikw = batch["interaction_kwargs"][i] if "interaction_kwargs" in batch else None
            loop = self._loop_for(agent, (ikw or {}).get("name"))
            tasks.append(loop.run(list(msgs) if msgs is not None else [], sampling_params, raw_prompt_ids=raw_ids,
                                  tools_kwargs=batch["tools_kwargs"][i] if "tools_kwargs" in batch else None,
                                  interaction_kwargs=ikw))
        return await asyncio.gather(*tasks)

    def generate_sequences(self, batch: Batch, sampling_params: Optional[Dict[str, Any]] = None) -> Batch:
        r = self.config.actor_rollout_ref.rollout
        sp = {"temperature": r.temperature, "top_k": r.top_k, "top_p": r.top_p,
              "eos_token_id": getattr(self.tokenizer, "eos_token_id", None)}
        sp.update(sampling_params or {})
        outs = asyncio.run(self._run_all(batch, sp))
        return self._postprocess(batch, outs)

    def _postprocess(self, batch: Batch, outs: List[AgentLoopOutput]) -> Batch:
        r = self.config.actor_rollout_ref.rollout
        P, R = r.prompt_length, r.response_length
        pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
        B = len(outs)
        prompts = torch.full((B, P), pad, dtype=torch.int64)
        pmask = torch.zeros(B, P, dtype=torch.int64)
        responses = torch.full((B, R), pad, dtype=torch.int64)
        rmask_attn = torch.zeros(B, R, dtype=torch.int64)
        loss_mask = torch.zeros(B, R, dtype=torch.int64)
        logps = torch.zeros(B, R)
        for i, o in enumerate(outs):
            p = o.prompt_ids[-P:]
            prompts[i, P - len(p):] = torch.tensor(p)
            pmask[i, P - len(p):] = 1
            L = min(len(o.response_ids), R)
            responses[i, :L] = torch.tensor(o.response_ids[:L])
            rmask_attn[i, :L] = 1
            loss_mask[i, :L] = torch.tensor(o.response_mask[:L])
            if o.response_logprobs:
                logps[i, :L] = torch.tensor(o.response_logprobs[:L])
        attn = torch.cat([pmask, rmask_attn], -1)
        out = Batch(dict(batch.tensors), dict(batch.non_tensors), dict(batch.meta))
        out["prompts"], out["responses"] = prompts, responses
        out["input_ids"] = torch.cat([prompts, responses], -1)
        out["attention_mask"] = attn
        out["position_ids"] = position_ids_from_mask(attn)
        out["response_mask"] = loss_mask          # the loss mask: assistant tokens only
        out["rollout_log_probs"] = logps
        out.set_non_tensor("num_turns", [o.num_turns for o in outs])
        out.set_non_tensor("tool_reward", [o.metrics.get("tool_reward", 0.0) for o in outs])
        return out
