"""Multi-turn agent loop, tools, interactions and the async rollout server (CPU)."""
import asyncio

import torch

from siirl_b200.data_coordinator import Batch
from siirl_b200.data_coordinator.dataloader import SyntheticTokenizer
from siirl_b200.engine.rollout.async_server import AsyncRolloutServer
from siirl_b200.engine.rollout.native_engine import RolloutEngine
from siirl_b200.execution.rollout_flow.multiturn.agent_loop.agent_loop import (AgentLoopManager, AsyncLLMServerManager,
                                                                              ToolAgentLoop, parse_hermes_tool_calls,
                                                                              truncate_text)
from siirl_b200.execution.rollout_flow.multiturn.interactions.base import (Gsm8kInteraction,
                                                                           initialize_interactions_from_config)
from siirl_b200.execution.rollout_flow.multiturn.tools.tool_registry import initialize_tools_from_config
from siirl_b200.models.config import get_config
from siirl_b200.models.decoder import build_model
from siirl_b200.params import parse_config

TOOLS = {"tools": [{"class_name": "CalculatorTool", "config": {},
                    "tool_schema": {"type": "function", "function": {
                        "name": "calc", "description": "evaluate", "parameters": {
                            "type": "object", "properties": {"expression": {"type": "string"}},
                            "required": ["expression"]}}}}]}


class ScriptedServer:
    """Returns scripted assistant texts turn by turn."""

    def __init__(self, tok, texts):
        self.tok, self.texts, self.calls = tok, list(texts), []

    async def generate(self, request_id, prompt_ids, sampling_params):
        self.calls.append((request_id, len(prompt_ids)))
        ids = self.tok.encode(self.texts.pop(0))[: sampling_params["max_new_tokens"]]
        return {"token_ids": ids, "logprobs": [-0.5] * len(ids), "finish_reason": "stop"}


def _cfg(**kw):
    return parse_config(["data.max_prompt_length=64", "data.max_response_length=200",
                         "actor_rollout_ref.rollout.multi_turn.enable=True"] + [f"{k}={v}" for k, v in kw.items()])


def test_parse_and_truncate():
    calls = parse_hermes_tool_calls('x <tool_call>{"name": "calc", "arguments": {"expression": "1+2"}}</tool_call> '
                                    '<tool_call>not json</tool_call>')
    assert len(calls) == 1 and calls[0].name == "calc" and calls[0].arguments == {"expression": "1+2"}
    assert truncate_text("abcdefghij", 4, "left").startswith("abcd")
    assert truncate_text("abcdefghij", 4, "right").endswith("ghij")
    assert "ab" in truncate_text("abcdefghij", 4, "middle") and "ij" in truncate_text("abcdefghij", 4, "middle")


def test_tool_agent_loop_masks_tool_tokens():
    tok = SyntheticTokenizer()
    tools = initialize_tools_from_config(TOOLS)
    server = ScriptedServer(tok, ['<tool_call>{"name": "calc", "arguments": {"expression": "6*7"}}</tool_call>',
                                  "the answer is 42"])
    loop = ToolAgentLoop(_cfg(), AsyncLLMServerManager([server]), tok, tools=tools)
    out = asyncio.run(loop.run([{"role": "user", "content": "what is 6*7?"}], {"temperature": 1.0}))
    text = tok.decode(out.response_ids)
    assert "42" in text and out.num_turns >= 3
    # tool output tokens carry mask 0, assistant tokens mask 1
    assert 0 in out.response_mask and 1 in out.response_mask and len(out.response_mask) == len(out.response_ids)
    first_zero = out.response_mask.index(0)
    assert all(m == 1 for m in out.response_mask[:first_zero])
    # both turns went to the same server with the same request id (sticky session), with a growing prompt
    assert server.calls[0][0] == server.calls[1][0] and server.calls[1][1] > server.calls[0][1]


def test_interaction_loop_and_registry():
    tok = SyntheticTokenizer()
    inter = initialize_interactions_from_config({"interaction": [
        {"name": "gsm8k", "class_name": "siirl_b200.execution.rollout_flow.multiturn.interactions.base.Gsm8kInteraction",
         "config": {}}]})
    assert isinstance(inter["gsm8k"], Gsm8kInteraction)
    server = ScriptedServer(tok, ["i think 5", "#### 7"])
    loop = ToolAgentLoop(_cfg(), AsyncLLMServerManager([server]), tok, interaction=inter["gsm8k"])
    out = asyncio.run(loop.run([{"role": "user", "content": "3+4?"}], {}, interaction_kwargs={"ground_truth": "7"}))
    assert out.metrics["tool_reward"] == 1.0 and "try again" in tok.decode(out.response_ids)


def test_async_server_batches_concurrent_requests_and_manager_collates():
    model = build_model(get_config("tiny"), dtype=torch.float32, seed=0)
    tok = SyntheticTokenizer()
    server = AsyncRolloutServer(RolloutEngine(model, max_num_seqs=8, max_model_len=128), tok)

    async def many():
        return await asyncio.gather(*[server.generate(str(i), [5, 6, 7 + i], {"max_new_tokens": 4, "temperature": 0.0})
                                      for i in range(5)])
    outs = asyncio.run(many())
    assert len(outs) == 5 and all(len(o["token_ids"]) == 4 for o in outs)
    assert server.num_batches == 1                      # all five shared one engine call
    cfg = parse_config(["data.max_prompt_length=16", "data.max_response_length=6"])
    mgr = AgentLoopManager(cfg, [server], tok)
    batch = Batch(non_tensors={"raw_prompt_ids": [[5, 6, 7], [8, 9]]})
    out = mgr.generate_sequences(batch, {"temperature": 0.0})
    assert out["responses"].shape == (2, 6) and out["input_ids"].shape == (2, 22)
    assert out["attention_mask"][0, :13].sum() == 0 and out["attention_mask"][0, 13:16].sum() == 3
    resp = asyncio.run(server.chat_completion({"messages": [{"role": "user", "content": "1+1="}], "max_tokens": 3}))
    assert resp["choices"][0]["message"]["role"] == "assistant" and resp["usage"]["completion_tokens"] == 3
