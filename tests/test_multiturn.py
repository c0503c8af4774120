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


def test_multiturn_pipeline_end_to_end(tmp_path):
    """GRPO with the rollout node served by agent loops (tool agent + in-process request server) for two steps."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, OMP_NUM_THREADS="2", SIIRL_LOG_DIR=str(tmp_path / "log"))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    args = ["algorithm.adv_estimator=grpo", "data.synthetic=parity", "data.synthetic_size=64",
            "data.synthetic_min_prompt=16", "data.synthetic_max_prompt=32", "data.max_prompt_length=32",
            "data.max_response_length=24", "data.train_batch_size=4", "actor_rollout_ref.model.arch_preset=tiny",
            "actor_rollout_ref.rollout.n=4", "actor_rollout_ref.rollout.max_num_seqs=16",
            "actor_rollout_ref.rollout.multi_turn.enable=True", "actor_rollout_ref.rollout.multi_turn.max_assistant_turns=2",
            "actor_rollout_ref.rollout.multi_turn.tool_config_path=examples/multi_turn/gsm8k_tool_config.yaml",
            "actor_rollout_ref.rollout.prompt_length=32", "actor_rollout_ref.rollout.response_length=24",
            "actor_rollout_ref.actor.ppo_mini_batch_size=4", "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8",
            "trainer.n_gpus_per_node=1", "trainer.device=cpu", "trainer.val_before_train=False",
            "trainer.logger=['jsonl']", "trainer.total_training_steps=2", "trainer.save_freq=-1"]
    out = subprocess.run([sys.executable, "-m", "siirl_b200.main_dag", *args], env=env, cwd=root, capture_output=True,
                         text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    with open(tmp_path / "log" / "metrics.jsonl") as f:
        m = [json.loads(line) for line in f]
    assert [r["step"] for r in m] == [1, 2] and all(r["num_turns/mean"] >= 1 for r in m)
    assert all(r["response_length/max"] <= 24 for r in m)


def test_service_backed_tools_against_a_local_server(tmp_path):
    """Search, Sandbox Fusion and MCP tools talk to one in-process HTTP server that answers in each service's format."""
    import asyncio
    import json
    import threading
    from http.server import BaseHTTPRequestHandler, HTTPServer

    from siirl_b200.execution.rollout_flow.multiturn.tools.remote_tools import TokenBucket
    from siirl_b200.execution.rollout_flow.multiturn.tools.tool_registry import initialize_tools_from_config, tools_by_name

    calls = []

    class H(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def do_POST(self):
            body = json.loads(self.rfile.read(int(self.headers["Content-Length"])))
            calls.append((self.path, body))
            if self.path == "/retrieve":
                out = {"result": [[{"document": {"contents": f"T{i}\nabout {q}"}, "score": 1.0 - i * 0.1}
                                   for i in range(body["topk"])] for q in body["queries"]]}
            elif self.path == "/run_code":
                out = {"status": "Success", "run_result": {"stdout": "42\n", "stderr": "", "return_code": 0}}
            else:
                m = body["method"]
                if m == "initialize":
                    res = {"protocolVersion": "2025-03-26", "capabilities": {}, "serverInfo": {"name": "t"}}
                elif m == "tools/list":
                    res = {"tools": [{"name": "web_search", "inputSchema": {"type": "object"}}]}
                elif m == "tools/call":
                    res = {"content": [{"type": "text", "text": json.dumps(
                        {"results": [{"title": "A", "content": body["params"]["arguments"]["query"]}]})}]}
                else:
                    res = None
                out = {"jsonrpc": "2.0", "id": body["id"], "result": res}
            data = json.dumps(out).encode()
            self.send_response(200)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

    srv = HTTPServer(("127.0.0.1", 0), H)
    port = srv.server_address[1]
    th = threading.Thread(target=srv.serve_forever, daemon=True)
    th.start()
    try:
        mcp_cfg = tmp_path / "mcp.json"
        mcp_cfg.write_text(json.dumps({"mcpServers": {"s": {"url": f"http://127.0.0.1:{port}/mcp"}}}))

        def schema(name, **props):
            return {"type": "function", "function": {"name": name, "description": name, "parameters": {
                "type": "object", "properties": {k: {"type": v} for k, v in props.items()}, "required": list(props)}}}
        tools = tools_by_name(initialize_tools_from_config({"tools": [
            {"class_name": "SearchTool", "config": {"retrieval_service_url": f"http://127.0.0.1:{port}/retrieve",
                                                    "topk": 2, "rate_limit": 100},
             "tool_schema": schema("search", query_list="array")},
            {"class_name": "SandboxFusionTool", "config": {"sandbox_fusion_url": f"http://127.0.0.1:{port}/run_code"},
             "tool_schema": schema("code_interpreter", code="string")},
            {"class_name": "McpSearchTool", "config": {"mcp_servers_config_path": str(mcp_cfg)},
             "tool_schema": schema("web_search", query="string")}]}))

        async def go():
            a = await tools["search"].execute("i", {"query_list": ["cats", "dogs"]})
            b = await tools["code_interpreter"].execute("i", {"code": "print(42)"})
            c = await tools["web_search"].execute("i", {"query": "b200"})
            d = await tools["search"].execute("i", {"query_list": []})
            return a, b, c, d
        a, b, c, d = asyncio.run(go())
        text = json.loads(a[0])["result"]
        assert "Doc 1 (Title: T0)\nabout cats" in text and "about dogs" in text and a[2]["documents"] == 4
        assert b[0] == "42" and b[2]["status"] == "Success"
        assert c[0] == "A: b200" and c[2]["status"] == "success"
        assert d[2]["status"] == "bad_request"
        methods = [body.get("method") for path, body in calls if path == "/mcp"]
        assert methods == ["initialize", "tools/list", "tools/call"]
    finally:
        srv.shutdown()
    tb = TokenBucket(rate=50, capacity=1)
    import time
    t0 = time.monotonic()
    assert all(tb.acquire(1.0) for _ in range(4))
    assert time.monotonic() - t0 >= 0.05          # 3 refills at 50 per second
