"""Built-in tools: GSM8K answer checker, Geo3K checker, calculator, local-corpus search, sandboxed Python.

Counterparts of the reference's gsm8k / geo3k / search / sandbox-fusion / MCP tools
(siirl/execution/rollout_flow/multiturn/tools/*).  The service-backed tools (retrieval server, Sandbox Fusion, MCP
servers) are in ``remote_tools.py``; the offline variants below (``LocalSearchTool`` over an in-memory corpus, ``PythonSandboxTool`` in a subprocess with a
time limit) make multi-turn training runnable without network."""
from __future__ import annotations

import ast
import asyncio
import json
import operator
import sys
from typing import Any, Dict, Tuple

from .....utils.reward_score import gsm8k as gsm8k_score
from .....utils.reward_score import math as math_score
from .base_tool import BaseTool


class Gsm8kTool(BaseTool):
    """The model submits an answer; the tool replies with the parsed value and rewards improvement."""

    def __init__(self, config, tool_schema):
        super().__init__(config, tool_schema)
        self._state: Dict[str, Dict[str, Any]] = {}

    async def create(self, instance_id=None, ground_truth=None, **kw) -> str:
        iid = await super().create(instance_id)
        self._state[iid] = {"response": "", "ground_truth": ground_truth, "reward": 0.0}
        return iid

    async def execute(self, instance_id, parameters, **kw) -> Tuple[str, float, Dict[str, Any]]:
        ans = str(parameters.get("answer", ""))
        st = self._state[instance_id]
        st["response"] = ans if ans.startswith("#### ") else "#### " + ans
        r = await self.calc_reward(instance_id)
        delta = 0.0 if r > st["reward"] else -0.05      # penalise non-improving submissions
        st["reward"] = max(st["reward"], r)
        return f"Current parsed answer={ans} reward={r}", delta, {}

    async def calc_reward(self, instance_id, **kw) -> float:
        st = self._state[instance_id]
        return gsm8k_score.compute_score(st["response"], st["ground_truth"], method="flexible")

    async def release(self, instance_id, **kw) -> None:
        self._state.pop(instance_id, None)


class Geo3kTool(Gsm8kTool):
    async def calc_reward(self, instance_id, **kw) -> float:
        st = self._state[instance_id]
        return math_score.compute_score("\\boxed{" + st["response"].replace("#### ", "") + "}", st["ground_truth"])


_OPS = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.Div: operator.truediv,
        ast.Pow: operator.pow, ast.USub: operator.neg, ast.Mod: operator.mod, ast.FloorDiv: operator.floordiv}


def _safe_eval(node):
    if isinstance(node, ast.Expression):
        return _safe_eval(node.body)
    if isinstance(node, ast.Constant) and isinstance(node.value, (int, float)):
        return node.value
    if isinstance(node, ast.BinOp) and type(node.op) in _OPS:
        return _OPS[type(node.op)](_safe_eval(node.left), _safe_eval(node.right))
    if isinstance(node, ast.UnaryOp) and type(node.op) in _OPS:
        return _OPS[type(node.op)](_safe_eval(node.operand))
    raise ValueError("unsupported expression")


class CalculatorTool(BaseTool):
    async def execute(self, instance_id, parameters, **kw):
        expr = str(parameters.get("expression", ""))
        try:
            return str(_safe_eval(ast.parse(expr, mode="eval"))), 0.0, {}
        except Exception as e:  # noqa: BLE001
            return f"error: {e}", 0.0, {"calc_error": 1}


class LocalSearchTool(BaseTool):
    """Keyword search over ``config["corpus"]`` (list of strings) — offline stand-in for the retrieval service."""

    async def execute(self, instance_id, parameters, **kw):
        qs = parameters.get("query_list") or [parameters.get("query", "")]
        corpus = self.config.get("corpus", [])
        topk = int(self.config.get("topk", 3))
        out = []
        for q in qs:
            words = set(str(q).lower().split())
            scored = sorted(corpus, key=lambda d: -len(words & set(d.lower().split())))[:topk]
            out.append({"query": q, "documents": scored})
        return json.dumps({"result": out}, ensure_ascii=False), 0.0, {"queries": len(qs)}


class RemoteServiceTool(BaseTool):
    """Base of tools backed by an HTTP service (retrieval server, Sandbox Fusion, MCP gateway)."""

    async def execute(self, instance_id, parameters, **kw):
        url = self.config.get("url") or self.config.get("retrieval_service_url") or self.config.get("sandbox_fusion_url")
        if not url:
            raise RuntimeError(f"tool '{self.name}' needs a service url in its config; none is set")
        import requests
        timeout = float(self.config.get("timeout", 30))
        resp = await asyncio.to_thread(requests.post, url, json=parameters, timeout=timeout)
        return resp.text, 0.0, {"status": resp.status_code}


class PythonSandboxTool(BaseTool):
    """Runs ``parameters["code"]`` in a fresh interpreter with a time limit; returns stdout/stderr."""

    async def execute(self, instance_id, parameters, **kw):
        code = str(parameters.get("code", ""))
        timeout = float(self.config.get("default_timeout", 10))
        proc = await asyncio.create_subprocess_exec(sys.executable, "-I", "-c", code, stdout=asyncio.subprocess.PIPE,
                                                    stderr=asyncio.subprocess.PIPE)
        try:
            out, err = await asyncio.wait_for(proc.communicate(), timeout=timeout)
        except asyncio.TimeoutError:
            proc.kill()
            return "error: timeout", 0.0, {"timeout": 1}
        text = out.decode(errors="replace") + (("\n" + err.decode(errors="replace")) if err else "")
        return text.strip(), 0.0, {"returncode": proc.returncode}
