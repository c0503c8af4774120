"""Tools backed by a service: retrieval search, Sandbox Fusion code execution, MCP (Model Context Protocol) servers.

Counterparts of the reference's ``search_tool.py`` (+ ``utils/search_r1_like_utils.py``), ``sandbox_fusion_tools.py``
and ``mcp_base_tool.py`` / ``mcp_search_tool.py`` / ``utils/mcp_clients/McpClientManager.py``
(siirl/execution/rollout_flow/multiturn/tools/*).  Differences by design: no Ray actors for rate limiting (a
process-wide token bucket and an asyncio semaphore do it in the worker process), and the MCP client speaks JSON-RPC 2.0
over plain HTTP POST (the "streamable HTTP" transport with JSON responses) with only the standard library plus
``requests``, so no MCP SDK is needed."""
from __future__ import annotations

import asyncio
import itertools
import json
import threading
import time
from typing import Any, Dict, List, Optional, Tuple

from .base_tool import BaseTool


class TokenBucket:
    """``rate`` acquisitions per second with bursts up to ``capacity``; thread-safe, blocking ``acquire``."""

    def __init__(self, rate: float, capacity: Optional[float] = None):
        self.rate = float(rate)
        self.capacity = float(capacity if capacity is not None else max(rate, 1.0))
        self._tokens = self.capacity
        self._t = time.monotonic()
        self._lock = threading.Lock()

    def acquire(self, timeout: float = 60.0) -> bool:
        deadline = time.monotonic() + timeout
        while True:
            with self._lock:
                now = time.monotonic()
                self._tokens = min(self.capacity, self._tokens + (now - self._t) * self.rate)
                self._t = now
                if self._tokens >= 1.0:
                    self._tokens -= 1.0
                    return True
                wait = (1.0 - self._tokens) / self.rate if self.rate > 0 else timeout
            if time.monotonic() + wait > deadline:
                return False
            time.sleep(min(wait, 0.05))


def _post_json(url: str, payload: Dict[str, Any], timeout: float, headers: Optional[Dict[str, str]] = None,
               retries: int = 2) -> Tuple[int, Any]:
    """POST with retries on connection errors and 5xx; returns (status, parsed JSON or text)."""
    import requests
    last: Any = None
    for attempt in range(retries + 1):
        try:
            r = requests.post(url, json=payload, timeout=timeout, headers=headers or {})
            if r.status_code >= 500 and attempt < retries:
                last = r.text
                time.sleep(0.2 * (attempt + 1))
                continue
            try:
                return r.status_code, r.json()
            except ValueError:
                return r.status_code, r.text
        except requests.RequestException as e:
            last = f"{type(e).__name__}: {e}"
            if attempt < retries:
                time.sleep(0.2 * (attempt + 1))
    return 0, last


class _RateLimited(BaseTool):
    """Shared plumbing: ``rate_limit`` (calls per second, process-wide per tool) and ``num_workers`` (concurrency)."""

    def __init__(self, config, tool_schema):
        super().__init__(config, tool_schema)
        rate = float(self.config.get("rate_limit", 0) or 0)
        self._bucket = TokenBucket(rate) if rate > 0 else None
        self._sem: Optional[asyncio.Semaphore] = None
        self._workers = int(self.config.get("num_workers", 16))
        self.timeout = float(self.config.get("timeout", 30))

    async def _guarded(self, fn, *args):
        if self._sem is None:
            self._sem = asyncio.Semaphore(self._workers)
        async with self._sem:
            if self._bucket is not None and not await asyncio.to_thread(self._bucket.acquire, self.timeout):
                return 0, "rate limit: no slot within the tool's timeout"
            return await asyncio.to_thread(fn, *args)


def format_search_results(result: Any) -> str:
    """``[{"document": {"contents": "title\\ntext"}, "score": s}, ...]`` -> "Doc 1 (Title: ...)\\ntext" blocks
    (the passage format of Search-R1 style training data)."""
    lines = []
    for i, item in enumerate(result or []):
        doc = item.get("document", item) if isinstance(item, dict) else {"contents": str(item)}
        content = doc.get("contents") or doc.get("content") or doc.get("text") or ""
        title, _, text = content.partition("\n")
        lines.append(f"Doc {i + 1} (Title: {title.strip()})\n{text.strip() or title.strip()}")
    return "\n\n".join(lines)


class SearchTool(_RateLimited):
    """Dense-retrieval search.  Config: ``retrieval_service_url``, ``topk`` (3), ``timeout``, ``rate_limit``.
    Parameters: ``query_list`` (or ``query``).  The service receives ``{"queries", "topk", "return_scores"}`` and
    answers ``{"result": [[hit, ...] per query]}``."""

    async def execute(self, instance_id, parameters, **kw):
        url = self.config.get("retrieval_service_url") or self.config.get("url")
        if not url:
            raise RuntimeError(f"tool '{self.name}': set retrieval_service_url in the tool config")
        queries = parameters.get("query_list") or ([parameters["query"]] if parameters.get("query") else [])
        queries = [str(q) for q in queries if str(q).strip()]
        if not queries:
            return json.dumps({"result": "error: empty query_list"}), 0.0, {"status": "bad_request"}
        payload = {"queries": queries, "topk": int(self.config.get("topk", 3)), "return_scores": True}
        status, body = await self._guarded(_post_json, url, payload, self.timeout)
        if status != 200 or not isinstance(body, dict) or "result" not in body:
            return json.dumps({"result": f"search error ({status}): {str(body)[:200]}"}), 0.0, {"status": "error"}
        blocks = [format_search_results(hits) for hits in body["result"]]
        text = "\n---\n".join(blocks)
        return json.dumps({"result": text}, ensure_ascii=False), 0.0, {"status": "success", "queries": len(queries),
                                                                       "documents": sum(len(h) for h in body["result"])}


class SandboxFusionTool(_RateLimited):
    """Runs model-written code in a Sandbox Fusion service.  Config: ``sandbox_fusion_url`` (its ``/run_code``
    endpoint), ``default_timeout`` (30 s of run time), ``default_language`` (python), ``memory_limit_mb``."""

    async def execute(self, instance_id, parameters, **kw):
        url = self.config.get("sandbox_fusion_url") or self.config.get("url")
        if not url:
            raise RuntimeError(f"tool '{self.name}': set sandbox_fusion_url in the tool config")
        code = parameters.get("code")
        if not isinstance(code, str) or not code.strip():
            return "error: no code given", 0.0, {"status": "bad_request"}
        run_timeout = float(parameters.get("timeout") or self.config.get("default_timeout", 30))
        payload = {"code": code, "language": parameters.get("language") or self.config.get("default_language", "python"),
                   "run_timeout": run_timeout, "compile_timeout": run_timeout,
                   "memory_limit_MB": int(self.config.get("memory_limit_mb", 1024))}
        status, body = await self._guarded(_post_json, url, payload, run_timeout + self.timeout)
        if status != 200 or not isinstance(body, dict):
            return f"sandbox error ({status}): {str(body)[:200]}", 0.0, {"status": "error"}
        run = body.get("run_result") or {}
        out = (run.get("stdout") or "") + (run.get("stderr") or "")
        if body.get("status") != "Success" and not out:
            out = f"sandbox status: {body.get('status')} {body.get('message', '')}".strip()
        return out.strip(), 0.0, {"status": str(body.get("status", "unknown")), "return_code": run.get("return_code")}


class McpClientManager:
    """Registry of MCP servers reachable over HTTP.  Config file (JSON), the layout MCP clients share::

        {"mcpServers": {"search": {"url": "http://host:port/mcp", "auth_token": "..."}, ...}}

    ``call_tool`` finds the server that lists the tool (``tools/list`` is fetched once per server) and sends
    ``tools/call``.  One token bucket covers all servers (``rate_limit`` calls per second)."""

    def __init__(self, config_path: Optional[str] = None, servers: Optional[Dict[str, Dict[str, Any]]] = None,
                 rate_limit: float = 10.0, timeout: float = 30.0):
        if config_path:
            with open(config_path, "r", encoding="utf-8") as f:
                servers = dict((json.load(f) or {}).get("mcpServers", {}))
        self.servers: Dict[str, Dict[str, Any]] = dict(servers or {})
        self.timeout = timeout
        self._bucket = TokenBucket(rate_limit) if rate_limit and rate_limit > 0 else None
        self._ids = itertools.count(1)
        self._tools: Dict[str, List[Dict[str, Any]]] = {}
        self._initialized: set = set()
        self._lock = threading.Lock()

    def _rpc(self, server: str, method: str, params: Optional[Dict[str, Any]] = None) -> Any:
        spec = self.servers[server]
        headers = {"Accept": "application/json, text/event-stream"}
        if spec.get("auth_token"):
            headers["Authorization"] = f"Bearer {spec['auth_token']}"
        payload = {"jsonrpc": "2.0", "id": next(self._ids), "method": method, "params": params or {}}
        if self._bucket is not None and not self._bucket.acquire(self.timeout):
            raise TimeoutError("MCP rate limit: no slot within the timeout")
        status, body = _post_json(spec["url"], payload, self.timeout, headers)
        if isinstance(body, str) and "data:" in body:             # a one-event SSE reply
            for line in body.splitlines():
                if line.startswith("data:"):
                    try:
                        body = json.loads(line[5:].strip())
                        break
                    except ValueError:
                        continue
        if status != 200 or not isinstance(body, dict):
            raise RuntimeError(f"MCP server '{server}' {method}: HTTP {status}: {str(body)[:200]}")
        if "error" in body:
            raise RuntimeError(f"MCP server '{server}' {method}: {body['error']}")
        return body.get("result")

    def _ensure(self, server: str) -> None:
        with self._lock:
            if server in self._initialized:
                return
            self._rpc(server, "initialize", {"protocolVersion": "2025-03-26", "capabilities": {},
                                             "clientInfo": {"name": "siirl_b200", "version": "0"}})
            self._initialized.add(server)

    def list_tools(self, server: Optional[str] = None) -> List[Dict[str, Any]]:
        out: List[Dict[str, Any]] = []
        for name in ([server] if server else list(self.servers)):
            if name not in self._tools:
                self._ensure(name)
                res = self._rpc(name, "tools/list") or {}
                self._tools[name] = list(res.get("tools", []))
            out.extend(self._tools[name])
        return out

    def server_of(self, tool_name: str) -> str:
        self.list_tools()
        for server, tools in self._tools.items():
            if any(t.get("name") == tool_name for t in tools):
                return server
        raise KeyError(f"no MCP server offers a tool named '{tool_name}'")

    def call_tool(self, tool_name: str, arguments: Dict[str, Any]) -> Dict[str, Any]:
        server = self.server_of(tool_name)
        return self._rpc(server, "tools/call", {"name": tool_name, "arguments": arguments}) or {}


_MANAGERS: Dict[str, McpClientManager] = {}


def get_mcp_manager(config_path: str, rate_limit: float = 10.0, timeout: float = 30.0) -> McpClientManager:
    """One manager per config file and process (tools of the same file share connections and the rate limit)."""
    if config_path not in _MANAGERS:
        _MANAGERS[config_path] = McpClientManager(config_path, rate_limit=rate_limit, timeout=timeout)
    return _MANAGERS[config_path]


class McpTool(_RateLimited):
    """A tool served by an MCP server.  Config: ``mcp_servers_config_path`` (or inline ``mcp_servers``),
    ``rate_limit``, ``timeout``.  The function name of the tool schema is the MCP tool's name."""

    def __init__(self, config, tool_schema):
        super().__init__(config, tool_schema)
        path = self.config.get("mcp_servers_config_path")
        rate = float(self.config.get("rate_limit", 10) or 0)
        if path:
            self.manager = get_mcp_manager(path, rate, self.timeout)
        else:
            self.manager = McpClientManager(servers=self.config.get("mcp_servers"), rate_limit=rate,
                                            timeout=self.timeout)
        self._bucket = None          # the manager's bucket already limits the calls

    def parse_result(self, result: Dict[str, Any]) -> Tuple[str, Dict[str, Any]]:
        parts = [c.get("text", "") for c in result.get("content", []) if isinstance(c, dict) and c.get("type") == "text"]
        return "\n".join(p for p in parts if p), {"is_error": bool(result.get("isError", False))}

    async def execute(self, instance_id, parameters, **kw):
        try:
            status_or_result = await self._guarded(lambda: (200, self.manager.call_tool(self.name, dict(parameters))))
            result = status_or_result[1]
            if not isinstance(result, dict):
                return f"error: {result}", 0.0, {"status": "error"}
        except Exception as e:  # noqa: BLE001 - a failing tool call is an observation for the model, not a crash
            return f"error: {type(e).__name__}: {e}", 0.0, {"status": "error"}
        text, meta = self.parse_result(result)
        return text, 0.0, {"status": "error" if meta["is_error"] else "success"}


class McpSearchTool(McpTool):
    """MCP search servers answer with a JSON document per text part; keep the ``query`` / ``results`` fields."""

    def parse_result(self, result):
        text, meta = super().parse_result(result)
        try:
            data = json.loads(text)
            if isinstance(data, dict):
                hits = data.get("results") or data.get("result") or []
                text = "\n".join(f"{h.get('title', '')}: {h.get('content') or h.get('snippet') or ''}".strip(": ")
                                 if isinstance(h, dict) else str(h) for h in hits) or text
        except ValueError:
            pass
        return text, meta
