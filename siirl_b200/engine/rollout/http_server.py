"""Network front ends of the asynchronous rollout server.

The reference reaches its vLLM / SGLang engines from the agent loops over HTTP (an OpenAI-compatible
``/v1/chat/completions`` endpoint served by FastAPI, siirl/engine/rollout/async_server.py and
vllm_rollout/vllm_async_server.py:92-235) and drives the engine workers over ZeroMQ
(vllm_async_server.py:41-90).  The native engine lives in the trainer's process, so both transports here are thin
front ends over :class:`AsyncRolloutServer`:

* :class:`OpenAIHttpServer` -- FastAPI + uvicorn in a background thread: ``GET /health``, ``GET /v1/models``,
  ``POST /v1/chat/completions``, ``POST /v1/completions`` and the token-level ``POST /generate`` the agent loops use
  (prompt ids in, token ids + log-probs out).  ``n``, ``max_tokens``, ``temperature``, ``top_p``, ``top_k``,
  ``logprobs`` and ``tools`` are honoured; streaming is not offered (training rollouts consume whole completions).
* :class:`ZmqRolloutServer` / :class:`ZmqRolloutClient` -- a REQ/REP pair carrying pickled ``(method, kwargs)``
  calls for processes on the same host that want the engine without HTTP overhead.

Both bind to the loopback interface by default: they expose the policy being trained and accept pickles (ZeroMQ), so
they must not listen on a public address.
"""
from __future__ import annotations

import asyncio
import pickle
import threading
import time
import uuid
from typing import Any, Dict, List, Optional

from .async_server import AsyncRolloutServer


class OpenAIHttpServer:
    def __init__(self, server: AsyncRolloutServer, host: str = "127.0.0.1", port: int = 0, model_name: str = "native"):
        self.server = server
        self.host, self.port = host, port
        self.model_name = model_name
        self._uvicorn = None
        self._thread: Optional[threading.Thread] = None
        self.app = self._build_app()

    # ---- routes -----------------------------------------------------------------------------------------------------------
    def _build_app(self):
        from fastapi import FastAPI, HTTPException

        app = FastAPI(title="siirl_b200 rollout server")
        srv = self.server

        @app.get("/health")
        async def health():
            return {"status": "ok", "inflight": srv.inflight, "batches": srv.num_batches}

        @app.get("/v1/models")
        async def models():
            return {"object": "list", "data": [{"id": self.model_name, "object": "model", "owned_by": "siirl_b200"}]}

        @app.post("/v1/chat/completions")
        async def chat(request: Dict[str, Any]):
            if not request.get("messages"):
                raise HTTPException(status_code=400, detail="'messages' is required")
            if request.get("stream"):
                raise HTTPException(status_code=400, detail="streaming is not supported")
            n = max(1, int(request.get("n", 1)))
            outs = await asyncio.gather(*[srv.chat_completion(dict(request, seed=int(request.get("seed", 0)) + i))
                                          for i in range(n)])
            first = outs[0]
            for i, o in enumerate(outs[1:], start=1):
                c = o["choices"][0]
                c["index"] = i
                first["choices"].append(c)
                for k in ("completion_tokens", "total_tokens"):
                    first["usage"][k] += o["usage"]["completion_tokens"]
            return first

        @app.post("/v1/completions")
        async def completions(request: Dict[str, Any]):
            prompt = request.get("prompt")
            if prompt is None:
                raise HTTPException(status_code=400, detail="'prompt' is required")
            tok = srv.tokenizer
            if isinstance(prompt, str):
                if tok is None:
                    raise HTTPException(status_code=400, detail="text prompts need a tokenizer; send token ids")
                ids = tok.encode(prompt)
            else:
                ids = [int(t) for t in prompt]
            sp = _sampling(request, tok)
            out = await srv.generate(uuid.uuid4().hex, ids, sp)
            text = tok.decode(out["token_ids"], skip_special_tokens=True) if tok is not None else ""
            choice = {"index": 0, "text": text, "finish_reason": out["finish_reason"], "token_ids": out["token_ids"]}
            if request.get("logprobs"):
                choice["logprobs"] = {"token_logprobs": out["logprobs"]}
            return {"id": "cmpl-" + uuid.uuid4().hex[:12], "object": "text_completion", "created": int(time.time()),
                    "model": request.get("model", self.model_name), "choices": [choice],
                    "usage": {"prompt_tokens": len(ids), "completion_tokens": len(out["token_ids"]),
                              "total_tokens": len(ids) + len(out["token_ids"])}}

        @app.post("/generate")
        async def generate(request: Dict[str, Any]):
            ids = request.get("prompt_ids")
            if not ids:
                raise HTTPException(status_code=400, detail="'prompt_ids' is required")
            return await srv.generate(str(request.get("request_id") or uuid.uuid4().hex), [int(t) for t in ids],
                                      dict(request.get("sampling_params") or {}))

        return app

    # ---- life cycle --------------------------------------------------------------------------------------------------------
    def start(self, wait_s: float = 20.0) -> str:
        """Serve in a daemon thread; returns ``host:port`` once the socket accepts connections."""
        import socket

        import uvicorn
        if self.port == 0:
            with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
                s.bind((self.host, 0))
                self.port = s.getsockname()[1]
        cfg = uvicorn.Config(self.app, host=self.host, port=self.port, log_level="warning", access_log=False)
        self._uvicorn = uvicorn.Server(cfg)
        self._thread = threading.Thread(target=self._uvicorn.run, name="siirl-rollout-http", daemon=True)
        self._thread.start()
        deadline = time.time() + wait_s
        while time.time() < deadline:
            if getattr(self._uvicorn, "started", False):
                return self.address
            time.sleep(0.05)
        raise RuntimeError(f"rollout HTTP server did not start on {self.host}:{self.port}")

    @property
    def address(self) -> str:
        return f"{self.host}:{self.port}"

    def stop(self) -> None:
        if self._uvicorn is not None:
            self._uvicorn.should_exit = True
        if self._thread is not None:
            self._thread.join(timeout=10)
            self._thread = None


def _sampling(request: Dict[str, Any], tok) -> Dict[str, Any]:
    return {"temperature": float(request.get("temperature", 1.0)), "top_p": float(request.get("top_p", 1.0)),
            "top_k": int(request.get("top_k", -1)), "max_new_tokens": int(request.get("max_tokens", 256)),
            "eos_token_id": getattr(tok, "eos_token_id", None), "seed": int(request.get("seed", 0))}


class ZmqRolloutServer:
    """REP socket on ``tcp://host:port`` (or ``ipc://path``) answering pickled ``(method, kwargs)`` requests with
    pickled ``("ok", result)`` / ``("error", message)``.  Methods: ``generate``, ``chat_completion``, ``wake_up``,
    ``sleep``, ``health``."""

    def __init__(self, server: AsyncRolloutServer, address: str = "tcp://127.0.0.1:0"):
        import zmq
        self.server = server
        self._ctx = zmq.Context.instance()
        self._sock = self._ctx.socket(zmq.REP)
        if address.endswith(":0"):
            port = self._sock.bind_to_random_port(address[:-2])
            self.address = f"{address[:-2]}:{port}"
        else:
            self._sock.bind(address)
            self.address = address
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._loop, name="siirl-rollout-zmq", daemon=True)
        self._thread.start()

    def _loop(self) -> None:
        import zmq
        loop = asyncio.new_event_loop()
        poller = zmq.Poller()
        poller.register(self._sock, zmq.POLLIN)
        try:
            while not self._stop.is_set():
                if not dict(poller.poll(100)):
                    continue
                try:
                    method, kwargs = pickle.loads(self._sock.recv())
                    if method == "health":
                        reply = ("ok", {"inflight": self.server.inflight, "batches": self.server.num_batches})
                    elif method in ("generate", "chat_completion", "wake_up", "sleep"):
                        reply = ("ok", loop.run_until_complete(getattr(self.server, method)(**kwargs)))
                    else:
                        reply = ("error", f"unknown method '{method}'")
                except Exception as e:  # noqa: BLE001  (the caller gets the message; the server keeps serving)
                    reply = ("error", f"{type(e).__name__}: {e}")
                self._sock.send(pickle.dumps(reply))
        finally:
            loop.close()
            self._sock.close(0)

    def stop(self) -> None:
        self._stop.set()
        self._thread.join(timeout=5)


class ZmqRolloutClient:
    def __init__(self, address: str, timeout_ms: int = 600000):
        import zmq
        self._sock = zmq.Context.instance().socket(zmq.REQ)
        self._sock.setsockopt(zmq.RCVTIMEO, timeout_ms)
        self._sock.setsockopt(zmq.LINGER, 0)
        self._sock.connect(address)

    def call(self, method: str, **kwargs) -> Any:
        self._sock.send(pickle.dumps((method, kwargs)))
        status, payload = pickle.loads(self._sock.recv())
        if status != "ok":
            raise RuntimeError(payload)
        return payload

    def generate(self, request_id: str, prompt_ids: List[int], sampling_params: Dict[str, Any]) -> Dict[str, Any]:
        return self.call("generate", request_id=request_id, prompt_ids=prompt_ids, sampling_params=sampling_params)

    def close(self) -> None:
        self._sock.close(0)
