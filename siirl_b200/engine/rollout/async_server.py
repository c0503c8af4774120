"""In-process asynchronous rollout server.

The reference serves multi-turn agent loops from vLLM/SGLang ``AsyncLLM`` servers reached over ZeroMQ / HTTP
(siirl/engine/rollout/vllm_rollout/vllm_async_server.py:41-235, siirl/engine/rollout/async_server.py).  Here the
native engine lives in the worker process, so the server is an asyncio front-end over it: coroutines call
``await server.generate(request_id, prompt_ids, sampling_params)``; a batching task collects the requests that
are pending at the same moment and runs them as one engine call (continuous batching at request granularity), so
many concurrent agent loops share every decode step.  ``chat_completion`` offers the OpenAI-style schema on top.
"""
from __future__ import annotations

import asyncio
import time
import uuid
from typing import Any, Dict, List, Optional, Tuple

from .native_engine import RolloutEngine, SamplingParams


class AsyncRolloutServer:
    def __init__(self, engine: RolloutEngine, tokenizer=None, max_wait_ms: float = 2.0):
        self.engine = engine
        self.tokenizer = tokenizer
        self.max_wait_ms = max_wait_ms
        self._pending: List[Tuple[List[int], Dict[str, Any], asyncio.Future]] = []
        self._task: Optional[asyncio.Task] = None
        self._lock = asyncio.Lock()
        self.num_batches = 0
        self.inflight = 0

    async def wake_up(self) -> None:
        self.engine.wake_up()

    async def sleep(self) -> None:
        self.engine.sleep()

    def _key(self, sp: Dict[str, Any]) -> Tuple:
        return (sp.get("temperature", 1.0), sp.get("top_k", -1), sp.get("top_p", 1.0), sp.get("max_new_tokens", 16),
                sp.get("eos_token_id"), sp.get("seed", 0))

    async def generate(self, request_id: str, prompt_ids: List[int], sampling_params: Dict[str, Any]) -> Dict[str, Any]:
        """Returns ``{"token_ids": [...], "logprobs": [...], "finish_reason": str}`` for one request."""
        loop = asyncio.get_running_loop()
        fut: asyncio.Future = loop.create_future()
        self._pending.append((list(prompt_ids), dict(sampling_params), fut))
        self.inflight += 1
        if self._task is None or self._task.done():
            self._task = loop.create_task(self._drain())
        try:
            return await fut
        finally:
            self.inflight -= 1

    async def _drain(self) -> None:
        await asyncio.sleep(self.max_wait_ms / 1000.0)
        while self._pending:
            batch, self._pending = self._pending, []
            groups: Dict[Tuple, List[int]] = {}
            for i, (_, sp, _) in enumerate(batch):
                groups.setdefault(self._key(sp), []).append(i)
            for key, idxs in groups.items():
                sp0 = batch[idxs[0]][1]
                sp = SamplingParams(n=1, temperature=float(sp0.get("temperature", 1.0)), top_k=int(sp0.get("top_k", -1)),
                                    top_p=float(sp0.get("top_p", 1.0)), max_new_tokens=int(sp0.get("max_new_tokens", 16)),
                                    eos_token_id=sp0.get("eos_token_id"), seed=int(sp0.get("seed", 0)) + self.num_batches)
                prompts = [batch[i][0] for i in idxs]
                try:
                    outs = await asyncio.to_thread(self._generate_on_engine_device, prompts, sp)
                    self.num_batches += 1
                    for i, o in zip(idxs, outs):
                        batch[i][2].set_result({"token_ids": o.token_ids, "logprobs": o.logprobs,
                                                "finish_reason": o.finish_reason})
                except Exception as e:  # noqa: BLE001
                    for i in idxs:
                        if not batch[i][2].done():
                            batch[i][2].set_exception(e)
            await asyncio.sleep(0)

    def _generate_on_engine_device(self, prompts, sp):
        """Engine call from a worker thread: a new thread starts on CUDA device 0, the engine may live elsewhere."""
        dev = getattr(self.engine, "device", None)
        if dev is not None and getattr(dev, "type", "cpu") == "cuda":
            import torch
            torch.cuda.set_device(dev)
        return self.engine.generate(prompts, sp)

    async def chat_completion(self, request: Dict[str, Any]) -> Dict[str, Any]:
        """OpenAI ``/v1/chat/completions``-shaped request and response (messages, max_tokens, temperature, top_p)."""
        assert self.tokenizer is not None, "chat_completion needs a tokenizer"
        ids = self.tokenizer.apply_chat_template(request["messages"], add_generation_prompt=True, tokenize=True,
                                                 tools=request.get("tools"))
        if isinstance(ids, dict):
            ids = ids["input_ids"]
        sp = {"temperature": request.get("temperature", 1.0), "top_p": request.get("top_p", 1.0),
              "top_k": request.get("top_k", -1), "seed": request.get("seed", 0),
              "max_new_tokens": request.get("max_tokens", 256), "eos_token_id": getattr(self.tokenizer, "eos_token_id", None)}
        out = await self.generate(uuid.uuid4().hex, list(ids), sp)
        text = self.tokenizer.decode(out["token_ids"], skip_special_tokens=True)
        choice = {"index": 0, "message": {"role": "assistant", "content": text}, "finish_reason": out["finish_reason"]}
        if request.get("logprobs"):
            choice["logprobs"] = {"content": [{"token": self.tokenizer.decode([t]), "logprob": lp}
                                              for t, lp in zip(out["token_ids"], out["logprobs"])]}
        return {"id": "chatcmpl-" + uuid.uuid4().hex[:12], "object": "chat.completion", "created": int(time.time()),
                "model": request.get("model", "native"),
                "choices": [choice],
                "usage": {"prompt_tokens": len(ids), "completion_tokens": len(out["token_ids"]),
                          "total_tokens": len(ids) + len(out["token_ids"])}}


def make_async_server(engine, tokenizer, agent_cfg=None):
    """The server agent loops talk to: :class:`AsyncRolloutServer`, or the class named by
    ``rollout.agent.custom_async_server`` (``path``: a module name or a ``.py`` file, ``name``: the class; the
    reference loads a custom rollout back end the same way, agent_loop.py:323-328).  A custom class is constructed as
    ``cls(engine, tokenizer)`` and has to offer ``generate`` / ``wake_up`` / ``sleep`` like the default one."""
    custom = getattr(agent_cfg, "custom_async_server", None) if agent_cfg is not None else None
    path, name = (getattr(custom, "path", None), getattr(custom, "name", None)) if custom is not None else (None, None)
    if not path or not name:
        return AsyncRolloutServer(engine, tokenizer)
    import importlib
    import importlib.util
    import os
    if str(path).endswith(".py") or os.path.sep in str(path):
        spec = importlib.util.spec_from_file_location("siirl_custom_async_server", os.path.expanduser(str(path)))
        if spec is None or spec.loader is None:
            raise ImportError(f"rollout.agent.custom_async_server.path={path!r} is not a loadable Python file")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    else:
        mod = importlib.import_module(str(path))
    cls = getattr(mod, name, None)
    if cls is None:
        raise AttributeError(f"{path}: no class {name!r} (rollout.agent.custom_async_server.name)")
    server = cls(engine, tokenizer)
    for need in ("generate", "wake_up", "sleep"):
        if not callable(getattr(server, need, None)):
            raise TypeError(f"custom async server {name} lacks the method {need}()")
    return server
