"""Asynchronous actor/rollout worker (reference: siirl/engine/fsdp_workers.py AsyncActorRolloutRefWorker and
siirl/engine/rollout/async_server.py): the same hybrid worker, with the rollout engine behind an in-process
request server so that agent loops (multi-turn, tools, multi-agent) submit single requests concurrently and the
server batches them into engine calls."""
from __future__ import annotations

import asyncio
from typing import Any, Dict, List

from .rollout.async_server import make_async_server
from .workers import ActorRolloutRefWorker


class AsyncActorRolloutRefWorker(ActorRolloutRefWorker):
    def init_model(self) -> None:
        super().init_model()
        self.server = make_async_server(self.engine, self.tokenizer, getattr(self.config.rollout, "agent", None)) \
            if self.engine is not None else None

    async def generate(self, request_id: str, prompt_ids: List[int], sampling_params: Dict[str, Any]) -> Dict[str, Any]:
        return await self.server.generate(request_id, prompt_ids, sampling_params)

    async def chat_completion(self, request: Dict[str, Any]) -> Dict[str, Any]:
        return await self.server.chat_completion(request)

    async def wake_up(self) -> None:
        await self.server.wake_up()

    async def sleep(self) -> None:
        await self.server.sleep()

    def start_http_server(self, host: str = "127.0.0.1", port: int = 0) -> str:
        """Serve the engine over an OpenAI-compatible HTTP API (``/v1/chat/completions``, ``/v1/completions``,
        ``/generate``); returns ``host:port``."""
        from .rollout.http_server import OpenAIHttpServer
        self.http = OpenAIHttpServer(self.server, host, port, model_name=str(self.config.model.path or "native"))
        return self.http.start()

    def start_zmq_server(self, address: str = "tcp://127.0.0.1:0") -> str:
        from .rollout.http_server import ZmqRolloutServer
        self.zmq = ZmqRolloutServer(self.server, address)
        return self.zmq.address

    def generate_many(self, prompts: List[List[int]], sampling_params: Dict[str, Any]) -> List[Dict[str, Any]]:
        """Synchronous convenience for callers without an event loop."""
        async def run():
            return await asyncio.gather(*[self.generate(f"r{i}", p, sampling_params) for i, p in enumerate(prompts)])
        loop = asyncio.new_event_loop()
        try:
            return loop.run_until_complete(run())
        finally:
            loop.close()
