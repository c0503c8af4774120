"""Network front ends of the asynchronous rollout server: OpenAI-compatible HTTP API and the ZeroMQ transport."""
import json
import urllib.error
import urllib.request

import pytest
import torch

from siirl_b200.data_coordinator.dataloader import SyntheticTokenizer
from siirl_b200.engine.rollout.async_server import AsyncRolloutServer
from siirl_b200.engine.rollout.http_server import OpenAIHttpServer, ZmqRolloutClient, ZmqRolloutServer
from siirl_b200.engine.rollout.native_engine import RolloutEngine
from siirl_b200.models.config import get_config
from siirl_b200.models.decoder import build_model


@pytest.fixture(scope="module")
def server():
    cfg = get_config("tiny")
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=1)
    engine = RolloutEngine(model, max_num_seqs=8, max_model_len=128, num_blocks=32)
    return AsyncRolloutServer(engine, SyntheticTokenizer(cfg.vocab_size))


def _post(addr, path, body):
    req = urllib.request.Request(f"http://{addr}{path}", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    return json.loads(urllib.request.urlopen(req, timeout=60).read())


def test_openai_compatible_http_api(server):
    http = OpenAIHttpServer(server)
    addr = http.start()
    try:
        assert json.loads(urllib.request.urlopen(f"http://{addr}/health", timeout=10).read())["status"] == "ok"
        assert json.loads(urllib.request.urlopen(f"http://{addr}/v1/models", timeout=10).read())["data"][0]["id"]
        r = _post(addr, "/v1/chat/completions", {"messages": [{"role": "user", "content": "1+1=?"}], "max_tokens": 5,
                                                 "temperature": 0.0, "n": 2, "logprobs": True})
        assert r["object"] == "chat.completion" and [c["index"] for c in r["choices"]] == [0, 1]
        assert r["choices"][0]["message"]["role"] == "assistant" and r["choices"][0]["finish_reason"] == "length"
        assert len(r["choices"][0]["logprobs"]["content"]) == 5
        assert r["usage"]["completion_tokens"] == 10 and r["usage"]["total_tokens"] == r["usage"]["prompt_tokens"] + 10
        g = _post(addr, "/generate", {"prompt_ids": [5, 6, 7], "sampling_params": {"max_new_tokens": 4,
                                                                                   "temperature": 0.0}})
        c = _post(addr, "/v1/completions", {"prompt": [5, 6, 7], "max_tokens": 4, "temperature": 0.0, "logprobs": 1})
        assert c["choices"][0]["token_ids"] == g["token_ids"] and len(g["logprobs"]) == 4
        assert c["choices"][0]["logprobs"]["token_logprobs"] == g["logprobs"]
        with pytest.raises(urllib.error.HTTPError) as err:
            _post(addr, "/v1/chat/completions", {"max_tokens": 3})
        assert err.value.code == 400
    finally:
        http.stop()


def test_zeromq_transport(server):
    z = ZmqRolloutServer(server)
    c = ZmqRolloutClient(z.address, timeout_ms=60000)
    try:
        assert "inflight" in c.call("health")
        out = c.generate("r", [5, 6, 7], {"max_new_tokens": 4, "temperature": 0.0})
        assert len(out["token_ids"]) == 4 and out["finish_reason"] == "length"
        with pytest.raises(RuntimeError):
            c.call("no_such_method")
        assert len(c.generate("r2", [9, 9], {"max_new_tokens": 2, "temperature": 0.0})["token_ids"]) == 2
    finally:
        c.close()
        z.stop()
