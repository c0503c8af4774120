"""Small host-side utilities: file helpers, device switch, rollout request schema, code scorer, activation offload
(a no-op without CUDA), wave-aware split-K factor."""
import os

import pytest
import torch


def test_fs_helpers_local(tmp_path):
    from siirl_b200.utils.extras import fs
    src = tmp_path / "a" / "x.txt"
    fs.makedirs(str(src.parent))
    src.write_text("hello")
    assert fs.exists(str(src)) and not fs.is_non_local(str(src))
    fs.copy(str(src), str(tmp_path / "b" / "y.txt"))
    assert (tmp_path / "b" / "y.txt").read_text() == "hello"
    fs.copy(str(tmp_path / "a"), str(tmp_path / "c"))
    assert (tmp_path / "c" / "x.txt").exists()
    assert fs.copy_to_local(str(src)) == str(src)
    assert fs.is_non_local("hdfs://nn/path") and len(fs.md5_encode("hdfs://nn/path")) == 32
    assert fs.get_local_temp_path("hdfs://nn/dir/model", str(tmp_path)).endswith(os.path.join("", "model"))


def test_device_helpers():
    from siirl_b200.utils.extras import device
    assert device.get_device_name() in ("cuda", "cpu")
    assert device.get_nccl_backend() in ("nccl", "gloo")
    assert device.is_npu_available is False
    device.device_synchronize()


def test_rollout_request_schema():
    from siirl_b200.engine.rollout.schemas import AsyncRolloutRequest, AsyncRolloutRequestStateEnum, FinishReasonTypeEnum
    r = AsyncRolloutRequest("r0", prompt_ids=[1, 2, 3], max_response_len=6, max_model_len=20)
    r.add_assistant_tokens([10, 11], [-0.1, -0.2])
    r.add_observation_tokens([20, 21, 22])
    r.add_assistant_tokens([12, 13], [-0.3, -0.4])
    assert r.response_loss_mask == [1, 1, 0, 0, 0, 1, 1] and r.remaining == 0
    assert r.input_ids == [1, 2, 3, 10, 11, 20, 21, 22, 12, 13] and r.position_ids == list(range(10))
    with pytest.raises(ValueError):
        r.finalize(None, {"tool": 1.0}, "tool_calls")      # a conversation cannot end in a tool call
    r.finalize(None, {"tool": 1.0}, "length")
    assert r.state == AsyncRolloutRequestStateEnum.COMPLETED and len(r.response_ids) == 6
    assert r.metrics["finish_reason"] == FinishReasonTypeEnum.LENGTH.value and r.reward_scores == {"tool": 1.0}
    assert r.response_position_ids == [3, 4, 5, 6, 7, 8]


def test_rollout_request_message_state_machine():
    """Messages join the conversation as token deltas; assistant tokens carry loss mask 1, everything else 0; the
    incrementally built ids equal one full rendering (no tokenisation drift with this template)."""
    from siirl_b200.data_coordinator.dataloader import SyntheticTokenizer
    from siirl_b200.engine.rollout.schemas import AsyncRolloutRequest, AsyncRolloutRequestStateEnum as St
    tok = SyntheticTokenizer(1024)
    r = AsyncRolloutRequest.create("r1", [{"role": "user", "content": "2+3=?"}], tok, max_response_len=64,
                                   max_model_len=256)
    assert tok.decode(r.prompt_ids) == "user:2+3=?\n" and tok.decode(r.generation_prompt_ids) == "assistant:"
    ids = r.get_generation_prompt_ids(tok)
    assert tok.decode(ids) == "user:2+3=?\nassistant:" and r.state == St.RUNNING
    assert r.get_generation_prompt_ids(tok) == ids                     # the header is appended once
    gen = tok.encode("calc(2+3)\n")
    r.add_assistant_message(tok, "calc(2+3)", tool_calls=[{"name": "calc"}], token_ids=gen, logprobs=[-0.5] * len(gen))
    assert r.state == St.TOOL_CALLING
    r.add_tool_response_messages(tok, ["5"])
    r.get_generation_prompt_ids(tok)
    r.add_assistant_message(tok, "5")                                  # re-tokenised from the text
    r.add_user_message(tok, "thanks")
    assert r.state == St.INTERACTING
    r.get_generation_prompt_ids(tok)                                   # header with no answer: finalize takes it back
    r.finalize(tok, {"acc": 1.0}, "stop")
    text = tok.decode(r.input_ids)
    assert text == "user:2+3=?\nassistant:calc(2+3)\ntool:5\nassistant:5\nuser:thanks\n"
    assert "tokenization_diffs" not in r.metrics
    masked = tok.decode([t for t, m in zip(r.input_ids, r.loss_mask) if m])
    assert masked == "calc(2+3)\n5\n"
    assert len(r.response_ids) == len(r.response_loss_mask) == len(r.response_logprobs) == len(r.response_position_ids)
    assert r.prompt_ids + r.response_ids == r.input_ids
    # a template that renders the history differently from the deltas is reported
    class Drifting(SyntheticTokenizer):
        def apply_chat_template(self, messages, add_generation_prompt=True, tokenize=False, **kw):
            text = "".join(f"{m['role']}:{m['content']}\n" for m in messages)
            if len(messages) > 3:
                text = text.replace("assistant:", "assistant: ")        # only in long histories
            if add_generation_prompt:
                text += "assistant:"
            return self.encode(text) if tokenize else text
    d = Drifting(1024)
    q = AsyncRolloutRequest.create("r2", [{"role": "user", "content": "a"}], d, tokenization_sanity_check_mode="strict")
    for turn in ("b", "c"):
        q.get_generation_prompt_ids(d)
        q.add_assistant_message(d, turn)
        q.add_user_message(d, "again")
    q.finalize(d)
    assert q.metrics.get("tokenization_diffs", 0) > 0
    q2 = AsyncRolloutRequest.create("r3", [{"role": "user", "content": "a"}], d,
                                    tokenization_sanity_check_mode="ignore_strippable")
    for turn in ("b", "c"):
        q2.get_generation_prompt_ids(d)
        q2.add_assistant_message(d, turn)
        q2.add_user_message(d, "again")
    q2.finalize(d)
    assert "tokenization_diffs" not in q2.metrics                      # the drift is whitespace only


def test_code_scorer_stdin_and_function_modes():
    from siirl_b200.utils.reward_score import compute_score
    ok = compute_score("apps", "```python\na, b = map(int, input().split())\nprint(a + b)\n```",
                       {"inputs": ["1 2\n", "5 7\n"], "outputs": ["3\n", "12\n"]})
    assert ok["score"] == 1.0 and ok["passed"] == 2
    half = compute_score("taco", "```python\ndef add(a, b):\n    return a + b\n```",
                         {"fn_name": "add", "inputs": [[1, 2], [2, 5]], "outputs": [3, 8]})
    assert half["score"] == 0.5
    crash = compute_score("codeforces", "```python\nraise SystemExit(3)\n```", {"inputs": ["1\n"], "outputs": ["1\n"]})
    assert crash["score"] == 0.0


def test_activation_offload_is_transparent_on_cpu():
    from siirl_b200.utils.model_utils.activation_offload import ActivationOffload
    off = ActivationOffload(min_bytes=0)
    x = torch.randn(8, 8, requires_grad=True)
    with off.region():
        y = (x * x).sum()
    y.backward()
    assert torch.allclose(x.grad, 2 * x)


def test_split_k_factor_fills_whole_waves():
    from siirl_b200.ops.dense import _skinny_splits
    for M, N, K in ((64, 3584, 18944), (256, 3584, 18944), (256, 3584, 3584), (128, 4608, 3584)):
        s = _skinny_splits(M, N, K)
        tiles = (N + 127) // 128 * ((M + 127) // 128) * s
        waves = -(-tiles // 148)
        assert tiles / (waves * 148) > 0.9, (M, N, K, s)
    assert _skinny_splits(256, 37888, 3584) == 1            # already more tiles than SMs


def test_math_equivalence_scorer():
    from siirl_b200.utils.reward_score import compute_score
    from siirl_b200.utils.reward_score.math_verify import is_equiv, to_number
    from fractions import Fraction
    same = [("\\frac{1}{2}", "0.5"), ("\\dfrac{3}{4}", "75\\%"), ("1,234", "1234"), ("2\\sqrt{2}", "\\sqrt{8}"),
            ("x=5", "5"), ("(1,2)", "(1, 2)"), ("\\{1,2\\}", "\\{2,1\\}"), ("3\\pi", "9.42477796"),
            ("1\\frac{1}{2}", "1.5"), ("2^{10}", "1024"), ("10 cm", "10"), ("\\frac{\\sqrt{3}}{2}", "0.8660254"),
            ("-\\frac{2}{3}", "-0.666667"), ("3, 1", "1, 3"), ("\\sqrt[3]{8}", "2"), ("90^\\circ", "90"),
            ("\\frac{2}{3}", "0.67"), ("(1,000, 2)", "(1000,2)"), ("\\text{yes}", "yes")]
    different = [("(1,2)", "(2,1)"), ("[0,1)", "[0,1]"), ("x+1", "1+x"), ("12", "13"), ("\\frac{2}{3}", "0.7"),
                 ("\\{1,2\\}", "\\{1,3\\}"), ("\\frac{1}{0}", "1")]
    for a, b in same:
        assert is_equiv(a, b), (a, b)
        assert is_equiv(b, a), (b, a)
    for a, b in different:
        assert not is_equiv(a, b), (a, b)
    assert to_number("\\frac{3}{6}") == Fraction(1, 2)
    assert to_number("__import__('os')") is None and to_number("9**9**9") is None and to_number("x") is None
    assert compute_score("prime_math", "thus \\boxed{\\frac{2}{4}}", "0.5") == 1.0
    assert compute_score("math_verify", "The answer is 7.", "\\boxed{7}") == 1.0
    assert compute_score("numina_olympiads", "no box here", "7") == 0.0


def test_memory_helpers_on_cpu():
    from siirl_b200.utils.memory_utils import memory_report, release_memory, reset_peak_stats
    rep = memory_report()
    assert set(rep) == {"allocated_gib", "reserved_gib", "max_allocated_gib", "free_gib", "total_gib"}
    assert release_memory() >= 0.0
    reset_peak_stats()


def test_external_lib_is_imported_before_models_are_built(tmp_path, monkeypatch):
    """``model.external_lib`` names modules to import (they register presets / scorers as a side effect)."""
    import sys
    import types

    from siirl_b200.dag_worker.dagworker import DAGWorker
    (tmp_path / "my_ext_lib.py").write_text("LOADED = True\n")
    monkeypatch.syspath_prepend(str(tmp_path))
    w = types.SimpleNamespace(config=types.SimpleNamespace(actor_rollout_ref=types.SimpleNamespace(
        model=types.SimpleNamespace(external_lib="my_ext_lib"))))
    DAGWorker._import_external_libs(w)
    assert sys.modules["my_ext_lib"].LOADED
    w.config.actor_rollout_ref.model.external_lib = "no_such_module_xyz"
    import pytest
    with pytest.raises(ModuleNotFoundError):
        DAGWorker._import_external_libs(w)


def test_expert_tensor_parallel_is_refused():
    import pytest

    from siirl_b200.execution.scheduler.launch import validate_config
    from siirl_b200.params import parse_config
    cfg = parse_config(["actor_rollout_ref.actor.megatron.expert_tensor_parallel_size=2", "trainer.n_gpus_per_node=1"])
    with pytest.raises(ValueError, match="expert_tensor_parallel_size"):
        validate_config(cfg, 1)


def test_dataloader_prefetch_keeps_order_and_resume_position():
    """One batch is prepared ahead by the loader threads; the sequence of batches and the checkpointed position are
    those of the synchronous loader (a prefetched, unused batch is drawn again after a resume)."""
    import torch

    from siirl_b200.data_coordinator.dataloader import DataLoaderNode, load_tokenizer
    from siirl_b200.params import parse_config
    args = ["data.synthetic=arith", "data.synthetic_size=40", "data.train_batch_size=6", "data.max_prompt_length=16",
            "actor_rollout_ref.model.arch_preset=tiny", "trainer.n_gpus_per_node=1"]
    tok = load_tokenizer(None, 1024)
    sync = DataLoaderNode(parse_config(args + ["data.num_loader_workers=0"]), tok, None, 1, 0, 1)
    pre = DataLoaderNode(parse_config(args + ["data.num_loader_workers=3"]), tok, None, 1, 0, 1)
    assert sync._pool is None and pre._pool is not None
    want = [sync.run()["input_ids"] for _ in range(9)]            # crosses an epoch boundary (40 / 6)
    got = []
    for k in range(4):
        got.append(pre.run()["input_ids"])
    state = pre.state_dict()
    assert state == {"epoch": 0, "cursor": 24, "seed": pre.seed, "batch_size": 6} and pre._ahead is not None
    resumed = DataLoaderNode(parse_config(args + ["data.num_loader_workers=3"]), tok, None, 1, 0, 1)
    resumed.load_state_dict(state)
    for k in range(5):
        got.append(resumed.run()["input_ids"])
    assert all(torch.equal(a, b) for a, b in zip(want, got))


def test_custom_async_server_is_loaded_from_a_file(tmp_path):
    import types

    import pytest

    from siirl_b200.engine.rollout.async_server import AsyncRolloutServer, make_async_server
    assert isinstance(make_async_server("engine", None, None), AsyncRolloutServer)
    f = tmp_path / "my_server.py"
    f.write_text("class Mine:\n    def __init__(self, engine, tokenizer):\n        self.engine = engine\n"
                 "    async def generate(self, *a, **k):\n        return {}\n"
                 "    async def wake_up(self):\n        pass\n    async def sleep(self):\n        pass\n"
                 "class Broken:\n    def __init__(self, engine, tokenizer):\n        pass\n")
    agent = types.SimpleNamespace(custom_async_server=types.SimpleNamespace(path=str(f), name="Mine"))
    s = make_async_server("the-engine", None, agent)
    assert type(s).__name__ == "Mine" and s.engine == "the-engine"
    agent.custom_async_server.name = "Broken"
    with pytest.raises(TypeError, match="generate"):
        make_async_server("e", None, agent)
    agent.custom_async_server.name = "Missing"
    with pytest.raises(AttributeError):
        make_async_server("e", None, agent)


def test_flops_counter_counts_active_parameters_per_family():
    """GEMM parameters one token touches: dense 7B, a routed mixture of experts, and the DeepSeek-V3 family (latent
    attention projections, shared experts, dense first layers) land on the models' published active sizes."""
    from siirl_b200.models.config import get_config
    from siirl_b200.utils.model_utils.flops_counter import FlopsCounter
    active = {n: FlopsCounter(get_config(n)).dense_params_per_token() / 1e9
              for n in ("qwen2.5-7b", "qwen3-30b-a3b", "moonlight-16b-a3b", "deepseek-v3")}
    assert 6.9 < active["qwen2.5-7b"] < 7.2              # 7.6 B with the input embedding, which is no GEMM
    assert 2.9 < active["qwen3-30b-a3b"] < 3.4           # "A3B"
    assert 2.2 < active["moonlight-16b-a3b"] < 3.0
    assert 35.0 < active["deepseek-v3"] < 38.5           # 37 B active
    f = FlopsCounter(get_config("moonlight-16b-a3b"))
    assert f.forward_flops([2048]) > 2 * f.dense_params_per_token() * 2048          # attention adds to the GEMMs
    achieved, _ = f.estimate_flops([1024, 1024], 1.0)
    assert achieved == 3 * f.forward_flops([1024, 1024]) / 1e12


def test_logging_setup_writes_rank_tagged_records(tmp_path, monkeypatch, capsys):
    import logging

    from siirl_b200.utils.logger import logging_utils as LU
    monkeypatch.setenv("SIIRL_LOG_DIR", str(tmp_path))
    monkeypatch.setenv("SIIRL_LOG_LEVEL", "debug")
    monkeypatch.setenv("RANK", "3")
    root = LU.set_basic_config(force=True)
    assert root.level == logging.DEBUG and LU.set_basic_config() is root           # second call changes nothing
    logging.getLogger("siirl_b200.engine.something").debug("hello %d", 7)
    LU.log_with_rank("only zero", 1, log_only_rank_0=True)
    LU.log_with_rank("everyone", 1)
    LU.DecoratorLoggerBase("[actor]", rank=0).log("via print")
    for h in root.handlers:
        h.flush()
    text = (tmp_path / "siirl_rank3.log").read_text()
    assert "rank 3" in text and "hello 7" in text and "[Rank 1] everyone" in text and "only zero" not in text
    assert "via print" in capsys.readouterr().out
    monkeypatch.delenv("SIIRL_LOG_DIR")
    monkeypatch.setenv("SIIRL_LOG_LEVEL", "nonsense")
    assert LU.set_basic_config(force=True).level == logging.INFO


def test_tracking_backends(tmp_path, monkeypatch, capsys):
    """Console, jsonl and TensorBoard sinks write every scalar; an unknown sink or a sink whose package is missing
    fails at construction, not in the middle of a run; MLflow gets flattened parameters through a stand-in module."""
    import json
    import sys
    import types

    import pytest

    from siirl_b200.utils.logger.tracking import Tracking, _flatten_params
    monkeypatch.setenv("SIIRL_LOG_DIR", str(tmp_path))
    monkeypatch.setenv("TENSORBOARD_DIR", str(tmp_path / "tb"))
    t = Tracking("proj", "exp", ["console", "jsonl", "tensorboard"], config={"a": {"b": 1}})
    t.log({"actor/pg_loss": 0.5, "training/global_step": 1, "note": "text is skipped by scalar sinks"}, step=1)
    t.log({"actor/pg_loss": 0.25}, step=2)
    t.finish()
    assert "step:2" in capsys.readouterr().out
    rows = [json.loads(line) for line in open(tmp_path / "metrics.jsonl")]
    assert [r["step"] for r in rows] == [1, 2] and rows[1]["actor/pg_loss"] == 0.25
    assert any(f.startswith("events.out.tfevents") for f in os.listdir(tmp_path / "tb"))
    with pytest.raises((ValueError, AssertionError, KeyError)):
        Tracking("proj", "exp", ["no_such_sink"])
    monkeypatch.setitem(sys.modules, "wandb", None)                        # importing it now raises ImportError
    with pytest.raises(ImportError):
        Tracking("proj", "exp", ["wandb"])
    assert _flatten_params({"a": {"b": 1, "c": [2, {"d": 3}]}}) == {"a/b": 1, "a/c/0": 2, "a/c/1/d": 3}
    calls = []
    fake = types.ModuleType("mlflow")
    fake.set_tracking_uri = lambda uri: calls.append(("uri", uri))
    fake.set_experiment = lambda name: (calls.append(("experiment", name)), types.SimpleNamespace(experiment_id="7"))[1]
    fake.start_run = lambda experiment_id=None, run_name=None: calls.append(("run", experiment_id, run_name))
    fake.log_params = lambda p: calls.append(("params", dict(p)))
    fake.log_metrics = lambda metrics, step=None: calls.append(("metrics", dict(metrics), step))
    fake.end_run = lambda: calls.append(("end",))
    monkeypatch.setitem(sys.modules, "mlflow", fake)
    m = Tracking("proj", "exp", ["mlflow"], config={"trainer": {"seed": 1}})
    m.log({"x/y@4": 1.5, "skip": "s"}, step=3)
    m.finish()
    kinds = [c[0] for c in calls]
    assert "params" in kinds and ("metrics" in kinds) and kinds[-1] == "end"
    logged = next(c for c in calls if c[0] == "metrics")
    assert logged[2] == 3 and logged[1] == {"x/y_at_4": 1.5} and ("run", "7", "exp") in calls
