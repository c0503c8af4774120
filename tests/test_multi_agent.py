"""Multi-agent (MARFT) workflows: the joint rollout loop, the declarative workflow file and a two-agent training run."""
import json
import os
import subprocess
import sys

import torch

from siirl_b200.data_coordinator import Batch
from siirl_b200.data_coordinator.dataloader.tokenizer import SyntheticTokenizer
from siirl_b200.execution.dag.config_loader import DAGConfigLoader
from siirl_b200.execution.rollout_flow.multi_agent.multiagent_generate import MultiAgentLoop
from siirl_b200.utils.import_string import import_string

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKFLOW = os.path.join(ROOT, "examples", "experimental", "marft", "config", "workflow_marft.yaml")


class _EchoWorker:
    """Answers every prompt with ``tag`` repeated (prompt length % 3) + 1 times."""

    def __init__(self, tok, tag, resp_len=6):
        self.tok, self.tag, self.R = tok, tag, resp_len
        self.calls = []

    def generate_sequences(self, pb: Batch) -> Batch:
        B, P = pb["input_ids"].shape
        self.calls.append([list(x) for x in pb["raw_prompt_ids"]])
        resp = torch.zeros(B, self.R, dtype=torch.long)
        mask = torch.zeros(B, self.R, dtype=torch.long)
        for i, ids in enumerate(pb["raw_prompt_ids"]):
            r = self.tok.encode(self.tag * (len(ids) % 3 + 1))
            resp[i, :len(r)] = torch.tensor(r)
            mask[i, :len(r)] = 1
        full = torch.cat([pb["input_ids"], resp], 1)
        att = torch.cat([pb["attention_mask"], mask], 1)
        pos = (att.cumsum(-1) - 1).clamp(min=0)
        out = Batch({"prompts": pb["input_ids"], "responses": resp, "input_ids": full, "attention_mask": att,
                     "position_ids": pos, "response_mask": mask}, pb.non_tensors, dict(pb.meta))
        out.meta["total_output_tokens"] = int(mask.sum())
        return out


class _StopOnB:
    """Finishes a sample when the last agent wrote exactly ``gt`` characters."""

    def reset(self):
        self.turns = 0

    async def step(self, actions, gt):
        self.turns += 1
        ok = len(actions[-1]) == int(gt)
        return [f"={len(a)}" for a in actions], float(ok), ok


def _prompts(tok, texts, gts):
    ids = [tok.encode(t) for t in texts]
    P = 16
    inp = torch.zeros(len(ids), P, dtype=torch.long)
    att = torch.zeros(len(ids), P, dtype=torch.long)
    for i, x in enumerate(ids):
        inp[i, P - len(x):] = torch.tensor(x)
        att[i, P - len(x):] = 1
    return Batch({"input_ids": inp, "attention_mask": att, "position_ids": (att.cumsum(-1) - 1).clamp(min=0)},
                 {"raw_prompt_ids": ids, "reward_model": [{"ground_truth": g} for g in gts],
                  "uid": [f"u{i}" for i in range(len(ids))]}, {})


def test_loop_runs_agents_in_order_and_lays_out_turns():
    tok = SyntheticTokenizer()
    wa, wb = _EchoWorker(tok, "a"), _EchoWorker(tok, "b")
    loop = MultiAgentLoop({1: wb, 0: wa}, tok, prompt_length=64, max_turns=3, env_factory=_StopOnB,
                          use_all_traj=True, obs_with_env=True)
    batch = _prompts(tok, ["1+1", "12+3", "7"], gts=[1, 99, 99])
    out = loop.generate_sequence(batch)
    # agent 0 always sees the prompt first; agent 1's prompt is agent 0's prompt + agent 0's response
    first_a, first_b = wa.calls[0], wb.calls[0]
    assert first_a[0] == tok.encode("1+1")
    assert first_b[0][:len(first_a[0])] == first_a[0] and tok.decode(first_b[0][len(first_a[0]):]).startswith("a")
    # sample 0 ("1+1": a -> "a", prompt 4 tokens -> b writes "bb"?) stops when b's answer has gt characters;
    # samples 1, 2 never match and use all 3 turns
    req = list(out.non_tensors["request_id"])
    lens = {r: req.count(r) for r in req}
    per_sample = [lens[r] for r in dict.fromkeys(req)]
    assert per_sample[1] == 3 and per_sample[2] == 3 and 1 <= per_sample[0] <= 3
    # rows of a sample are consecutive, latest turn first, traj_len = rows of the sample
    for r in dict.fromkeys(req):
        rows = [i for i, x in enumerate(req) if x == r]
        assert rows == list(range(rows[0], rows[0] + len(rows)))
        steps = [out.non_tensors["traj_step"][i] for i in rows]
        assert steps == sorted(steps, reverse=True)
        assert all(out.non_tensors["traj_len"][i] == len(rows) for i in rows)
    assert out.meta["agent_group_ids"] == [0]
    for key in ("responses", "response_mask", "input_ids", "attention_mask"):
        assert f"agent_group_0_{key}" in out.tensors and key in out.tensors
    # later turns restart from the original prompt plus the observation (obs_with_env)
    second_a = wa.calls[1]
    assert all(tok.decode(p).endswith(tuple("0123456789")) and "=" in tok.decode(p) for p in second_a)
    # finished samples are not generated again
    if per_sample[0] == 1:
        assert len(wa.calls[1]) == 2
    # env score of the stopping turn is 1
    rows0 = [i for i, x in enumerate(req) if x == req[0]]
    if per_sample[0] < 3:
        assert out.non_tensors["env_score"][rows0[0]] == 1.0


def test_last_turn_only_when_use_all_traj_is_off():
    tok = SyntheticTokenizer()
    loop = MultiAgentLoop({0: _EchoWorker(tok, "a"), 1: _EchoWorker(tok, "b")}, tok, 64, max_turns=2,
                          env_factory=_StopOnB, use_all_traj=False)
    out = loop.generate_sequence(_prompts(tok, ["1+1", "12+3"], gts=[99, 99]))
    assert out.batch_size == 2 and list(out.non_tensors["traj_len"]) == [1, 1]
    assert list(out.non_tensors["traj_step"]) == [1, 1]


def test_import_string_forms(tmp_path):
    f = tmp_path / "hooks.py"
    f.write_text("class Env:\n    tag = 7\n\ndef fn():\n    return 3\n")
    assert import_string(f"{f}:Env").tag == 7
    assert import_string(f"{f}:fn")() == 3
    assert import_string("os.path:join") is os.path.join
    assert import_string("os.path.join") is os.path.join
    assert import_string(f"{f}:Env") is import_string(f"{f}:Env")


def test_code_workflow_variant_loads_and_its_env_scores():
    g = DAGConfigLoader.load_from_file(WORKFLOW.replace("workflow_marft.yaml", "workflow_marft_code.yaml"))
    env_ref = g.nodes["rollout_actor"].agent_options["env_path"][0]
    env = import_string(os.path.join(ROOT, env_ref.split(":")[0]) + ":" + env_ref.split(":")[1])()
    env.reset()
    spec = json.dumps({"inputs": ["1 2\n", "5 7\n"], "outputs": ["3\n", "12\n"]})
    good = "```python\na, b = map(int, input().split())\nprint(a + b)\n```"
    obs, score, stop = env.step(["plan: add them", good], spec)
    assert score == 1.0 and stop and len(obs) == 2 and "All tests pass" in obs[1]
    obs, score, stop = env.step(["plan", "```python\nprint(3)\n```"], spec)
    assert score == 0.5 and not stop


def test_example_workflow_file_loads():
    g = DAGConfigLoader.load_from_file(WORKFLOW)
    assert sorted({n.agent_group for n in g.nodes.values()}) == [0, 1]
    order = g.get_topological_sort()
    assert order[0] == "rollout_reasoner" and order[-1] == "actor_train"
    assert g.nodes["actor_value"].agent_options["share_instance"] == 0
    assert g.nodes["reasoner_train"].agent_options["train_cycle"] == 15
    env = g.nodes["rollout_actor"].agent_options["env_path"][0]
    assert os.path.isfile(os.path.join(ROOT, env.split(":")[0]))


def test_two_agent_marft_training_run(tmp_path):
    """Two tiny policies + one shared critic, env-scored turns, alternating updates (train_cycle 1)."""
    env_file = tmp_path / "env.py"
    env_file.write_text(
        "class LenEnv:\n"
        "    def reset(self):\n        pass\n"
        "    def step(self, actions, gt):\n"
        "        s = 1.0 if len(actions[-1]) % 2 == 0 else 0.0\n"
        "        return [f'seen {len(a)}' for a in actions], s, s > 0\n")
    wf = open(WORKFLOW).read().replace("examples/experimental/marft/config/math_env.py:MathEnv", f"{env_file}:LenEnv")
    wf = wf.replace("train_cycle: 15", "train_cycle: 1")
    wf_file = tmp_path / "wf.yaml"
    wf_file.write_text(wf)
    log = tmp_path / "log"
    env = dict(os.environ, OMP_NUM_THREADS="2", SIIRL_LOG_DIR=str(log))
    env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
    args = [f"dag.workflow_path={wf_file}", "algorithm.adv_estimator=gae_marft", "data.synthetic=arith",
            "data.synthetic_size=32", "data.max_prompt_length=160", "data.max_response_length=12",
            "data.train_batch_size=4", "actor_rollout_ref.model.arch_preset=tiny", "critic.model.arch_preset=tiny",
            "actor_rollout_ref.rollout.n=1", "actor_rollout_ref.rollout.max_num_seqs=8",
            "actor_rollout_ref.actor.ppo_mini_batch_size=4", "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4",
            "critic.ppo_mini_batch_size=4", "critic.ppo_micro_batch_size_per_gpu=4",
            "actor_rollout_ref.actor.use_kl_loss=True", "actor_rollout_ref.rollout.agent.rewards_with_env=True",
            "actor_rollout_ref.rollout.multi_turn.max_assistant_turns=2",
            "actor_rollout_ref.rollout.multi_turn.use_all_traj=True", "trainer.n_gpus_per_node=1",
            "trainer.device=cpu", "trainer.val_before_train=False", "trainer.logger=['jsonl']",
            "trainer.total_training_steps=2", "trainer.save_freq=2", "trainer.test_freq=2", f"trainer.default_local_dir={tmp_path / 'ck'}"]
    out = subprocess.run([sys.executable, "-m", "siirl_b200.main_dag", *args], env=env, cwd=ROOT, capture_output=True,
                         text=True, timeout=900)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    with open(log / "metrics.jsonl") as f:
        m = [json.loads(line) for line in f]
    assert [r["step"] for r in m] == [1, 2]
    # the agents take turns being trained; the shared critic learns from both agents' tokens every step
    assert "agent_0_actor/grad_norm" in m[0] and "agent_1_actor/grad_norm" not in m[0]
    assert "agent_1_actor/grad_norm" in m[1] and "agent_0_actor/grad_norm" not in m[1]
    for r in m:
        assert r["agent_0_critic/grad_norm"] > 0 and r["agent_1_critic/grad_norm"] > 0
        assert 0.0 <= r["critic/score/mean"] <= 1.0
        assert 1 <= r["num_turns/mean"] <= r["num_turns/max"] <= 2 and 0.0 <= r["env/score_mean"] <= 1.0
    assert "val-core/all/reward/mean" in m[1]          # validation runs the joint loop too
    step = tmp_path / "ck" / "global_step_2"
    assert (step / "actor_agent_0").is_dir() and (step / "actor_agent_1").is_dir()
    assert (step / "critic_agent_0").is_dir() and not (step / "critic_agent_1").exists()
