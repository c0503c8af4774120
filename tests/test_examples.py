"""Every example launcher's overrides must parse against the config schema (catches renamed or misspelt keys)."""
import glob
import os
import re
import shlex

import pytest

from siirl_b200.params.parser import parse_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPTS = sorted(glob.glob(os.path.join(ROOT, "examples", "*", "*.sh")) +
                 glob.glob(os.path.join(ROOT, "examples", "*", "*", "*.sh")))


@pytest.mark.parametrize("script", SCRIPTS, ids=[os.path.relpath(s, ROOT) for s in SCRIPTS])
def test_example_overrides_parse(script):
    text = open(script).read().replace("\\\n", " ").replace("$HOME", "/home/user")
    cmd = [ln for ln in text.splitlines() if "siirl_b200.main_dag" in ln]
    assert cmd, "launcher does not call siirl_b200.main_dag"
    toks = [t for t in shlex.split(cmd[0]) if re.match(r"^[+~]?[A-Za-z_][\w\.]*=", t)]
    assert len(toks) >= 5
    cfg = parse_config(toks)
    assert cfg.trainer.n_gpus_per_node >= 1


def test_custom_pipeline_example_builds():
    import importlib.util
    spec = importlib.util.spec_from_file_location("custom_grpo", os.path.join(ROOT, "examples", "custom_pipeline_example",
                                                                              "custom_grpo.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    g = mod.grpo_without_reference()
    assert "actor_train" in g.nodes and "reference_log_prob" not in g.nodes


def test_custom_batch_reward_example():
    import torch
    from siirl_b200.data_coordinator import Batch
    from siirl_b200.data_coordinator.dataloader.tokenizer import SyntheticTokenizer
    from siirl_b200.params.parser import parse_config
    from siirl_b200.execution.scheduler.reward import create_reward_manager
    tok = SyntheticTokenizer()
    cfg = parse_config([f"custom_reward_function.path={ROOT}/examples/custom_reward/rewardfunc_gsm8k.py",
                        "custom_reward_function.name=compute_score", "reward_model.reward_manager=batch"])
    rm = create_reward_manager(cfg, tok)
    texts = ["so #### 42", "it is 41", "#### 7"]
    R = 12
    resp = torch.zeros(3, R, dtype=torch.long)
    mask = torch.zeros(3, R, dtype=torch.long)
    for i, t in enumerate(texts):
        ids = tok.encode(t)
        resp[i, :len(ids)] = torch.tensor(ids)
        mask[i, :len(ids)] = 1
    prompts = torch.ones(3, 4, dtype=torch.long)
    b = Batch({"prompts": prompts, "responses": resp, "attention_mask": torch.cat([torch.ones(3, 4, dtype=torch.long), mask], 1)},
              {"reward_model": [{"ground_truth": "42"}, {"ground_truth": "41"}, {"ground_truth": "8"}],
               "data_source": ["openai/gsm8k"] * 3}, {})
    reward = rm(b)
    assert reward.sum(-1).tolist() == [1.0, 0.0, 0.0]
    assert reward[0, len(tok.encode(texts[0])) - 1] == 1.0
