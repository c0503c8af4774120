"""Every example launcher's overrides must parse against the config schema (catches renamed or misspelt keys)."""
import glob
import os
import re
import shlex

import pytest

from siirl_b200.params.parser import parse_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SCRIPTS = sorted(glob.glob(os.path.join(ROOT, "examples", "*", "*.sh")))


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
