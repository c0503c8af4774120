"""Config loader: dotted overrides, YAML merge, coercion, errors."""
import pytest

from siirl_b200.params import ConfigError, get_by_path, parse_config, pretty


def test_overrides_and_coercion(tmp_path):
    c = parse_config(["algorithm.adv_estimator=grpo", "data.train_files=[a.parquet,b.parquet]",
                      "actor_rollout_ref.actor.optim.lr=1e-5", "actor_rollout_ref.rollout.n=8",
                      "trainer.logger=['console','jsonl']", "actor_rollout_ref.actor.use_kl_loss=True",
                      "+actor_rollout_ref.model.override_config.num_hidden_layers=2", "data.val_files=x.parquet",
                      "trainer.total_training_steps=null", "actor_rollout_ref.rollout.temperature=1"])
    assert c.algorithm.adv_estimator == "grpo" and c.data.train_files == ["a.parquet", "b.parquet"]
    assert c.actor_rollout_ref.actor.optim.lr == 1e-5 and isinstance(c.actor_rollout_ref.rollout.temperature, float)
    assert c.trainer.logger == ["console", "jsonl"] and c.data.val_files == ["x.parquet"]
    assert c.actor_rollout_ref.model.override_config == {"num_hidden_layers": 2}
    assert c.trainer.total_training_steps is None
    assert c.actor_rollout_ref.rollout.response_length == c.data.max_response_length
    assert get_by_path(c, "actor_rollout_ref.actor.optim.lr") == 1e-5
    assert "adv_estimator: grpo" in pretty(c)


def test_yaml_file_then_cli(tmp_path):
    f = tmp_path / "c.yaml"
    f.write_text("data:\n  train_batch_size: 64\nalgorithm:\n  kl_ctrl:\n    type: adaptive\n    kl_coef: 0.5\n")
    c = parse_config(["--config", str(f), "data.train_batch_size=32", "~algorithm.kl_ctrl.kl_coef"])
    assert c.data.train_batch_size == 32 and c.algorithm.kl_ctrl.type == "adaptive"
    assert c.algorithm.kl_ctrl.kl_coef == 0.001


def test_errors():
    with pytest.raises(ConfigError):
        parse_config(["algoritm.x=1"])
    with pytest.raises(ConfigError):
        parse_config(["data.train_batch_size=abc"])
    with pytest.raises(ConfigError):
        parse_config(["data.train_batch_size"])
    with pytest.raises(ConfigError):
        parse_config(["actor_rollout_ref.actor.optim.nope=1"])


def test_cpgd_switch():
    c = parse_config(["algorithm.adv_estimator=cpgd"])
    assert c.actor_rollout_ref.actor.use_cpgd_loss and c.actor_rollout_ref.actor.policy_loss.loss_mode == "cpgd"
