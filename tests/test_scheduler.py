"""Scheduler / process-group manager / config validation."""
import pytest

from siirl_b200.execution.dag import Node, NodeRole, NodeType, Pipeline, TaskGraph, grpo_pipeline
from siirl_b200.execution.scheduler import ProcessGroupManager, TaskScheduler, update_task_graph_node_configs
from siirl_b200.execution.scheduler.launch import validate_config
from siirl_b200.execution.scheduler.task_scheduler import (_parse_model_params_string, estimate_graph_model_params,
                                                           log_schedule_assignments)
from siirl_b200.params import SiiRLArguments, parse_config


def _g(gid, params=None, n=2):
    g = TaskGraph(gid)
    prev = None
    for i in range(n):
        g.add_node(Node(f"{gid}_n{i}", NodeType.MODEL_TRAIN, NodeRole.ACTOR, dependencies=[prev] if prev else [],
                        config={"model_params": params} if params is not None else {}))
        prev = f"{gid}_n{i}"
    return g


def test_param_string_parsing():
    assert _parse_model_params_string("70B") == 70e9
    assert _parse_model_params_string("500m") == 500e6
    assert _parse_model_params_string("1.5K") == 1500
    assert _parse_model_params_string(3) == 3.0
    assert _parse_model_params_string("abc") == 0.0
    assert estimate_graph_model_params(_g("a", "7B")) == 14e9
    plain = TaskGraph("p"); plain.add_node(Node("x"))
    assert estimate_graph_model_params(plain) == 1.0


def test_single_graph_gets_all_workers():
    ts = TaskScheduler(2, 4)
    a = ts.schedule_and_assign_tasks([grpo_pipeline()])
    assert len(a) == 8 and all(g is not None for g in a.values())
    assert len(ts.get_unique_assigned_task_graphs()) == 1
    assert "8 workers" in log_schedule_assignments(a, 8, log=lambda s: None)


def test_param_aware_apportioning_and_cohesion():
    ts = TaskScheduler(2, 4)
    big, small = _g("big", "30B"), _g("small", "10B")
    a = ts.schedule_and_assign_tasks([big, small], apportion_strategy="param_aware")
    big_ranks = sorted(r for r, g in a.items() if g.graph_id.startswith("big"))
    small_ranks = sorted(r for r, g in a.items() if g.graph_id.startswith("small"))
    assert len(big_ranks) == 6 and len(small_ranks) == 2
    assert len({r // 4 for r in small_ranks}) == 1          # the small task stays on one physical node
    ts2 = TaskScheduler(1, 8)
    a2 = ts2.schedule_and_assign_tasks([big, small], apportion_strategy="even")
    assert sum(g.graph_id.startswith("big") for g in a2.values()) == 4


def test_too_many_subgraphs_raises():
    ts = TaskScheduler(1, 1)
    with pytest.raises(ValueError):
        ts.schedule_and_assign_tasks([_g("a"), _g("b")])
    assert all(v is None for v in TaskScheduler(1, 2).schedule_and_assign_tasks([]).values())


def test_process_group_manager_dedups_rank_tuples():
    fan = Pipeline("f").add_node("gen", print, node_type=NodeType.MODEL_INFERENCE, node_role=NodeRole.ROLLOUT) \
        .add_node("t1", print, ["gen"], node_type=NodeType.MODEL_TRAIN, node_role=NodeRole.ACTOR) \
        .add_node("t2", print, ["gen"], node_type=NodeType.MODEL_TRAIN, node_role=NodeRole.CRITIC).build()
    ts = TaskScheduler(1, 4)
    a = ts.schedule_and_assign_tasks([fan])
    pgm = ProcessGroupManager(4, a)
    assert pgm.get_node_assignment("gen")["ranks"] == [0, 1, 2, 3]
    r1, r2 = pgm.get_node_assignment("t1")["ranks"], pgm.get_node_assignment("t2")["ranks"]
    assert sorted(r1 + r2) == [0, 1, 2, 3] and len(pgm.process_group_spec) == 3
    assert pgm.get_process_groups_for_node_type("MODEL_TRAIN") == {pgm.get_node_assignment("t1")["process_group_name"],
                                                                   pgm.get_node_assignment("t2")["process_group_name"]}
    assert pgm.get_process_groups_for_node_type("COMPUTE") == set()
    assert pgm.get_node_assignment("nope") is None
    with pytest.raises(ValueError):
        ProcessGroupManager(0, {})
    with pytest.raises(ValueError):
        ProcessGroupManager(2, {}, relevant_node_types_param=["x"])


def test_graph_updater_attaches_role_config_and_overrides():
    cfg = SiiRLArguments()
    g = Pipeline("p").add_node("a", print, node_type=NodeType.MODEL_TRAIN, node_role=NodeRole.ACTOR) \
        .add_node("c", print, ["a"], node_type=NodeType.MODEL_TRAIN, node_role=NodeRole.CRITIC).build()
    g.nodes["a"].config = {"actor.optim.lr": 3e-4, "custom_key": 1}
    update_task_graph_node_configs(g, cfg)
    assert g.nodes["a"].config["intern_config"].actor.optim.lr == 3e-4
    assert cfg.actor_rollout_ref.actor.optim.lr == 1e-6            # global config untouched
    assert g.nodes["a"].config["custom_key"] == 1 and g.nodes["a"].config["_node_id_"] == "a"
    assert type(g.nodes["c"].config["intern_config"]).__name__ == "CriticArguments"


def test_validate_config_rules():
    ok = parse_config(["data.train_batch_size=16", "actor_rollout_ref.actor.ppo_mini_batch_size=16",
                       "algorithm.adv_estimator=grpo", "trainer.n_gpus_per_node=4"])
    validate_config(ok)
    with pytest.raises(ValueError):
        validate_config(parse_config(["data.train_batch_size=10", "trainer.n_gpus_per_node=4"]))
    with pytest.raises(ValueError):
        validate_config(parse_config(["data.train_batch_size=16", "actor_rollout_ref.actor.ppo_mini_batch_size=16",
                                      "actor_rollout_ref.actor.loss_agg_mode=bogus", "trainer.n_gpus_per_node=4"]))
    with pytest.raises(ValueError):
        validate_config(parse_config(["data.train_batch_size=16", "actor_rollout_ref.actor.ppo_mini_batch_size=16",
                                      "actor_rollout_ref.actor.ppo_micro_batch_size=4",
                                      "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=2",
                                      "trainer.n_gpus_per_node=4"]))
    with pytest.raises(ValueError):
        validate_config(parse_config(["data.train_batch_size=16", "trainer.n_gpus_per_node=4",
                                      "actor_rollout_ref.rollout.tensor_model_parallel_size=3"]))
