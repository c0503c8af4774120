"""Planner unit tests: node model, task graph, pipeline builder, declarative loader, graph splitting."""
import json

import pytest

from siirl_b200.execution.dag import (DAGConfigLoader, Node, NodeRole, NodeStatus, NodeType, Pipeline, TaskGraph,
                                      dapo_pipeline, discover_and_split_parallel_paths, embodied_srpo_pipeline,
                                      generate_structural_signature, grpo_pipeline, ppo_pipeline)


def _fn(batch=None, **kw):
    return ("ran", batch)


class Owner:
    def method(self, batch=None, **kw):
        return ("method", self, batch)


def test_node_basics_and_validation():
    n = Node("a", NodeType.COMPUTE, executable_ref=_fn, dependencies=["x", "x"])
    assert n.dependencies == ["x"] and n.status == NodeStatus.PENDING
    with pytest.raises(ValueError):
        Node("")
    with pytest.raises(ValueError):
        n.add_dependency("a")
    with pytest.raises(ValueError):
        Node("b", NodeType.DATA_LOAD, NodeRole.ACTOR)
    assert n.run(batch=3) == ("ran", 3) and n.status == NodeStatus.COMPLETED


def test_node_string_refs_and_binding():
    n = Node("m", executable_ref="tests.test_dag:Owner.method")
    o = Owner()
    assert n.run(batch=1, _dag_worker_instance=o) == ("method", o, 1)
    f = Node("f", executable_ref="tests.test_dag:_fn")
    assert f.run(batch=2, _dag_worker_instance=o) == ("ran", 2)
    with pytest.raises(ImportError):
        Node("bad", executable_ref="no_such_mod_xyz:fn").run()
    with pytest.raises(AttributeError):
        Node("bad2", executable_ref="tests.test_dag:nope").run()


def test_node_failure_and_retry_counters():
    def boom(**kw):
        raise RuntimeError("x")
    n = Node("r", executable_ref=boom, retry_limit=2)
    with pytest.raises(RuntimeError):
        n.run()
    assert n.status == NodeStatus.FAILED and "RuntimeError" in n.error_info
    assert n.can_retry()
    n.increment_retry_count(); n.increment_retry_count()
    assert not n.can_retry()
    n.reset()
    assert n.status == NodeStatus.PENDING and n.retries_done == 0


def test_task_graph_validation_and_topology():
    g = TaskGraph("g")
    g.add_nodes([Node("a"), Node("b", dependencies=["a"]), Node("c", dependencies=["a"]), Node("d", dependencies=["b", "c"])])
    assert g.validate_graph() == (True, None)
    order = g.get_topological_sort()
    assert order.index("a") < order.index("b") < order.index("d") and order.index("c") < order.index("d")
    assert [n.node_id for n in g.get_entry_nodes()] == ["a"] and [n.node_id for n in g.get_exit_nodes()] == ["d"]
    with pytest.raises(ValueError):
        g.add_node(Node("a"))
    g.add_node(Node("e", dependencies=["zzz"]))
    ok, msg = g.validate_graph()
    assert not ok and "zzz" in msg
    cyc = TaskGraph("c")
    cyc.add_nodes([Node("x", dependencies=["y"]), Node("y", dependencies=["x"])])
    assert not cyc.validate_graph()[0]
    with pytest.raises(ValueError):
        cyc.get_topological_sort()


def test_builtin_pipelines_have_reference_node_ids():
    assert grpo_pipeline().get_topological_sort() == ["rollout_actor", "function_reward", "calculate_advantages",
                                                      "actor_old_log_prob", "reference_log_prob", "actor_train"]
    p = ppo_pipeline()
    assert {"compute_value", "critic_train"} <= set(p.nodes)
    assert p.nodes["actor_old_log_prob"].only_forward_compute
    assert "dynamic_sampling" in dapo_pipeline().nodes
    assert embodied_srpo_pipeline().nodes["dynamic_sampling"].node_role == NodeRole.DYNAMIC_SAMPLING


def test_pipeline_builder_contract():
    p = Pipeline("p").add_node("a", _fn).add_node("b", _fn, deps=["a"], node_type=NodeType.MODEL_TRAIN,
                                                  node_role=NodeRole.ACTOR, only_forward_compute=True, my_opt=5)
    with pytest.raises(ValueError):
        p.add_node("a", _fn)
    g = p.build()
    assert g.nodes["b"].only_forward_compute and g.nodes["b"].user_options["my_opt"] == 5
    with pytest.raises(ValueError):
        Pipeline("q").add_node("a", _fn, deps=["missing"]).build()


def test_yaml_loader_with_refs(tmp_path):
    text = """
dag_id: demo
global_config: {lr: 0.5, nested: {x: 7}}
nodes:
  - node_id: gen
    node_type: MODEL_INFERENCE
    node_role: ROLLOUT
    executable_ref: "tests.test_dag:_fn"
    config: {lr: !Ref global_config.lr, x: !Ref global_config.nested.x}
  - node_id: train
    node_type: model_train
    node_role: actor
    dependencies: [gen]
"""
    f = tmp_path / "d.yaml"
    f.write_text(text)
    g = DAGConfigLoader.load_from_file(str(f))
    assert g.nodes["gen"].config["lr"] == 0.5 and g.nodes["gen"].config["x"] == 7
    assert g.nodes["train"].node_type == NodeType.MODEL_TRAIN
    bad = text.replace("global_config.lr", "global_config.missing")
    with pytest.raises(ValueError):
        DAGConfigLoader.load_from_string(bad)
    with pytest.raises(ValueError):
        DAGConfigLoader.from_dict({"dag_id": "x", "nodes": [{"node_id": "a", "node_type": "BOGUS"}]})
    with pytest.raises(ValueError):
        DAGConfigLoader.from_dict({"dag_id": "x", "nodes": [{"node_id": "a", "node_type": "COMPUTE"},
                                                            {"node_id": "a", "node_type": "COMPUTE"}]})
    j = tmp_path / "d.json"
    j.write_text(json.dumps({"dag_id": "j", "nodes": [{"node_id": "a", "node_type": "COMPUTE"}]}))
    assert len(DAGConfigLoader.load_from_file(str(j), "json")) == 1


def test_graph_splitting():
    chain = grpo_pipeline()
    parts = discover_and_split_parallel_paths(chain)
    assert len(parts) == 1 and generate_structural_signature(parts[0]) == generate_structural_signature(chain)
    diamond = Pipeline("d").add_node("a", _fn).add_node("b", _fn, ["a"]).add_node("c", _fn, ["a"]) \
        .add_node("d", _fn, ["b", "c"]).build()
    parts = discover_and_split_parallel_paths(diamond)
    assert sorted(sorted(p.nodes) for p in parts) == [["a", "b", "d"], ["a", "c", "d"]]
    fan = Pipeline("f").add_node("a", _fn).add_node("b", _fn, ["a"]).add_node("c", _fn, ["a"]).build()
    parts = discover_and_split_parallel_paths(fan)
    assert sorted(sorted(p.nodes) for p in parts) == [["a", "b"], ["a", "c"]]
    for p in parts:
        assert p.validate_graph()[0]
    join = Pipeline("j").add_node("a", _fn).add_node("b", _fn).add_node("c", _fn, ["a", "b"]).build()
    parts = discover_and_split_parallel_paths(join)
    assert sorted(sorted(p.nodes) for p in parts) == [["a", "c"], ["b", "c"]]
