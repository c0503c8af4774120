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


def _simulate_pipeline(P, M, V):
    """Run every stage's order against blocking receives and asynchronous, order-matched sends (the transport of
    ``parallel/pipeline.py``): returns the number of executed passes; raises on a deadlock or when the k-th receive
    on a link would not get the k-th message sent on it."""
    from siirl_b200.parallel.pipeline import schedule_interleaved
    orders = [schedule_interleaved(s, P, M, V) for s in range(P)]
    at = [0] * P
    sent = {}                                   # (kind, src, dst) -> list of message tags in sending order
    taken = {}                                  # (kind, src, dst) -> number of messages received so far
    total = sum(len(o) for o in orders)
    done = 0
    last_chunk = V - 1
    while done < total:
        progressed = False
        for s in range(P):
            while at[s] < len(orders[s]):
                op, i, c = orders[s][at[s]]
                if op == "F":
                    first = s == 0 and c == 0
                    if not first:
                        src = (s - 1) % P
                        link = ("F", src, s)
                        k = taken.get(link, 0)
                        if k >= len(sent.get(link, [])):
                            break                                           # would block in recv
                        want = (i, c if s > 0 else c - 1)
                        assert sent[link][k] == want, f"stage {s}: forward recv {k} gets {sent[link][k]}, needs {want}"
                        taken[link] = k + 1
                    if not (s == P - 1 and c == last_chunk):
                        sent.setdefault(("F", s, (s + 1) % P), []).append((i, c))
                else:
                    last = s == P - 1 and c == last_chunk
                    if not last:
                        src = (s + 1) % P
                        link = ("B", src, s)
                        k = taken.get(link, 0)
                        if k >= len(sent.get(link, [])):
                            break
                        want = (i, c if s < P - 1 else c + 1)
                        assert sent[link][k] == want, f"stage {s}: backward recv {k} gets {sent[link][k]}, needs {want}"
                        taken[link] = k + 1
                    if not (s == 0 and c == 0):
                        sent.setdefault(("B", s, (s - 1) % P), []).append((i, c))
                at[s] += 1
                done += 1
                progressed = True
        assert progressed, f"deadlock at P={P} M={M} V={V}: positions {at}"
    return done


def test_pipeline_schedules_are_deadlock_free_and_order_matched():
    """Every stage walks its own list; messages carry no tag, so the k-th receive on a link must be served by the
    k-th send on it, and blocking receives must never wait on each other in a cycle."""
    from siirl_b200.parallel.pipeline import schedule_interleaved
    for P in (2, 3, 4, 5):
        for V in (1, 2, 3):
            for M in (1, P - 1, P, P + 1, 2 * P, 3 * P + 2):
                if M < 1:
                    continue
                assert _simulate_pipeline(P, M, V) == 2 * P * M * V
                for s in range(P):
                    order = schedule_interleaved(s, P, M, V)
                    seen = set()
                    for op, i, c in order:                                   # a backward follows its own forward
                        if op == "F":
                            seen.add((i, c))
                        else:
                            assert (i, c) in seen


def test_context_parallel_chunk_assignments_cover_and_balance():
    """Both chunk assignments give every position to exactly one rank; under the zig-zag assignment every rank has
    the same number of (query, visible key) pairs, under the contiguous one the last rank has the most."""
    import torch

    from siirl_b200.parallel.ring_attention import chunk_positions, split_for_context_parallel
    for cp in (2, 3, 4):
        L = 12 * cp
        for zz in (False, True):
            pos = [chunk_positions([L // cp], cp, r, zz) for r in range(cp)]
            assert sorted(torch.cat(pos).tolist()) == list(range(L))
            work = [int(sum(p + 1 for p in ps.tolist())) for ps in pos]       # keys visible to each causal query
            if zz:
                assert max(work) - min(work) == 0, work
            else:
                assert work == sorted(work) and work[-1] > work[0]
            rows, p2, info = split_for_context_parallel([L, 2 * L], cp, 1, zigzag=zz)
            assert info.seqlens == [L // cp, 2 * L // cp] and rows.numel() == 3 * L // cp
            assert torch.equal(p2[: L // cp], pos[1])
