"""Data coordinator: buffer semantics of the reference tests (tests/data_buffer/test_data_buffer.py,
tests/dag_worker/test_dapo_*.py) plus length balancing, sample conversion and filters."""
import numpy as np
import pytest
import torch

from siirl_b200.data_coordinator import (Batch, DataCoordinator, Dict2Samples, SampleInfo, Samples2Dict, filter_batch,
                                         preprocess_dataloader)
from siirl_b200.params import parse_config
from siirl_b200.user_interface.filter_interface.dapo import dynamic_sampling
from siirl_b200.utils.model_utils.seqlen_balancing import (_kk_python, get_seqlen_balanced_partitions, karmarkar_karp,
                                                           rearrange_micro_batches)


def _info(tokens, key="k", node=None):
    return SampleInfo(sum_tokens=tokens, node_id=node, dict_info={"key": key})


def test_put_get_fifo_and_insufficient():
    dc = DataCoordinator()
    for i in range(5):
        dc.put(_info(10 + i), f"s{i}")
    assert dc.get_valid_size() == 5
    assert dc.get_batch(8, 0) == []
    assert dc.get_batch(3, 0) == ["s0", "s1", "s2"]
    assert dc.get_valid_size() == 2
    with pytest.raises(ValueError):
        dc.put_batch([_info(1)], [])


def test_filter_plugin_and_node_affinity():
    dc = DataCoordinator()
    dc.put_batch([_info(5, "a"), _info(6, "b"), _info(7, "a")], ["x", "y", "z"], caller_node_id="n1")
    got = dc.get_batch(2, 0, filter_plugin=lambda i: i.dict_info["key"] == "a")
    assert got == ["x", "z"] and dc.get_valid_size() == 1
    assert dc.get_all_by_filter(lambda i: i.node_id == "n1") == ["y"]


def test_balanced_partitions_cached_per_dp_rank():
    dc = DataCoordinator()
    toks = [100, 4000, 200, 3000, 1500, 1600, 50, 2500]
    dc.put_batch([_info(t) for t in toks], list(range(8)))
    p0 = dc.get_batch(4, 0, balance_partitions=2)
    p1 = dc.get_batch(4, 1, balance_partitions=2)
    assert sorted(p0 + p1) == list(range(8)) and len(p0) == len(p1) == 4
    s0, s1 = sum(toks[i] for i in p0), sum(toks[i] for i in p1)
    assert abs(s0 - s1) < 0.2 * (s0 + s1)
    # short samples at both ends, long in the middle
    assert toks[p0[0]] <= max(toks[i] for i in p0[1:-1]) and toks[p0[-1]] <= max(toks[i] for i in p0[1:-1])
    dc.reset_cache()
    assert dc.get_valid_size() == 0


def test_peek_source_dp_size():
    dc = DataCoordinator()
    info = _info(3)
    info.dict_info["source_dp_size"] = 4
    dc.put(info, "r")
    assert dc.peek_source_dp_size(lambda i: True) == 4
    assert dc.peek_source_dp_size(lambda i: False) is None


def test_kk_native_matches_python_and_is_balanced():
    rng = np.random.RandomState(0)
    for n, k in [(16, 4), (64, 8), (9, 3)]:
        xs = rng.randint(10, 5000, size=n).tolist()
        for eq in (True, False):
            a, b = karmarkar_karp(xs, k, eq), _kk_python(xs, k, eq)
            assert sorted(sum(xs[i] for i in p) for p in a) == sorted(sum(xs[i] for i in p) for p in b)
        parts = get_seqlen_balanced_partitions(xs, k, equal_size=True)
        sums = [sum(xs[i] for i in p) for p in parts]
        assert max(sums) - min(sums) <= max(xs)
        assert all(len(p) == n // k for p in parts)


def test_dynamic_micro_batches_respect_budget():
    lens = [100, 900, 500, 300, 1200, 50, 700]
    parts = rearrange_micro_batches(lens, 1500)
    assert sorted(i for p in parts for i in p) == list(range(7))
    assert all(sum(lens[i] for i in p) <= 1500 for p in parts)
    with pytest.raises(AssertionError):
        rearrange_micro_batches([2000], 1500)


def test_preprocess_repeat_and_uid_and_roundtrip():
    b = Batch({"input_ids": torch.arange(6).reshape(3, 2), "attention_mask": torch.ones(3, 2, dtype=torch.long)},
              {"raw": ["a", "b", "c"]}, {"step": 1})
    r = preprocess_dataloader(b, 2)
    assert r.batch_size == 6 and r["uid"].tolist() == [0, 0, 1, 1, 2, 2] and list(r["raw"]) == list("aabbcc")
    infos, samples = Dict2Samples(r, key="next")
    assert len(samples) == 6 and infos[0].dict_info["key"] == "next" and infos[0].sum_tokens == 2
    back = Samples2Dict(samples)
    assert torch.equal(back["input_ids"], r["input_ids"]) and list(back["raw"]) == list(r["raw"])
    assert back.meta["global_token_num"] == [2] * 6 and back.meta["step"] == 1


def test_filter_batch_mask_indices_and_non_tensors():
    b = Batch({"x": torch.arange(4)}, {"s": ["a", "b", "c", "d"]})
    assert filter_batch(b, torch.tensor([True, False, True, False]))["x"].tolist() == [0, 2]
    k = filter_batch(b, [3, 1])
    assert k["x"].tolist() == [3, 1] and list(k["s"]) == ["d", "b"]
    assert filter_batch(b, np.array([False, False, False, False])).batch_size == 0


def test_dapo_dynamic_sampling_keeps_only_mixed_groups():
    cfg = parse_config(["algorithm.filter_groups.enable=True", "algorithm.filter_groups.metric=seq_reward"])
    b = Batch({"uid": torch.tensor([0, 0, 1, 1, 2, 3, 3]), "seq_reward": torch.tensor([1., 0., 1., 1., 0., 0., 0.]),
               "x": torch.arange(7)})
    out = dynamic_sampling(cfg, b)
    assert out.batch["x"].tolist() == [0, 1, 4]           # mixed group 0, singleton group 2
    assert out.metrics["dapo_sampling/initial_trajectories"] == 7 and out.metrics["dapo_sampling/final_trajectories"] == 3
    cfg.algorithm.filter_groups.enable = False
    assert dynamic_sampling(cfg, b).batch.batch_size == 7


def test_batch_container_ops():
    b = Batch({"a": torch.arange(6).reshape(3, 2)}, {"n": [1, 2, 3]}, {"m": 5})
    assert "a" in b and "n" in b and "m" in b and b["m"] == 5
    b["new"] = torch.ones(3)
    b["scalar"] = 7
    assert b.meta["scalar"] == 7 and "new" in b.tensors
    c = Batch.concat([b, b])
    assert c.batch_size == 6 and c.chunk(4)[0].batch_size == 2 and len(c.split(4)) == 2
    with pytest.raises(ValueError):
        Batch({"a": torch.zeros(2)}, {"n": [1, 2, 3]})


def test_balanced_plan_keeps_the_responses_of_a_prompt_together():
    """Group-relative advantages are computed per rank: redistribution moves whole groups when it can."""
    from siirl_b200.data_coordinator.data_buffer import balanced_plan
    import random
    rnd = random.Random(0)
    n_groups, size, parts = 12, 4, 3
    keys = [("p", g) for g in range(n_groups) for _ in range(size)]
    order = list(range(len(keys)))
    rnd.shuffle(order)                                            # producers interleave in the global FIFO order
    keys = [keys[i] for i in order]
    tokens = [rnd.randint(10, 400) for _ in keys]
    plan = balanced_plan(tokens, keys, parts)
    assert sorted(i for p in plan for i in p) == list(range(len(keys))) and {len(p) for p in plan} == {16}
    for p in plan:
        per_key = {}
        for i in p:
            per_key[keys[i]] = per_key.get(keys[i], 0) + 1
        assert set(per_key.values()) == {size}                    # every group is whole on its partition
    loads = [sum(tokens[i] for i in p) for p in plan]
    assert max(loads) - min(loads) < 0.25 * max(loads)
    # ragged groups (or no uid): falls back to balancing single samples
    ragged = balanced_plan(tokens[:-2], keys[:-2], 2)
    assert sorted(i for p in ragged for i in p) == list(range(len(keys) - 2))
    nokeys = balanced_plan(tokens, [None] * len(tokens), parts)
    assert {len(p) for p in nokeys} == {16}


def test_group_ids_do_not_collide_across_ranks_and_draws():
    from siirl_b200.data_coordinator.sample import preprocess_dataloader
    ids = set()
    for draw in range(2):
        for rank in range(3):
            b = Batch({"input_ids": torch.zeros(4, 5, dtype=torch.long)})
            out = preprocess_dataloader(b, 2, uid_offset=(draw * 3 + rank) * 4)
            u = out["uid"].tolist()
            assert u[0] == u[1] and u[2] == u[3] and len(set(u)) == 4
            assert not (ids & set(u))
            ids |= set(u)
    assert len(ids) == 24
