"""Attach the typed configuration to every node of a task graph.

Role -> config group (reference: siirl/execution/scheduler/graph_updater.py:57-128): ACTOR,
ROLLOUT, REFERENCE, ADVANTAGE-with-model nodes use ``actor_rollout_ref``; CRITIC uses ``critic``;
REWARD uses ``reward_model``.  Per-node overrides found in ``node.config`` (nested mappings or dotted
keys) are merged over a deep copy, and the result is stored as
``node.config = {"intern_config": <dataclass>, "_node_id_": id, ...original keys}``.
"""
from __future__ import annotations

from typing import Any, Dict

from ...params.parser import merge_node_overrides
from ...params.schema import SiiRLArguments
from ..dag.node import NodeRole, NodeType
from ..dag.task_graph import TaskGraph

_RESERVED = {"_node_id_", "intern_config", "model_params"}


def config_group_for_role(cfg: SiiRLArguments, role: NodeRole):
    if role == NodeRole.CRITIC:
        return cfg.critic
    if role == NodeRole.REWARD:
        return cfg.reward_model
    return cfg.actor_rollout_ref


def update_task_graph_node_configs(graph: TaskGraph, cfg: SiiRLArguments) -> TaskGraph:
    for node in graph.nodes.values():
        base = config_group_for_role(cfg, node.node_role)
        overrides: Dict[str, Any] = {k: v for k, v in node.config.items() if k not in _RESERVED}
        known = {}
        extra = {}
        for k, v in overrides.items():
            head = k.split(".")[0]
            (known if hasattr(base, head) else extra)[k] = v
        intern = merge_node_overrides(base, known) if node.node_type in (
            NodeType.MODEL_TRAIN, NodeType.MODEL_INFERENCE, NodeType.COMPUTE, NodeType.CUSTOM) else base
        new_cfg = dict(node.config)
        new_cfg["intern_config"] = intern
        new_cfg["_node_id_"] = node.node_id
        new_cfg.update(extra)
        if "model_params" not in new_cfg and node.node_type in (NodeType.MODEL_TRAIN, NodeType.MODEL_INFERENCE):
            new_cfg["model_params"] = 0.0
        node.config = new_cfg
    return graph
