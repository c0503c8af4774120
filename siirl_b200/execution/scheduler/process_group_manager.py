"""Derivation of communication groups from a schedule.

Given ``rank -> sub-DAG`` (output of :class:`TaskScheduler`), every MODEL_INFERENCE / MODEL_TRAIN node
is executed by the union of ranks whose sub-DAG contains it.  Each distinct rank tuple becomes one
named group ``process_group_{i}`` (numbered in order of first use, after sorting node ids so that all
processes agree).  Query methods match the reference
(siirl/execution/scheduler/process_group_manager.py:22-282).
"""
from __future__ import annotations

import collections
from typing import Any, Dict, List, Optional, Set, Tuple

from ..dag.node import NodeType
from ..dag.task_graph import TaskGraph


class ProcessGroupManager:
    def __init__(self, total_num_workers: int, ranks_taskgraph_mapping: Dict[int, Optional[TaskGraph]],
                 relevant_node_types_param: Optional[Set[NodeType]] = None):
        if total_num_workers <= 0:
            raise ValueError("Total number of workers must be positive.")
        if relevant_node_types_param is None:
            relevant = {NodeType.MODEL_INFERENCE, NodeType.MODEL_TRAIN}
        else:
            if not isinstance(relevant_node_types_param, set) or not all(
                    isinstance(t, NodeType) for t in relevant_node_types_param):
                raise ValueError("relevant_node_types_param must be a set of NodeType enums.")
            relevant = relevant_node_types_param
        self.total_num_workers = total_num_workers
        self.ranks_taskgraph_mapping = dict(ranks_taskgraph_mapping)
        self.relevant_node_types = relevant
        self.node_ranks_mapping: Dict[str, List[int]] = {}
        self.process_group_spec: Dict[str, List[int]] = {}
        self.node_process_group_mapping: Dict[str, str] = {}
        self.node_type_process_group_mapping: Dict[str, Set[str]] = collections.defaultdict(set)
        self.subgraph_node_type_pg_mapping: Dict[str, Dict[str, Set[str]]] = collections.defaultdict(
            lambda: collections.defaultdict(set))
        self._compute_group_configurations()

    def _compute_group_configurations(self) -> None:
        node_ranks: Dict[str, Set[int]] = collections.defaultdict(set)
        node_type: Dict[str, NodeType] = {}
        graph_nodes: Dict[str, Set[str]] = collections.defaultdict(set)
        for rank, graph in self.ranks_taskgraph_mapping.items():
            if graph is None:
                continue
            if not (0 <= rank < self.total_num_workers):
                raise ValueError(f"rank {rank} outside [0, {self.total_num_workers})")
            for nid, node in graph.nodes.items():
                if node.node_type in self.relevant_node_types:
                    node_ranks[nid].add(rank)
                    node_type[nid] = node.node_type
                    graph_nodes[graph.graph_id].add(nid)
        rank_tuple_to_name: Dict[Tuple[int, ...], str] = {}
        for nid in sorted(node_ranks):
            ranks = tuple(sorted(node_ranks[nid]))
            self.node_ranks_mapping[nid] = list(ranks)
            if ranks not in rank_tuple_to_name:
                name = f"process_group_{len(rank_tuple_to_name) + 1}"
                rank_tuple_to_name[ranks] = name
                self.process_group_spec[name] = list(ranks)
            name = rank_tuple_to_name[ranks]
            self.node_process_group_mapping[nid] = name
            self.node_type_process_group_mapping[node_type[nid].value].add(name)
        for gid, nids in graph_nodes.items():
            for nid in nids:
                self.subgraph_node_type_pg_mapping[gid][node_type[nid].value].add(
                    self.node_process_group_mapping[nid])

    # ---- queries -----------------------------------------------------------------------------
    def get_group_spec(self, group_name: str) -> Optional[Dict[str, Any]]:
        ranks = self.process_group_spec.get(group_name)
        return {"ranks": ranks} if ranks is not None else None

    def get_all_specs(self) -> Dict[str, Dict[str, Any]]:
        return {name: {"ranks": ranks} for name, ranks in self.process_group_spec.items()}

    def get_node_assignment(self, node_id: str) -> Optional[Dict[str, Any]]:
        if node_id not in self.node_process_group_mapping:
            return None
        return {"ranks": self.node_ranks_mapping[node_id],
                "process_group_name": self.node_process_group_mapping[node_id]}

    def get_process_groups_for_node_type(self, node_type_value: str) -> Set[str]:
        if any(t.value == node_type_value for t in self.relevant_node_types):
            return set(self.node_type_process_group_mapping.get(node_type_value, set()))
        return set()

    def get_process_group_for_node_type_in_subgraph(self, graph_id: str, node_type_value: str) -> Set[str]:
        if any(t.value == node_type_value for t in self.relevant_node_types):
            return set(self.subgraph_node_type_pg_mapping.get(graph_id, {}).get(node_type_value, set()))
        return set()

    def describe(self) -> str:
        lines = [f"process groups ({len(self.process_group_spec)}):"]
        for name, ranks in self.process_group_spec.items():
            nodes = [n for n, g in self.node_process_group_mapping.items() if g == name]
            lines.append(f"  {name}: ranks={ranks} nodes={nodes}")
        return "\n".join(lines)


def log_process_group_manager_details(pgm: ProcessGroupManager, log=print) -> None:
    log(pgm.describe())
