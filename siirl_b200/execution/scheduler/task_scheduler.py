"""Placement of sub-DAGs on GPU ranks.

Contract of the reference scheduler (siirl/execution/scheduler/task_scheduler.py:24-566): the input
graphs are split into irreducible sub-DAGs, each sub-DAG receives a share of the workers
(``even`` or ``param_aware`` by estimated model size, at least one each), and workers are picked one
slot at a time by the score ``(cohesion with peers already placed, -load of the physical node,
-rank)``.  The schedule is a pure function of its inputs, so every per-GPU process computes the same
assignment locally; there is no central scheduler process.
"""
from __future__ import annotations

import logging
import re
from typing import Callable, Dict, List, Optional, Tuple

from ..dag.node import NodeType
from ..dag.task_graph import TaskGraph
from ..dag.task_loader import discover_and_split_parallel_paths, generate_structural_signature

logger = logging.getLogger(__name__)


def _parse_model_params_string(value) -> float:
    """``"7B"`` -> 7e9, ``"500M"`` -> 5e8, ``"100K"`` -> 1e5, numbers pass through; garbage -> 0."""
    if isinstance(value, bool):
        return 0.0
    if isinstance(value, (int, float)):
        return float(value)
    if isinstance(value, str):
        m = re.match(r"^\s*(\d+(?:\.\d+)?)\s*([KMBT]?)\s*$", value.upper())
        if not m:
            return 0.0
        scale = {"": 1.0, "K": 1e3, "M": 1e6, "B": 1e9, "T": 1e12}[m.group(2)]
        return float(m.group(1)) * scale
    return 0.0


def estimate_graph_model_params(graph: TaskGraph) -> float:
    """Sum of ``config["model_params"]`` over model nodes; node count when the graph has no model node;
    0 when model nodes carry no positive size."""
    if graph is None or not graph.nodes:
        return 0.0
    model_nodes = [n for n in graph.nodes.values() if n.node_type in (NodeType.MODEL_TRAIN, NodeType.MODEL_INFERENCE)]
    if not model_nodes:
        return float(len(graph.nodes))
    return sum(max(_parse_model_params_string(n.config.get("model_params", 0.0)), 0.0) for n in model_nodes)


class TaskScheduler:
    def __init__(self, num_physical_nodes: int, gpus_per_node: int):
        if num_physical_nodes <= 0 or gpus_per_node <= 0:
            raise ValueError("num_physical_nodes and gpus_per_node must be positive")
        self.num_physical_nodes = num_physical_nodes
        self.gpus_per_node = gpus_per_node
        self.num_workers = num_physical_nodes * gpus_per_node
        self._reset_scheduler_state()

    def _reset_scheduler_state(self) -> None:
        self.worker_to_graph_assignment: Dict[int, Optional[TaskGraph]] = {r: None for r in range(self.num_workers)}
        self.node_active_worker_count: List[int] = [0] * self.num_physical_nodes
        self.node_free_gpus: List[List[int]] = [
            list(range(n * self.gpus_per_node, (n + 1) * self.gpus_per_node)) for n in range(self.num_physical_nodes)]
        self.subgraph_to_ranks: Dict[str, List[int]] = {}

    def _apportion_workers_to_tasks(self, tasks: List[Tuple[TaskGraph, float]], total_workers: int,
                                    strategy: str) -> Dict[str, int]:
        """Number of workers per sub-DAG: every task gets one, the remainder is spread evenly
        (``even``) or proportionally to size by largest remainder (``param_aware``)."""
        n = len(tasks)
        if n == 0:
            return {}
        if total_workers < n:
            raise ValueError(f"{n} sub-graphs need at least {n} workers, only {total_workers} available")
        counts = {g.graph_id: 1 for g, _ in tasks}
        rest = total_workers - n
        total_size = sum(s for _, s in tasks)
        if strategy == "param_aware" and total_size > 0:
            quotas = [(g.graph_id, rest * s / total_size) for g, s in tasks]
            floors = {gid: int(q) for gid, q in quotas}
            for gid, f in floors.items():
                counts[gid] += f
            left = rest - sum(floors.values())
            by_frac = sorted(quotas, key=lambda x: (x[1] - int(x[1]), x[1]), reverse=True)
            for gid, _ in by_frac[:left]:
                counts[gid] += 1
        else:
            if strategy not in ("even", "param_aware"):
                raise ValueError(f"unknown apportion strategy '{strategy}'")
            base, extra = divmod(rest, n)
            for i, (g, _) in enumerate(tasks):
                counts[g.graph_id] += base + (1 if i < extra else 0)
        return counts

    def schedule_and_assign_tasks(self, original_task_graphs: List[TaskGraph],
                                  size_estimator: Callable[[TaskGraph], float] = estimate_graph_model_params,
                                  apportion_strategy: str = "param_aware", consider_node_cohesion: bool = True,
                                  consider_node_load: bool = True,
                                  consider_rank_preference: bool = True) -> Dict[int, Optional[TaskGraph]]:
        self._reset_scheduler_state()
        subgraphs: List[TaskGraph] = []
        for g in original_task_graphs or []:
            if g is None or not g.nodes:
                continue
            subgraphs.extend(discover_and_split_parallel_paths(g))
        if not subgraphs:
            return self.worker_to_graph_assignment
        sized = sorted(((g, float(size_estimator(g))) for g in subgraphs), key=lambda x: x[1], reverse=True)
        if len(sized) > self.num_workers:
            raise ValueError(f"Cannot assign all tasks. Number of schedulable subgraphes ({len(sized)}) exceeds "
                             f"the total number of available workers ({self.num_workers}).")
        counts = self._apportion_workers_to_tasks(sized, self.num_workers, apportion_strategy)
        order = sorted(sized, key=lambda x: (counts[x[0].graph_id], x[1]), reverse=True)
        for graph, _ in order:
            placed: List[int] = []
            for _slot in range(counts[graph.graph_id]):
                peers_nodes = {r // self.gpus_per_node for r in placed}
                best, best_score = -1, (float("-inf"),) * 3
                for pn in range(self.num_physical_nodes):
                    if not self.node_free_gpus[pn]:
                        continue
                    cand = self.node_free_gpus[pn][0]
                    cohesion = 1.0 if consider_node_cohesion and (not placed or pn in peers_nodes) else 0.0
                    load = -float(self.node_active_worker_count[pn]) if consider_node_load else 0.0
                    pref = -float(cand) if consider_rank_preference else 0.0
                    score = (cohesion, load, pref)
                    if score > best_score:
                        best, best_score = cand, score
                if best < 0:
                    raise RuntimeError(f"no free worker left while placing '{graph.graph_id}'")
                pn = best // self.gpus_per_node
                self.worker_to_graph_assignment[best] = graph
                self.node_active_worker_count[pn] += 1
                self.node_free_gpus[pn].remove(best)
                placed.append(best)
            self.subgraph_to_ranks[graph.graph_id] = sorted(placed)
        return self.worker_to_graph_assignment

    def get_unique_assigned_task_graphs(self) -> Dict[str, TaskGraph]:
        out: Dict[str, TaskGraph] = {}
        for g in self.worker_to_graph_assignment.values():
            if g is not None and g.graph_id not in out:
                out[g.graph_id] = g
        return out

    def get_ranks_for_graph(self, graph_id: str) -> List[int]:
        return list(self.subgraph_to_ranks.get(graph_id, []))


def _format_ranks_for_logging(ranks: Optional[List[int]], detailed: bool, threshold: int = 10) -> str:
    if not ranks:
        return "[]"
    ranks = sorted(ranks)
    if detailed or len(ranks) <= threshold:
        return str(ranks)
    return f"[{ranks[0]}..{ranks[-1]}] ({len(ranks)} ranks)"


def log_schedule_assignments(assignment: Dict[int, Optional[TaskGraph]], num_workers: int,
                             detailed_rank_printing: bool = False, log: Callable[[str], None] = logger.info) -> str:
    """Human-readable schedule summary (one block per sub-DAG); also returned as a string."""
    by_graph: Dict[str, List[int]] = {}
    graphs: Dict[str, TaskGraph] = {}
    idle = []
    for r in range(num_workers):
        g = assignment.get(r)
        if g is None:
            idle.append(r)
        else:
            by_graph.setdefault(g.graph_id, []).append(r)
            graphs[g.graph_id] = g
    lines = [f"schedule: {num_workers} workers, {len(by_graph)} sub-graph(s), {len(idle)} idle"]
    for gid, ranks in by_graph.items():
        lines.append(f"  {gid}: ranks {_format_ranks_for_logging(ranks, detailed_rank_printing)} "
                     f"nodes={list(graphs[gid].nodes)} sig={hash(generate_structural_signature(graphs[gid])) & 0xffff:04x}")
    if idle:
        lines.append(f"  idle: {_format_ranks_for_logging(idle, detailed_rank_printing)}")
    text = "\n".join(lines)
    log(text)
    return text
