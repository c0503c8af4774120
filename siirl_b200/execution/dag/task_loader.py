"""Decomposition of a workflow DAG into independent sub-DAGs.

A sub-DAG is a chain-like slice of the workflow that one group of GPUs can execute on its own; the
scheduler then places sub-DAGs on disjoint rank sets.  Functions and their meaning follow the
reference (siirl/execution/dag/task_loader.py:24-561) but the algorithm here is a single recursive
rule: pick the first node with several children (a fork) — or, failing that, several parents (a
join) — and emit one sub-DAG per branch, each keeping the shared prefix and (for re-converging
branches) the shared suffix.  Repeat until no fork or join is left; identical structures are
emitted once (``generate_structural_signature``).
"""
from __future__ import annotations

import hashlib
from typing import Dict, List, Optional, Set

from .task_graph import TaskGraph


def generate_structural_signature(graph: TaskGraph) -> str:
    """Canonical string of node ids/types/roles and edges; independent of ``graph_id`` and insertion order."""
    if graph is None or not graph.nodes:
        return "empty"
    parts = []
    for nid in sorted(graph.nodes):
        n = graph.nodes[nid]
        deps = ",".join(sorted(d for d in n.dependencies if d in graph.nodes))
        parts.append(f"{nid}|{n.node_type.value}|{n.node_role.value}|{int(n.only_forward_compute)}|{n.agent_group}|[{deps}]")
    return ";".join(parts)


def signature_hash(graph: TaskGraph) -> str:
    return hashlib.sha1(generate_structural_signature(graph).encode()).hexdigest()[:12]


def get_all_downstream_nodes_recursive(graph: TaskGraph, start: str, visited: Optional[Set[str]] = None) -> Set[str]:
    """``start`` and every node reachable from it."""
    out: Set[str] = set() if visited is None else visited
    stack = [start]
    while stack:
        k = stack.pop()
        if k in out:
            continue
        out.add(k)
        stack.extend(n.node_id for n in graph.get_dependents(k))
    return out


def get_all_ancestors(graph: TaskGraph, node_id: str) -> Set[str]:
    """Every node ``node_id`` transitively depends on (excluding itself)."""
    out: Set[str] = set()
    stack = [d for d in graph.nodes[node_id].dependencies if d in graph.nodes]
    while stack:
        k = stack.pop()
        if k in out:
            continue
        out.add(k)
        stack.extend(d for d in graph.nodes[k].dependencies if d in graph.nodes)
    return out


def find_all_paths(graph: TaskGraph, start: str, end: str) -> List[List[str]]:
    paths: List[List[str]] = []

    def dfs(cur: str, path: List[str]):
        if cur == end:
            paths.append(path + [cur])
            return
        for nxt in sorted(n.node_id for n in graph.get_dependents(cur)):
            if nxt not in path:
                dfs(nxt, path + [cur])

    if start in graph.nodes and end in graph.nodes:
        dfs(start, [])
    return paths


def _closure_with_ancestors(graph: TaskGraph, keep: Set[str], banned: Set[str]) -> Set[str]:
    out = set(keep)
    for k in list(keep):
        out |= {a for a in get_all_ancestors(graph, k) if a not in banned}
    return out


def split_by_fan_out_to_exits(graph: TaskGraph, naming_prefix_idx: int = 0) -> List[TaskGraph]:
    """Split at a fork whose branches never meet again (each reaches its own exits)."""
    graph.build_adjacency_lists()
    ok, _ = graph.validate_graph()
    if not ok or len(graph.get_exit_nodes()) <= 1:
        return []
    for fork in sorted(graph.nodes):
        children = sorted(n.node_id for n in graph.get_dependents(fork))
        if len(children) < 2:
            continue
        branches = [get_all_downstream_nodes_recursive(graph, c) for c in children]
        disjoint = all(not (branches[i] & branches[j]) for i in range(len(branches)) for j in range(i + 1, len(branches)))
        if not disjoint:
            continue
        subs = []
        for i, br in enumerate(branches):
            others = set().union(*(b for j, b in enumerate(branches) if j != i))
            keep = _closure_with_ancestors(graph, br | {fork}, banned=others)
            subs.append(graph.subgraph(keep, f"{graph.graph_id}_fo{naming_prefix_idx}_{i}"))
        return subs
    return []


def split_by_reconverging_paths(graph: TaskGraph, naming_prefix_idx: int = 0) -> List[TaskGraph]:
    """Split parallel branches that meet again: each sub-DAG = prefix + one branch + common suffix."""
    graph.build_adjacency_lists()
    ok, _ = graph.validate_graph()
    if not ok:
        return []
    for fork in sorted(graph.nodes):
        children = sorted(n.node_id for n in graph.get_dependents(fork))
        if len(children) < 2:
            continue
        branches = [get_all_downstream_nodes_recursive(graph, c) for c in children]
        common = set.intersection(*branches)
        if not common:
            continue
        subs = []
        for i, br in enumerate(branches):
            exclusive_others = set().union(*(b for j, b in enumerate(branches) if j != i)) - br
            keep = _closure_with_ancestors(graph, br | {fork}, banned=exclusive_others)
            subs.append(graph.subgraph(keep, f"{graph.graph_id}_rc{naming_prefix_idx}_{i}"))
        return subs
    # no fork: several entries that join
    for join in sorted(graph.nodes):
        parents = sorted(d for d in graph.nodes[join].dependencies if d in graph.nodes)
        if len(parents) < 2:
            continue
        down = get_all_downstream_nodes_recursive(graph, join)
        subs = []
        anc = [get_all_ancestors(graph, p) | {p} for p in parents]
        for i, a in enumerate(anc):
            others = set().union(*(b for j, b in enumerate(anc) if j != i)) - a
            keep = (a | down) - others
            subs.append(graph.subgraph(keep, f"{graph.graph_id}_jn{naming_prefix_idx}_{i}"))
        return subs
    return []


def discover_and_split_parallel_paths(graph: TaskGraph) -> List[TaskGraph]:
    """Irreducible sub-DAGs of ``graph`` (the graph itself when it has no parallel paths)."""
    if graph is None or not graph.nodes:
        return []
    root = graph.copy()
    ok, _ = root.validate_graph()
    if not ok:
        return [root]
    final: List[TaskGraph] = []
    seen: Set[str] = set()
    queue = [root]
    it = 0
    while queue:
        cur = queue.pop(0)
        sig = generate_structural_signature(cur)
        if sig in seen:
            continue
        seen.add(sig)
        it += 1
        parts = split_by_fan_out_to_exits(cur, it) or split_by_reconverging_paths(cur, it)
        if parts:
            queue.extend(parts)
        else:
            final.append(cur)
    for i, g in enumerate(final):
        if len(final) > 1:
            g.graph_id = f"{graph.graph_id}_sub_{i}"
    return final


def count_roles(graphs: List[TaskGraph]) -> Dict[str, int]:
    out: Dict[str, int] = {}
    for g in graphs:
        for n in g.nodes.values():
            out[n.node_role.value] = out.get(n.node_role.value, 0) + 1
    return out
