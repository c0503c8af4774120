"""TaskGraph: container of :class:`Node` objects with validation, topological order and export.

Mirrors the reference container's public methods (siirl/execution/dag/task_graph.py:23-462):
``add_node(s)``, ``get_node``, ``get_dependencies/get_dependents/get_downstream_nodes``,
``get_entry_nodes/get_exit_nodes``, ``validate_graph`` (missing dependencies, cycles),
``get_topological_sort`` (Kahn), ``get_nodes_by_type/role``, ``load_from_config``, ``save_dag_pic``.
"""
from __future__ import annotations

from collections import deque
from typing import Any, Dict, Iterable, List, Optional, Tuple

from .node import Node, NodeRole, NodeType


class TaskGraph:
    def __init__(self, graph_id: str):
        if not graph_id:
            raise ValueError("graph_id must be non-empty")
        self.graph_id = graph_id
        self.nodes: Dict[str, Node] = {}
        self._adj: Dict[str, List[str]] = {}
        self._rev: Dict[str, List[str]] = {}
        self._dirty = True

    # ---- construction ------------------------------------------------------------------------
    def add_node(self, node: Node) -> None:
        if not isinstance(node, Node):
            raise TypeError("add_node expects a Node")
        if node.node_id in self.nodes:
            raise ValueError(f"node '{node.node_id}' already exists in graph '{self.graph_id}'")
        self.nodes[node.node_id] = node
        self._dirty = True

    def add_nodes(self, nodes: Iterable[Node]) -> None:
        for n in nodes:
            self.add_node(n)

    def remove_node(self, node_id: str) -> None:
        self.nodes.pop(node_id)
        for n in self.nodes.values():
            n.remove_dependency(node_id)
        self._dirty = True

    def get_node(self, node_id: str) -> Optional[Node]:
        return self.nodes.get(node_id)

    def build_adjacency_lists(self) -> None:
        self._adj = {k: [] for k in self.nodes}
        self._rev = {k: [] for k in self.nodes}
        for nid, node in self.nodes.items():
            for dep in node.dependencies:
                if dep in self.nodes:
                    self._adj[dep].append(nid)
                    self._rev[nid].append(dep)
        self._dirty = False

    def _ensure(self) -> None:
        if self._dirty:
            self.build_adjacency_lists()

    # ---- queries -----------------------------------------------------------------------------
    def get_dependencies(self, node_id: str) -> List[Node]:
        self._ensure()
        return [self.nodes[d] for d in self._rev.get(node_id, [])]

    def get_dependents(self, node_id: str) -> List[Node]:
        self._ensure()
        return [self.nodes[d] for d in self._adj.get(node_id, [])]

    get_downstream_nodes = get_dependents

    def get_entry_nodes(self) -> List[Node]:
        return [n for n in self.nodes.values() if not n.dependencies]

    def get_exit_nodes(self) -> List[Node]:
        self._ensure()
        return [self.nodes[k] for k, v in self._adj.items() if not v]

    def get_nodes_by_type(self, node_type: NodeType) -> List[Node]:
        return [n for n in self.nodes.values() if n.node_type == node_type]

    def get_nodes_by_role(self, node_role: NodeRole) -> List[Node]:
        return [n for n in self.nodes.values() if n.node_role == node_role]

    def validate_graph(self) -> Tuple[bool, Optional[str]]:
        for nid, node in self.nodes.items():
            for dep in node.dependencies:
                if dep not in self.nodes:
                    return False, f"node '{nid}' depends on unknown node '{dep}'"
        order = self._kahn()
        if order is None:
            return False, f"graph '{self.graph_id}' contains a cycle"
        return True, None

    def _kahn(self) -> Optional[List[str]]:
        self.build_adjacency_lists()
        indeg = {k: len(v) for k, v in self._rev.items()}
        q = deque(sorted(k for k, d in indeg.items() if d == 0))
        out: List[str] = []
        while q:
            k = q.popleft()
            out.append(k)
            for nxt in self._adj[k]:
                indeg[nxt] -= 1
                if indeg[nxt] == 0:
                    q.append(nxt)
        return out if len(out) == len(self.nodes) else None

    def get_topological_sort(self) -> List[str]:
        ok, msg = self.validate_graph()
        if not ok:
            raise ValueError(msg)
        return self._kahn() or []

    def reset_status(self) -> None:
        for n in self.nodes.values():
            n.reset()

    def copy(self, graph_id: Optional[str] = None) -> "TaskGraph":
        g = TaskGraph(graph_id or self.graph_id)
        for n in self.nodes.values():
            g.add_node(n.copy())
        return g

    def subgraph(self, node_ids: Iterable[str], graph_id: str) -> "TaskGraph":
        keep = set(node_ids)
        g = TaskGraph(graph_id)
        for nid in self.nodes:
            if nid in keep:
                n = self.nodes[nid].copy()
                n.dependencies = [d for d in n.dependencies if d in keep]
                g.add_node(n)
        return g

    # ---- (de)serialisation -------------------------------------------------------------------
    @classmethod
    def load_from_config(cls, graph_id: str, nodes_config: List[Dict[str, Any]]) -> "TaskGraph":
        g = cls(graph_id)
        for nc in nodes_config:
            nc = dict(nc)
            if "node_id" not in nc:
                raise ValueError(f"node config without node_id: {nc}")
            g.add_node(Node(
                node_id=nc["node_id"],
                node_type=nc.get("node_type", NodeType.COMPUTE),
                node_role=nc.get("node_role", NodeRole.DEFAULT),
                only_forward_compute=nc.get("only_forward_compute", False),
                agent_group=nc.get("agent_group", 0),
                dependencies=nc.get("dependencies", []),
                config=nc.get("config", {}),
                executable_ref=nc.get("executable_ref"),
                agent_options=nc.get("agent_options"),
                retry_limit=nc.get("retry_limit", 0),
                user_options=nc.get("user_options"),
            ))
        ok, msg = g.validate_graph()
        if not ok:
            raise ValueError(f"invalid graph '{graph_id}': {msg}")
        return g

    def to_config(self) -> List[Dict[str, Any]]:
        out = []
        for n in self.nodes.values():
            out.append({
                "node_id": n.node_id, "node_type": n.node_type.value, "node_role": n.node_role.value,
                "only_forward_compute": n.only_forward_compute, "agent_group": n.agent_group,
                "dependencies": list(n.dependencies),
                "executable_ref": n.executable_ref if isinstance(n.executable_ref, str) else None,
            })
        return out

    def to_dot(self) -> str:
        """Graphviz source of the graph (no dependency on the graphviz package)."""
        shape = {NodeType.MODEL_TRAIN: "box", NodeType.MODEL_INFERENCE: "ellipse", NodeType.COMPUTE: "hexagon"}
        lines = [f'digraph "{self.graph_id}" {{', "  rankdir=LR;"]
        for n in self.nodes.values():
            label = f"{n.node_id}\\n{n.node_type.value}/{n.node_role.value}"
            lines.append(f'  "{n.node_id}" [label="{label}", shape={shape.get(n.node_type, "oval")}];')
        for n in self.nodes.values():
            for d in n.dependencies:
                lines.append(f'  "{d}" -> "{n.node_id}";')
        lines.append("}")
        return "\n".join(lines)

    def save_dag_pic(self, filename: str = "dag", directory: str = ".", fmt: str = "png") -> str:
        """Render with the ``graphviz`` package when present, else write the .dot source."""
        import os
        os.makedirs(directory, exist_ok=True)
        try:
            import graphviz  # type: ignore
            dot = graphviz.Digraph(self.graph_id, format=fmt)
            for n in self.nodes.values():
                dot.node(n.node_id, f"{n.node_id}\n{n.node_type.value}/{n.node_role.value}")
            for n in self.nodes.values():
                for d in n.dependencies:
                    dot.edge(d, n.node_id)
            return dot.render(filename=filename, directory=directory, cleanup=True)
        except Exception:  # noqa: BLE001
            path = os.path.join(directory, filename + ".dot")
            with open(path, "w") as f:
                f.write(self.to_dot())
            return path

    def __len__(self) -> int:
        return len(self.nodes)

    def __repr__(self) -> str:
        return f"TaskGraph({self.graph_id!r}, nodes={list(self.nodes)})"
