"""Declarative DAG files (YAML or JSON).

File layout (same as the reference's legacy loader, siirl/execution/dag/config_loader.py:25-246):

    dag_id: my_flow
    description: optional text
    global_config: {any: mapping}
    nodes:
      - node_id: rollout
        node_type: MODEL_INFERENCE
        node_role: ROLLOUT
        dependencies: []
        executable_ref: "pkg.mod:Class.method"
        config: {lr: !Ref global_config.any}
        agent_group: 0
        agent_options: {share_instance: 0, train_cycle: 2, env_path: [...], process_path: ...}

``!Ref global_config.a.b`` is replaced by the value found in ``global_config``.
"""
from __future__ import annotations

import json
from typing import Any, Dict

import yaml

from .node import Node, NodeRole, NodeType
from .task_graph import TaskGraph


class Ref:
    def __init__(self, path: str):
        self.path = path

    def __repr__(self) -> str:
        return f"!Ref {self.path}"


class _RefLoader(yaml.SafeLoader):
    pass


_RefLoader.add_constructor("!Ref", lambda loader, node: Ref(loader.construct_scalar(node)))


def resolve_refs(item: Any, global_config: Dict[str, Any]) -> Any:
    if isinstance(item, dict):
        return {k: resolve_refs(v, global_config) for k, v in item.items()}
    if isinstance(item, list):
        return [resolve_refs(v, global_config) for v in item]
    if isinstance(item, Ref):
        parts = item.path.split(".")
        if parts[0] != "global_config":
            raise ValueError(f"unsupported reference root '{parts[0]}' in '{item.path}' (only global_config)")
        cur: Any = global_config
        for p in parts[1:]:
            if not isinstance(cur, dict) or p not in cur or cur[p] is None:
                raise ValueError(f"Unresolved reference '{item.path}'.")
            cur = cur[p]
        return cur
    return item


class DAGConfigLoader:
    @staticmethod
    def from_dict(raw: Dict[str, Any], origin: str = "<dict>") -> TaskGraph:
        if not raw or not isinstance(raw, dict):
            raise ValueError(f"'{origin}' is empty or not a mapping")
        dag_id = raw.get("dag_id")
        if not dag_id:
            raise ValueError(f"'dag_id' is missing in '{origin}'")
        if "nodes" not in raw:
            raise ValueError(f"'nodes' list is missing in '{origin}'")
        if not isinstance(raw["nodes"], list):
            raise ValueError(f"'nodes' in '{origin}' must be a list")
        global_config = raw.get("global_config", {}) or {}
        graph = TaskGraph(dag_id)
        graph.description = raw.get("description")
        seen = set()
        for i, nc in enumerate(raw["nodes"]):
            if not isinstance(nc, dict):
                continue
            nid = nc.get("node_id")
            if not nid:
                raise ValueError(f"node #{i + 1} in '{origin}' has no 'node_id'")
            if nid in seen:
                raise ValueError(f"Duplicate node ID '{nid}' in '{origin}'")
            seen.add(nid)
            if "node_type" not in nc:
                raise ValueError(f"Node '{nid}' is missing 'node_type'")
            try:
                ntype = NodeType[str(nc["node_type"]).upper()]
            except KeyError:
                raise ValueError(f"node '{nid}': invalid node_type '{nc['node_type']}'") from None
            try:
                nrole = NodeRole[str(nc.get("node_role", "DEFAULT")).upper()]
            except KeyError:
                raise ValueError(f"node '{nid}': invalid node_role '{nc.get('node_role')}'") from None
            deps = nc.get("dependencies", [])
            if not isinstance(deps, list):
                raise ValueError(f"node '{nid}': 'dependencies' must be a list")
            cfg = resolve_refs(nc.get("config", {}) or {}, global_config)
            cfg["_node_id_"] = nid
            graph.add_node(Node(node_id=nid, node_type=ntype, node_role=nrole,
                                only_forward_compute=nc.get("only_forward_compute", False),
                                agent_group=nc.get("agent_group", 0), dependencies=deps, config=cfg,
                                executable_ref=nc.get("executable_ref"), agent_options=nc.get("agent_options"),
                                filter_plugin=nc.get("filter_plugin"), retry_limit=nc.get("retry_limit", 0)))
        ok, msg = graph.validate_graph()
        if not ok:
            raise ValueError(f"The graph loaded from '{origin}' is invalid: {msg}")
        return graph

    @staticmethod
    def load_from_file(file_path: str, file_type: str = "yaml") -> TaskGraph:
        with open(file_path, "r", encoding="utf-8") as f:
            if file_type in ("yaml", "yml"):
                raw = yaml.load(f, Loader=_RefLoader)
            elif file_type == "json":
                raw = json.load(f)
            else:
                raise ValueError(f"Unsupported file type: '{file_type}'. Please use yaml, yml, or json.")
        return DAGConfigLoader.from_dict(raw, file_path)

    @staticmethod
    def load_from_string(text: str, file_type: str = "yaml") -> TaskGraph:
        raw = yaml.load(text, Loader=_RefLoader) if file_type in ("yaml", "yml") else json.loads(text)
        return DAGConfigLoader.from_dict(raw, "<string>")
