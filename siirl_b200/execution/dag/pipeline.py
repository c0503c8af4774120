"""Python builder for training workflows.

``Pipeline(pipeline_id, description).add_node(node_id, func, deps=None, config=None, **kwargs)`` is
chainable, rejects duplicate ids, and ``build()`` returns a validated :class:`TaskGraph`
(contract of siirl/execution/dag/pipeline.py:37-180).  ``func`` is a callable or a string
``"pkg.mod:function"`` / ``"pkg.mod:Class.method"``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Union

from .node import Node, NodeRole, NodeType
from .task_graph import TaskGraph


@dataclass
class NodeConfig:
    agent_group: int = 0
    config: Dict[str, Any] = field(default_factory=dict)


class Pipeline:
    def __init__(self, pipeline_id: str, description: str = ""):
        self.pipeline_id = pipeline_id
        self.description = description
        self._nodes: Dict[str, Dict[str, Any]] = {}

    def add_node(self, node_id: str, func: Union[str, Callable], deps: Optional[List[str]] = None,
                 config: Optional[NodeConfig] = None, **kwargs) -> "Pipeline":
        if node_id in self._nodes:
            raise ValueError(f"Node '{node_id}' already exists in pipeline '{self.pipeline_id}'")
        self._nodes[node_id] = {"func": func, "deps": list(deps or []), "config": config or NodeConfig(),
                                "kwargs": kwargs}
        return self

    def build(self) -> TaskGraph:
        graph = TaskGraph(self.pipeline_id)
        for node_id, spec in self._nodes.items():
            kw = dict(spec["kwargs"])
            cfg: NodeConfig = spec["config"]
            graph.add_node(Node(
                node_id=node_id,
                node_type=kw.pop("node_type", NodeType.COMPUTE),
                node_role=kw.pop("node_role", NodeRole.DEFAULT),
                only_forward_compute=kw.pop("only_forward_compute", False),
                agent_group=kw.pop("agent_group", cfg.agent_group),
                dependencies=spec["deps"],
                config=dict(cfg.config),
                executable_ref=spec["func"],
                agent_options=kw.pop("agent_options", None),
                retry_limit=kw.pop("retry_limit", 0),
                filter_plugin=kw.pop("filter_plugin", None),
                agent_process=kw.pop("agent_process", None),
                user_options=kw,
            ))
        ok, msg = graph.validate_graph()
        if not ok:
            raise ValueError(f"Pipeline '{self.pipeline_id}' is invalid: {msg}")
        return graph

    def visualize(self, directory: str = ".", filename: Optional[str] = None) -> str:
        return self.build().save_dag_pic(filename or self.pipeline_id, directory)

    def __repr__(self) -> str:
        return f"Pipeline({self.pipeline_id!r}, nodes={list(self._nodes)})"
