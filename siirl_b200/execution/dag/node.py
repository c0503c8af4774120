"""DAG node model: what one stage of an RL step is, what it depends on and how it is executed.

Public surface follows the reference (siirl/execution/dag/node.py:44-499): ``NodeType``,
``NodeRole``, ``NodeStatus``, ``AgentProcess`` hooks for multi-agent flows and ``Node`` with an
``executable_ref`` given either as a callable or as ``"pkg.mod:func"`` / ``"pkg.mod:Class.method"``.
Unbound ``Class.method`` references are bound at run time to the worker instance passed as
``_dag_worker_instance`` so the same graph description works in every per-GPU process.
"""
from __future__ import annotations

import asyncio
import enum
import importlib
import inspect
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Union


class NodeType(str, enum.Enum):
    COMPUTE = "COMPUTE"
    DATA_LOAD = "DATA_LOAD"
    ENV_INTERACT = "ENV_INTERACT"
    MODEL_INFERENCE = "MODEL_INFERENCE"
    MODEL_TRAIN = "MODEL_TRAIN"
    PUT_TO_BUFFER = "PUT_TO_BUFFER"
    GET_FROM_BUFFER = "GET_FROM_BUFFER"
    BARRIER_SYNC = "BARRIER_SYNC"
    CUSTOM = "CUSTOM"


class NodeRole(str, enum.Enum):
    DEFAULT = "DEFAULT"
    ACTOR = "ACTOR"
    ADVANTAGE = "ADVANTAGE"
    CRITIC = "CRITIC"
    ROLLOUT = "ROLLOUT"
    REFERENCE = "REFERENCE"
    REWARD = "REWARD"
    DYNAMIC_SAMPLING = "DYNAMIC_SAMPLING"


class NodeStatus(str, enum.Enum):
    PENDING = "PENDING"
    READY = "READY"
    RUNNING = "RUNNING"
    COMPLETED = "COMPLETED"
    FAILED = "FAILED"
    SKIPPED = "SKIPPED"


def _coerce_enum(enum_cls, value):
    if isinstance(value, enum_cls):
        return value
    if isinstance(value, str):
        key = value.split(".")[-1].upper()
        return enum_cls[key]
    raise TypeError(f"cannot interpret {value!r} as {enum_cls.__name__}")


def resolve_callable(ref: Union[str, Callable, None]) -> Optional[Callable]:
    """``"pkg.mod:attr.sub"`` or ``"pkg.mod.func"`` -> object; callables pass through."""
    if ref is None or callable(ref):
        return ref
    if not isinstance(ref, str) or not ref:
        raise ValueError(f"invalid executable reference {ref!r}")
    if ":" in ref:
        mod_name, attr_path = ref.split(":", 1)
    else:
        mod_name, _, attr_path = ref.rpartition(".")
        if not mod_name:
            raise ValueError(f"executable reference '{ref}' has no module part")
    try:
        obj: Any = importlib.import_module(mod_name)
    except ImportError as e:
        raise ImportError(f"cannot import module '{mod_name}' for executable '{ref}': {e}") from e
    for part in attr_path.split("."):
        if not hasattr(obj, part):
            raise AttributeError(f"'{mod_name}' has no attribute path '{attr_path}' (failed at '{part}')")
        obj = getattr(obj, part)
    if not callable(obj):
        raise TypeError(f"executable '{ref}' resolved to a non-callable {type(obj).__name__}")
    return obj


@dataclass
class AgentProcess:
    """Optional pre/post/env hooks of a node in multi-agent pipelines
    (reference: siirl/execution/dag/node.py:90-208)."""
    pre_process: Optional[Union[str, Callable]] = None
    post_process: Optional[Union[str, Callable]] = None
    env: Optional[Union[str, Callable, List[Any]]] = None
    pre_process_kwargs: Dict[str, Any] = field(default_factory=dict)
    post_process_kwargs: Dict[str, Any] = field(default_factory=dict)
    env_managers: List[Any] = field(default_factory=list)

    def resolve(self) -> None:
        self.pre_process = resolve_callable(self.pre_process)
        self.post_process = resolve_callable(self.post_process)
        if isinstance(self.env, (str,)):
            self.env = resolve_callable(self.env)

    def apply_pre_process(self, *args, **kwargs):
        if self.pre_process is None:
            return args[0] if args else None
        return self.pre_process(*args, **{**self.pre_process_kwargs, **kwargs})

    def apply_post_process(self, *args, **kwargs):
        if self.post_process is None:
            return args[0] if args else None
        return self.post_process(*args, **{**self.post_process_kwargs, **kwargs})


class Node:
    """One vertex of a :class:`TaskGraph`."""

    def __init__(self, node_id: str, node_type: Union[NodeType, str] = NodeType.COMPUTE,
                 node_role: Union[NodeRole, str] = NodeRole.DEFAULT, only_forward_compute: bool = False,
                 agent_group: int = 0, dependencies: Optional[List[str]] = None,
                 config: Optional[Dict[str, Any]] = None, executable_ref: Union[str, Callable, None] = None,
                 agent_options: Any = None, retry_limit: int = 0, user_options: Optional[Dict[str, Any]] = None,
                 filter_plugin: Optional[Callable] = None, agent_process: Optional[AgentProcess] = None):
        if not isinstance(node_id, str) or not node_id:
            raise ValueError("node_id must be a non-empty string")
        self.node_id = node_id
        self.node_type = _coerce_enum(NodeType, node_type)
        self.node_role = _coerce_enum(NodeRole, node_role)
        if self.node_role != NodeRole.DEFAULT and self.node_type not in (
                NodeType.MODEL_INFERENCE, NodeType.MODEL_TRAIN, NodeType.COMPUTE, NodeType.CUSTOM):
            raise ValueError(f"node '{node_id}': role {self.node_role.value} needs a model/compute node type, "
                             f"got {self.node_type.value}")
        self.only_forward_compute = bool(only_forward_compute)
        self.agent_group = int(agent_group)
        self.dependencies: List[str] = list(dict.fromkeys(dependencies or []))
        self.config: Dict[str, Any] = dict(config or {})
        self.executable_ref = executable_ref
        self._executable: Optional[Callable] = None
        self.agent_options = agent_options
        self.agent_process = agent_process
        self.user_options = dict(user_options or {})
        self.filter_plugin = filter_plugin
        self.retry_limit = int(retry_limit)
        self.retries_done = 0
        self.status = NodeStatus.PENDING
        self.output: Any = None
        self.error_info: Optional[str] = None
        if executable_ref is not None and callable(executable_ref):
            self._executable = executable_ref

    # ---- dependencies ------------------------------------------------------------------------
    def add_dependency(self, dep_id: str) -> None:
        if dep_id == self.node_id:
            raise ValueError(f"node '{self.node_id}' cannot depend on itself")
        if dep_id not in self.dependencies:
            self.dependencies.append(dep_id)

    def remove_dependency(self, dep_id: str) -> None:
        if dep_id in self.dependencies:
            self.dependencies.remove(dep_id)

    def is_ready(self, completed: set) -> bool:
        return all(d in completed for d in self.dependencies)

    # ---- status ------------------------------------------------------------------------------
    def update_status(self, status: NodeStatus, error_info: Optional[str] = None) -> None:
        self.status = status
        if status == NodeStatus.FAILED:
            self.error_info = error_info
        elif status in (NodeStatus.PENDING, NodeStatus.COMPLETED):
            self.error_info = None

    def can_retry(self) -> bool:
        return self.retries_done < self.retry_limit

    def increment_retry_count(self) -> None:
        self.retries_done += 1

    def reset(self) -> None:
        self.status = NodeStatus.PENDING
        self.output = None
        self.error_info = None
        self.retries_done = 0

    # ---- execution ---------------------------------------------------------------------------
    @property
    def executable(self) -> Optional[Callable]:
        if self._executable is None and self.executable_ref is not None:
            self._executable = resolve_callable(self.executable_ref)
        return self._executable

    @executable.setter
    def executable(self, fn: Optional[Callable]) -> None:
        self._executable = fn

    def _bind(self, fn: Callable, worker: Any) -> Callable:
        """Bind ``Class.method`` looked up on the class object to the worker instance."""
        if worker is None or inspect.ismethod(fn):
            return fn
        qual = getattr(fn, "__qualname__", "")
        if "." in qual and "<locals>" not in qual:
            owner_name, meth = qual.rsplit(".", 1)
            for klass in type(worker).__mro__:
                if klass.__name__ == owner_name.split(".")[-1] and hasattr(worker, meth):
                    return getattr(worker, meth)
        return fn

    def run(self, *args, **kwargs) -> Any:
        """Execute the node.  BARRIER_SYNC nodes without an executable run ``dist.barrier``."""
        worker = kwargs.pop("_dag_worker_instance", None)
        fn = self.executable
        self.update_status(NodeStatus.RUNNING)
        try:
            if fn is None:
                if self.node_type == NodeType.BARRIER_SYNC:
                    import torch.distributed as dist
                    if dist.is_available() and dist.is_initialized():
                        dist.barrier(group=kwargs.get("process_group"))
                    result = None
                else:
                    raise RuntimeError(f"node '{self.node_id}' has no executable")
            else:
                bound = self._bind(fn, worker)
                if bound is fn and worker is not None and "_dag_worker_instance" in inspect.signature(fn).parameters:
                    kwargs["_dag_worker_instance"] = worker
                result = bound(*args, **kwargs)
                if inspect.iscoroutine(result):
                    result = asyncio.get_event_loop().run_until_complete(result) if not _loop_running() \
                        else asyncio.run_coroutine_threadsafe(result, asyncio.get_event_loop()).result()
            self.output = result
            self.update_status(NodeStatus.COMPLETED)
            return result
        except Exception as e:  # noqa: BLE001
            self.update_status(NodeStatus.FAILED, f"{type(e).__name__}: {e}")
            raise

    def copy(self) -> "Node":
        n = Node(self.node_id, self.node_type, self.node_role, self.only_forward_compute, self.agent_group,
                 list(self.dependencies), dict(self.config), self.executable_ref, self.agent_options,
                 self.retry_limit, dict(self.user_options), self.filter_plugin, self.agent_process)
        n._executable = self._executable
        return n

    def __repr__(self) -> str:
        return (f"Node({self.node_id!r}, {self.node_type.value}, {self.node_role.value}, "
                f"deps={self.dependencies}, status={self.status.value})")


def _loop_running() -> bool:
    try:
        return asyncio.get_event_loop().is_running()
    except RuntimeError:
        return False
