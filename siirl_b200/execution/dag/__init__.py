from .builtin_pipelines import (BUILTIN_PIPELINES, dapo_pipeline, embodied_srpo_pipeline, grpo_pipeline,  # noqa: F401
                                ppo_pipeline)
from .config_loader import DAGConfigLoader, Ref, resolve_refs  # noqa: F401
from .node import AgentProcess, Node, NodeRole, NodeStatus, NodeType, resolve_callable  # noqa: F401
from .pipeline import NodeConfig, Pipeline  # noqa: F401
from .task_graph import TaskGraph  # noqa: F401
from .task_loader import (discover_and_split_parallel_paths, generate_structural_signature,  # noqa: F401
                          split_by_fan_out_to_exits, split_by_reconverging_paths)
