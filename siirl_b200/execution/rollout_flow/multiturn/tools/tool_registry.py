"""Tool configuration loading: YAML ``tools: [{class_name, config, tool_schema}]`` -> tool instances
(reference: siirl/execution/rollout_flow/multiturn/tools/tool_registry.py)."""
from __future__ import annotations

import importlib
from typing import Dict, List

import yaml

from .base_tool import BaseTool
from .schemas import OpenAIFunctionToolSchema


def get_tool_class(name: str):
    mod, _, cls = name.rpartition(".")
    if mod:
        return getattr(importlib.import_module(mod), cls)
    pkg = "siirl_b200.execution.rollout_flow.multiturn.tools"
    for sub in ("builtin_tools", "remote_tools"):
        m = importlib.import_module(f"{pkg}.{sub}")
        if hasattr(m, cls):
            return getattr(m, cls)
    raise AttributeError(f"no built-in tool class named '{cls}'")


def initialize_tools_from_config(path_or_dict) -> List[BaseTool]:
    if isinstance(path_or_dict, str):
        with open(path_or_dict) as f:
            cfg = yaml.safe_load(f)
    else:
        cfg = path_or_dict
    tools: List[BaseTool] = []
    for t in (cfg or {}).get("tools", []):
        cls = get_tool_class(t["class_name"])
        schema = OpenAIFunctionToolSchema.from_dict(t["tool_schema"])
        tools.append(cls(config=t.get("config", {}), tool_schema=schema))
    return tools


def tools_by_name(tools: List[BaseTool]) -> Dict[str, BaseTool]:
    return {t.name: t for t in tools}

