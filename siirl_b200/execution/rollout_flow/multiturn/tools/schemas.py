"""OpenAI function-tool schema objects (reference: siirl/execution/rollout_flow/multiturn/tools/schemas.py)."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class OpenAIFunctionPropertySchema:
    type: str
    description: Optional[str] = None
    enum: Optional[List[str]] = None


@dataclass
class OpenAIFunctionParametersSchema:
    type: str = "object"
    properties: Dict[str, Any] = field(default_factory=dict)
    required: List[str] = field(default_factory=list)


@dataclass
class OpenAIFunctionSchema:
    name: str
    description: str = ""
    parameters: OpenAIFunctionParametersSchema = field(default_factory=OpenAIFunctionParametersSchema)
    strict: bool = False


@dataclass
class OpenAIFunctionToolSchema:
    type: str = "function"
    function: Optional[OpenAIFunctionSchema] = None

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "OpenAIFunctionToolSchema":
        f = d.get("function", {})
        p = f.get("parameters", {}) or {}
        return cls(type=d.get("type", "function"), function=OpenAIFunctionSchema(
            name=f["name"], description=f.get("description", ""),
            parameters=OpenAIFunctionParametersSchema(type=p.get("type", "object"), properties=p.get("properties", {}),
                                                      required=p.get("required", [])), strict=f.get("strict", False)))

    def to_dict(self) -> Dict[str, Any]:
        f = self.function
        return {"type": self.type, "function": {"name": f.name, "description": f.description,
                                                 "parameters": {"type": f.parameters.type,
                                                                "properties": f.parameters.properties,
                                                                "required": f.parameters.required}}}


@dataclass
class OpenAIFunctionCallSchema:
    name: str
    arguments: Dict[str, Any]

    @staticmethod
    def from_raw(name: str, arguments: Any):
        """Returns ``(call, has_decode_error)``; arguments may arrive as a JSON string."""
        err = False
        if isinstance(arguments, str):
            try:
                arguments = json.loads(arguments)
            except json.JSONDecodeError:
                arguments, err = {}, True
        if not isinstance(arguments, dict):
            arguments, err = {}, True
        return OpenAIFunctionCallSchema(name, arguments), err


@dataclass
class OpenAIFunctionToolCall:
    id: str
    function: OpenAIFunctionCallSchema
    type: str = "function"
