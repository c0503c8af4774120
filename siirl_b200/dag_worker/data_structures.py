"""Small records passed around by the DAG worker (reference: siirl/dag_worker/data_structures.py:23-50)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass
class NodeOutput:
    """What a node function returns: the (possibly new) batch and a flat metric dict."""
    batch: Any = None
    metrics: Dict[str, Any] = field(default_factory=dict)


@dataclass
class ValidationResult:
    input_text: str
    output_text: str
    score: float
    data_source: str
    extra_rewards: Dict[str, Any] = field(default_factory=dict)


@dataclass
class ValidationPayload:
    results: List[ValidationResult] = field(default_factory=list)
    metrics: Optional[Dict[str, float]] = None
