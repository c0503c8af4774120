"""Resolve ``"package.module:attr"`` and ``"path/to/file.py:attr"`` strings to Python objects.

Used by the pipeline hook (``dag.custom_pipeline_fn``), custom reward functions and the multi-agent workflow's
``process_path`` / ``env_path`` options (reference: siirl/utils/import_string.py:1-27 for the module form; the file
form is what its workflow YAMLs use for per-agent hooks)."""
from __future__ import annotations

import hashlib
import importlib
import importlib.util
import os
import sys
from types import ModuleType
from typing import Any


def load_module_from_file(path: str) -> ModuleType:
    """Import a Python file that is not on ``sys.path``; the same file is imported once per process."""
    full = os.path.abspath(os.path.expanduser(path))
    if not os.path.isfile(full):
        raise FileNotFoundError(f"no such Python file: {path}")
    name = "_siirl_user_" + hashlib.sha1(full.encode()).hexdigest()[:16]
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, full)
    if spec is None or spec.loader is None:
        raise ImportError(f"cannot import {path}")
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    try:
        spec.loader.exec_module(mod)
    except BaseException:
        sys.modules.pop(name, None)
        raise
    return mod


def import_string(ref: str) -> Any:
    """``"pkg.mod:attr"``, ``"pkg.mod.attr"`` or ``"dir/file.py:attr"`` -> the attribute (dotted attrs allowed)."""
    if not isinstance(ref, str) or not ref.strip():
        raise ValueError("import string must be a non-empty str")
    ref = ref.strip()
    target, sep, attr = ref.partition(":")
    if target.endswith(".py") or os.sep in target:
        mod = load_module_from_file(target)
        if not sep:
            return mod
    else:
        if not sep:
            target, _, attr = ref.rpartition(".")
            if not target:
                return importlib.import_module(ref)
        mod = importlib.import_module(target)
    obj: Any = mod
    for part in attr.split("."):
        if not hasattr(obj, part):
            raise AttributeError(f"'{ref}': {getattr(obj, '__name__', obj)!r} has no attribute '{part}'")
        obj = getattr(obj, part)
    return obj
