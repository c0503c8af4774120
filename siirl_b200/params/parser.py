"""Config loader: YAML file(s) + Hydra-style ``a.b.c=value`` command-line overrides merged into the
typed dataclass tree of :mod:`siirl_b200.params.schema`.

Behaviour follows the reference's CLI contract (siirl/params/parser.py:33-59: unknown argv entries
are dotted overrides) without Hydra, OmegaConf or dacite:

* ``key=value``   set (value parsed as YAML: ints, floats, bools, null, lists ``[a,b]``, dicts ``{k: v}``)
* ``+key=value``  same as ``key=value`` (accepted for Hydra compatibility; also adds new dict entries)
* ``~key``        reset the key to its default
* ``--config path.yaml`` (repeatable) is merged before the overrides; ``--print-config`` dumps the result
* unknown keys raise ``ConfigError`` listing the closest valid names
"""
from __future__ import annotations

import argparse
import copy
import difflib
import sys
import typing
from dataclasses import fields, is_dataclass
from typing import Any, Dict, List, Optional, Sequence

import yaml

from .schema import SiiRLArguments, to_dict


class ConfigError(ValueError):
    pass


def _parse_scalar(text: str) -> Any:
    try:
        return yaml.safe_load(text)
    except yaml.YAMLError:
        return text


def _strip_optional(tp):
    origin = typing.get_origin(tp)
    if origin is typing.Union:
        args = [a for a in typing.get_args(tp) if a is not type(None)]
        if len(args) == 1:
            return args[0], True
    return tp, False


def _coerce(value: Any, tp: Any, path: str) -> Any:
    """Coerce a parsed YAML value to the annotated field type."""
    tp, optional = _strip_optional(tp)
    if value is None:
        return None
    origin = typing.get_origin(tp)
    if is_dataclass(tp):
        if isinstance(value, dict):
            inst = tp()
            apply_dict(inst, value, path)
            return inst
        if is_dataclass(value):
            return value
        raise ConfigError(f"{path}: expected a mapping for {tp.__name__}, got {value!r}")
    if tp is bool:
        if isinstance(value, bool):
            return value
        if isinstance(value, str) and value.lower() in ("true", "false", "1", "0", "yes", "no"):
            return value.lower() in ("true", "1", "yes")
        if isinstance(value, (int, float)):
            return bool(value)
        raise ConfigError(f"{path}: expected bool, got {value!r}")
    if tp is int:
        if isinstance(value, bool):
            return int(value)
        if isinstance(value, int):
            return value
        if isinstance(value, float) and value.is_integer():
            return int(value)
        if isinstance(value, str):
            try:
                return int(value)
            except ValueError:
                pass
        raise ConfigError(f"{path}: expected int, got {value!r}")
    if tp is float:
        if isinstance(value, (int, float)) and not isinstance(value, bool):
            return float(value)
        if isinstance(value, str):
            try:
                return float(value)
            except ValueError:
                pass
        raise ConfigError(f"{path}: expected float, got {value!r}")
    if tp is str:
        return value if isinstance(value, str) else str(value)
    if origin in (list, List) or tp is list:
        if isinstance(value, str):
            value = [value]
        if not isinstance(value, (list, tuple)):
            value = [value]
        args = typing.get_args(tp)
        if args:
            return [_coerce(v, args[0], f"{path}[{i}]") for i, v in enumerate(value)]
        return list(value)
    if origin is tuple or tp is tuple:
        if isinstance(value, (list, tuple)):
            return tuple(value)
        raise ConfigError(f"{path}: expected a sequence, got {value!r}")
    if origin in (dict, Dict) or tp is dict:
        if isinstance(value, dict):
            return dict(value)
        raise ConfigError(f"{path}: expected a mapping, got {value!r}")
    return value


def _type_hints(cls) -> Dict[str, Any]:
    return typing.get_type_hints(cls)


def apply_dict(obj: Any, values: Dict[str, Any], prefix: str = "") -> None:
    """Recursively merge a nested mapping into a dataclass instance."""
    hints = _type_hints(type(obj))
    names = {f.name for f in fields(obj)}
    for k, v in values.items():
        path = f"{prefix}.{k}" if prefix else k
        if k not in names:
            close = difflib.get_close_matches(k, names, n=3)
            raise ConfigError(f"unknown config key '{path}'" + (f" (did you mean {close}?)" if close else ""))
        cur = getattr(obj, k)
        if is_dataclass(cur) and isinstance(v, dict):
            apply_dict(cur, v, path)
        else:
            setattr(obj, k, _coerce(v, hints[k], path))


def set_by_path(obj: Any, dotted: str, value: Any, allow_new: bool = False) -> None:
    parts = dotted.split(".")
    cur = obj
    for i, p in enumerate(parts[:-1]):
        if isinstance(cur, dict):
            cur = cur.setdefault(p, {})
            continue
        if not is_dataclass(cur) or p not in {f.name for f in fields(cur)}:
            names = [f.name for f in fields(cur)] if is_dataclass(cur) else []
            close = difflib.get_close_matches(p, names, n=3)
            raise ConfigError(f"unknown config key '{'.'.join(parts[: i + 1])}'" +
                              (f" (did you mean {close}?)" if close else ""))
        nxt = getattr(cur, p)
        if nxt is None:
            tp, _ = _strip_optional(_type_hints(type(cur))[p])
            if is_dataclass(tp):
                nxt = tp()
                setattr(cur, p, nxt)
        cur = nxt
    last = parts[-1]
    if isinstance(cur, dict):
        cur[last] = value
        return
    if not is_dataclass(cur):
        raise ConfigError(f"cannot set '{dotted}': parent is not a config group")
    names = {f.name for f in fields(cur)}
    if last not in names:
        close = difflib.get_close_matches(last, names, n=3)
        raise ConfigError(f"unknown config key '{dotted}'" + (f" (did you mean {close}?)" if close else ""))
    setattr(cur, last, _coerce(value, _type_hints(type(cur))[last], dotted))


def reset_by_path(obj: Any, dotted: str) -> None:
    parts = dotted.split(".")
    cur = obj
    for p in parts[:-1]:
        cur = getattr(cur, p)
    default_parent = type(cur)()
    setattr(cur, parts[-1], getattr(default_parent, parts[-1]))


def get_by_path(obj: Any, dotted: str) -> Any:
    cur = obj
    for p in dotted.split("."):
        cur = cur[p] if isinstance(cur, dict) else getattr(cur, p)
    return cur


def parse_overrides(cfg: SiiRLArguments, overrides: Sequence[str]) -> SiiRLArguments:
    for item in overrides:
        if item.startswith("~"):
            reset_by_path(cfg, item[1:].split("=")[0])
            continue
        if "=" not in item:
            raise ConfigError(f"override '{item}' is not of the form key=value")
        key, text = item.split("=", 1)
        allow_new = key.startswith("+")
        key = key.lstrip("+")
        set_by_path(cfg, key, _parse_scalar(text), allow_new=allow_new)
    return cfg


def load_yaml(cfg: SiiRLArguments, path: str) -> SiiRLArguments:
    with open(path) as f:
        data = yaml.safe_load(f) or {}
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: top level must be a mapping")
    apply_dict(cfg, data)
    return cfg


def parse_config(argv: Optional[Sequence[str]] = None) -> SiiRLArguments:
    """Entry used by ``python -m siirl_b200.main_dag``."""
    argv = list(sys.argv[1:] if argv is None else argv)
    ap = argparse.ArgumentParser(add_help=True, description="siirl_b200 configuration")
    ap.add_argument("--config", action="append", default=[], help="YAML file merged before the overrides")
    ap.add_argument("--print-config", action="store_true")
    known, unknown = ap.parse_known_args(argv)
    cfg = SiiRLArguments()
    for path in known.config:
        load_yaml(cfg, path)
    parse_overrides(cfg, unknown)
    finalize(cfg)
    if known.print_config:
        print(yaml.safe_dump(to_dict(cfg), sort_keys=False))
    return cfg


def finalize(cfg: SiiRLArguments) -> SiiRLArguments:
    """Derived defaults shared by all entry points (reference: siirl/main_dag.py:110-111 and worker init)."""
    ro = cfg.actor_rollout_ref.rollout
    if ro.prompt_length is None:
        ro.prompt_length = cfg.data.max_prompt_length
    if ro.response_length is None:
        ro.response_length = cfg.data.max_response_length
    if cfg.algorithm.adv_estimator == "cpgd":
        cfg.actor_rollout_ref.actor.use_cpgd_loss = True
    if cfg.actor_rollout_ref.actor.use_cpgd_loss and cfg.actor_rollout_ref.actor.policy_loss.loss_mode == "vanilla":
        cfg.actor_rollout_ref.actor.policy_loss.loss_mode = "cpgd"
    return cfg


def merge_node_overrides(base: Any, overrides: Dict[str, Any]) -> Any:
    """Deep-copy a config group and merge per-node overrides (reference: graph_updater.py:57-128)."""
    out = copy.deepcopy(base)
    if overrides:
        flat = {k: v for k, v in overrides.items() if "." in k}
        nested = {k: v for k, v in overrides.items() if "." not in k}
        if nested:
            apply_dict(out, nested)
        for k, v in flat.items():
            set_by_path(out, k, v)
    return out


def pretty(cfg: Any) -> str:
    return yaml.safe_dump(to_dict(cfg), sort_keys=False)


__all__ = ["ConfigError", "parse_config", "parse_overrides", "load_yaml", "apply_dict", "set_by_path",
           "get_by_path", "merge_node_overrides", "finalize", "pretty"]
