"""Experiment tracking: ``Tracking(project, experiment, backends, config).log(data, step)``.

Backends (reference: siirl/utils/logger/tracking.py:27-148): ``console``, ``jsonl`` (native addition, always
available), ``tensorboard`` (``TENSORBOARD_DIR``), ``wandb`` / ``mlflow`` / ``swanlab`` / ``clearml`` when the
package is importable — a missing package raises at construction, not in the middle of a run."""
from __future__ import annotations

import json
import os
import time
from typing import Any, Dict, List, Optional, Union

SUPPORTED = ["console", "jsonl", "tensorboard", "wandb", "mlflow", "swanlab", "clearml", "vemlp_wandb"]


def concat_dict_to_str(d: Dict[str, Any], step: int) -> str:
    parts = [f"step:{step}"]
    for k in sorted(d):
        v = d[k]
        parts.append(f"{k}:{v:.4g}" if isinstance(v, float) else f"{k}:{v}")
    return " - ".join(parts)


class _Console:
    def log(self, data, step):
        print(concat_dict_to_str(data, step), flush=True)

    def finish(self):
        pass


class _Jsonl:
    def __init__(self, path: str):
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        self.f = open(path, "a")

    def log(self, data, step):
        self.f.write(json.dumps({"step": step, "time": time.time(), **data}) + "\n")
        self.f.flush()

    def finish(self):
        self.f.close()


class _TensorBoard:
    def __init__(self, log_dir: str):
        from torch.utils.tensorboard import SummaryWriter
        self.w = SummaryWriter(log_dir)

    def log(self, data, step):
        for k, v in data.items():
            if isinstance(v, (int, float)):
                self.w.add_scalar(k, v, step)

    def finish(self):
        self.w.close()


class _Wandb:
    def __init__(self, project, name, config):
        import wandb
        wandb.init(project=project, name=name, config=config)
        self.wandb = wandb

    def log(self, data, step):
        self.wandb.log(data, step=step)

    def finish(self):
        self.wandb.finish()


class Tracking:
    def __init__(self, project_name: str, experiment_name: str, default_backend: Union[str, List[str]] = "console",
                 config: Optional[Dict[str, Any]] = None, log_dir: Optional[str] = None):
        if isinstance(default_backend, str):
            default_backend = [default_backend]
        for b in default_backend:
            if b not in SUPPORTED:
                raise ValueError(f"logger backend '{b}' is not supported (have {SUPPORTED})")
        self.loggers: Dict[str, Any] = {}
        base = log_dir or os.environ.get("SIIRL_LOG_DIR", os.path.join("outputs", project_name, experiment_name))
        for b in default_backend:
            if b == "console":
                self.loggers[b] = _Console()
            elif b == "jsonl":
                self.loggers[b] = _Jsonl(os.path.join(base, "metrics.jsonl"))
            elif b == "tensorboard":
                self.loggers[b] = _TensorBoard(os.environ.get("TENSORBOARD_DIR", os.path.join(base, "tensorboard")))
            elif b in ("wandb", "vemlp_wandb"):
                self.loggers[b] = _Wandb(project_name, experiment_name, config)
            else:
                __import__(b)  # mlflow / swanlab / clearml: fail early when absent
                raise NotImplementedError(f"backend '{b}' is importable but not wired in this build")

    def log(self, data: Dict[str, Any], step: int, backend: Optional[List[str]] = None) -> None:
        for name, lg in self.loggers.items():
            if backend is None or name in backend:
                lg.log(data, step)

    def finish(self) -> None:
        for lg in self.loggers.values():
            lg.finish()


class ValidationGenerationsLogger:
    """Dumps a table of (input, output, score) per validation step as JSON lines."""

    def __init__(self, directory: str):
        self.directory = directory

    def log(self, samples, step: int) -> str:
        os.makedirs(self.directory, exist_ok=True)
        path = os.path.join(self.directory, f"{step}.jsonl")
        with open(path, "w") as f:
            for inp, out, score in samples:
                f.write(json.dumps({"input": inp, "output": out, "score": score, "step": step}) + "\n")
        return path
