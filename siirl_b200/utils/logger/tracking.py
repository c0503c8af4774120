"""Experiment tracking: ``Tracking(project, experiment, backends, config).log(data, step)``.

Backends (reference: siirl/utils/logger/tracking.py:27-148): ``console``, ``jsonl`` (native addition, always
available), ``tensorboard`` (``TENSORBOARD_DIR``), ``wandb`` / ``mlflow`` / ``swanlab`` / ``clearml`` / ``vemlp_wandb`` when the
package is importable — a missing package raises ``ImportError`` at construction, not in the middle of a run."""
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
        proxy = ((config or {}).get("trainer") or {}).get("wandb_proxy") if isinstance(config, dict) else None
        wandb.init(project=project, name=name, config=config,
                   settings=wandb.Settings(https_proxy=proxy) if proxy else None)
        self.wandb = wandb

    def log(self, data, step):
        self.wandb.log(data, step=step)

    def finish(self):
        self.wandb.finish()


def _flatten_params(obj: Any, prefix: str = "", sep: str = "/") -> Dict[str, Any]:
    """Nested config -> flat ``{"a/b/c": value}`` dict (what MLflow's ``log_params`` wants)."""
    out: Dict[str, Any] = {}
    if isinstance(obj, dict):
        for k, v in obj.items():
            out.update(_flatten_params(v, f"{prefix}{sep}{k}" if prefix else str(k), sep))
    elif isinstance(obj, (list, tuple)):
        for i, v in enumerate(obj):
            out.update(_flatten_params(v, f"{prefix}{sep}{i}" if prefix else str(i), sep))
    else:
        out[prefix] = obj
    return out


class _Mlflow:
    """MLflow run: ``MLFLOW_TRACKING_URI`` selects the server, the project is the MLflow experiment, the
    experiment name the run name; metric keys have '@' replaced (MLflow rejects it)."""

    def __init__(self, project, name, config):
        import mlflow
        uri = os.environ.get("MLFLOW_TRACKING_URI")
        if uri:
            mlflow.set_tracking_uri(uri)
        exp = mlflow.set_experiment(project)
        mlflow.start_run(experiment_id=exp.experiment_id, run_name=name)
        params = _flatten_params(config or {})
        items = list(params.items())
        for i in range(0, len(items), 100):       # MLflow limits a batch to 100 parameters
            mlflow.log_params({k: str(v)[:250] for k, v in items[i:i + 100]})
        self.mlflow = mlflow

    def log(self, data, step):
        self.mlflow.log_metrics({k.replace("@", "_at_"): float(v) for k, v in data.items()
                                 if isinstance(v, (int, float))}, step=step)

    def finish(self):
        self.mlflow.end_run()


class _Swanlab:
    def __init__(self, project, name, config):
        import swanlab
        key = os.environ.get("SWANLAB_API_KEY")
        if key:
            swanlab.login(key)
        swanlab.init(project=project, experiment_name=name, config={"FRAMEWORK": "siirl_b200", **(config or {})},
                     logdir=os.environ.get("SWANLAB_LOG_DIR", "swanlog"), mode=os.environ.get("SWANLAB_MODE", "cloud"))
        self.swanlab = swanlab

    def log(self, data, step):
        self.swanlab.log({k: v for k, v in data.items() if isinstance(v, (int, float))}, step=step)

    def finish(self):
        self.swanlab.finish()


class _ClearML:
    """One ClearML task; a metric key ``a/b/c`` becomes title ``a``, series ``b/c``."""

    def __init__(self, project, name, config):
        import clearml
        self.task = clearml.Task.init(task_name=name, project_name=project, continue_last_task=True,
                                      output_uri=False)
        self.task.connect_configuration(config or {}, name="Hyperparameters")
        self.logger = self.task.get_logger()

    def log(self, data, step):
        for k, v in data.items():
            if isinstance(v, (int, float)):
                title, _, series = k.partition("/")
                self.logger.report_scalar(title=title, series=series or title, value=float(v), iteration=step)

    def finish(self):
        self.task.mark_completed()


class _VemlpWandb(_Wandb):
    """Volcengine ML platform's wandb-compatible tracker (credentials from ``VOLC_ACCESS_KEY_ID``,
    ``VOLC_SECRET_ACCESS_KEY``, ``MLP_TRACKING_REGION``)."""

    def __init__(self, project, name, config):
        import volcengine_ml_platform
        from volcengine_ml_platform import wandb as vw
        volcengine_ml_platform.init(ak=os.environ["VOLC_ACCESS_KEY_ID"], sk=os.environ["VOLC_SECRET_ACCESS_KEY"],
                                    region=os.environ["MLP_TRACKING_REGION"])
        vw.init(project=project, name=name, config=config, sync_tensorboard=True)
        self.wandb = vw


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
            elif b == "wandb":
                self.loggers[b] = _Wandb(project_name, experiment_name, config)
            else:
                cls = {"mlflow": _Mlflow, "swanlab": _Swanlab, "clearml": _ClearML, "vemlp_wandb": _VemlpWandb}[b]
                self.loggers[b] = cls(project_name, experiment_name, config)

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
