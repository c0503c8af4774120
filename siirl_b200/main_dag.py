"""Command-line entry: ``python -m siirl_b200.main_dag key=value ...`` (same dotted keys as the reference's
``python3 -m siirl.main_dag``, siirl/main_dag.py:225-256).

Started directly it acts as the launcher: it spawns one process per GPU (``trainer.n_gpus_per_node``) and each
process re-enters here as a rank (torchrun's RANK / WORLD_SIZE environment also works).  Every rank runs the planner
locally — pipeline selection, node-config update, task scheduling and process-group derivation are deterministic
functions of the config — then builds its DAGWorker and executes the task graph."""
from __future__ import annotations

import datetime
import importlib
import os
import sys
from typing import List, Optional

import torch
import torch.distributed as dist

from .execution.dag import BUILTIN_PIPELINES, DAGConfigLoader, TaskGraph
from .execution.scheduler import ProcessGroupManager, TaskScheduler, update_task_graph_node_configs
from .execution.scheduler.launch import launch_local, validate_config
from .params import SiiRLArguments, parse_config


def load_pipeline(config: SiiRLArguments) -> TaskGraph:
    """Pipeline selection (reference: siirl/main_dag.py:44-139): a user hook ``dag.custom_pipeline_fn="mod:func"``
    wins; then a declarative ``dag.workflow_path``; else by ``algorithm.workflow_type`` and the advantage estimator."""
    hook = config.dag.custom_pipeline_fn
    if hook:
        mod_name, _, fn_name = hook.partition(":")
        if not fn_name:
            raise ValueError("dag.custom_pipeline_fn must look like 'package.module:function'")
        fn = getattr(importlib.import_module(mod_name), fn_name)
        graph = fn()
        if not isinstance(graph, TaskGraph):
            raise TypeError(f"{hook} returned {type(graph).__name__}, expected TaskGraph")
        return graph
    if config.dag.workflow_path:
        p = config.dag.workflow_path
        return DAGConfigLoader.load_from_file(p, "json" if p.endswith(".json") else "yaml")
    wt = config.algorithm.workflow_type.lower()
    if wt == "embodied":
        return BUILTIN_PIPELINES["embodied_srpo"]()
    if wt == "dapo":
        return BUILTIN_PIPELINES["dapo"]()
    if config.algorithm.adv_estimator == "gae":
        return BUILTIN_PIPELINES["ppo"]()
    return BUILTIN_PIPELINES["grpo"]()


def plan(config: SiiRLArguments, world_size: int):
    """Planner: TaskGraph -> per-rank sub-graphs -> process-group specs (pure function of its inputs)."""
    graph = load_pipeline(config)
    update_task_graph_node_configs(graph, config)
    gpus = max(1, min(config.trainer.n_gpus_per_node, world_size))
    nodes = max(1, world_size // gpus)
    scheduler = TaskScheduler(nodes, world_size // nodes)
    assignment = scheduler.schedule_and_assign_tasks([graph])
    pgm = ProcessGroupManager(world_size, assignment)
    return graph, assignment, pgm


def init_distributed(config: SiiRLArguments) -> int:
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return 1
    use_cuda = (config.trainer.device or "cuda") == "cuda" and torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")) % torch.cuda.device_count())
    backend = "cpu:gloo,cuda:nccl" if use_cuda else "gloo"
    dist.init_process_group(backend=backend, timeout=datetime.timedelta(minutes=30))
    return world


def run_rank(config: SiiRLArguments):
    from .dag_worker.dagworker import DAGWorker
    from .execution.scheduler.launch import start_heartbeat
    from .utils.logger.logging_utils import set_basic_config
    set_basic_config()
    start_heartbeat(config.fault.heartbeat_interval_s)
    world = init_distributed(config)
    validate_config(config, world)
    _, assignment, pgm = plan(config, world)
    comm = None
    if world > 1 and torch.cuda.is_available() and (config.trainer.device or "cuda") == "cuda":
        try:
            from .parallel.symm import SymmComm
            comm = SymmComm.create(dist.group.WORLD)
        except Exception as e:  # noqa: BLE001
            print(f"[siirl_b200] peer-memory communicator unavailable, using NCCL collectives: {e}", file=sys.stderr)
    worker = DAGWorker(config, pgm, assignment, comm=comm)
    worker.init_graph()
    history = worker.execute_task_graph()
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return history


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    config = parse_config(argv)
    already_rank = "RANK" in os.environ and "WORLD_SIZE" in os.environ
    nnodes = max(1, int(config.trainer.nnodes))
    nproc = config.trainer.n_gpus_per_node
    if already_rank or nproc * nnodes <= 1:
        run_rank(config)
        return 0
    from .execution.scheduler.launch import node_placement
    node_rank, master_addr, master_port = node_placement(nnodes)
    restarts = 0
    while True:
        run_argv = list(argv)
        if restarts > 0:
            # a relaunch continues from the newest complete checkpoint of this job when there is one (also when the
            # first launch started from ``resume_from_path``: reloading that path would repeat the steps since)
            from .utils.checkpoint.checkpoint_manager import find_latest_complete_ckpt_path
            root = os.path.expanduser(config.trainer.default_local_dir)
            if config.trainer.resume_mode == "disable" or find_latest_complete_ckpt_path(root, log=lambda *_: None):
                run_argv.append("trainer.resume_mode=auto")
        code = launch_local(run_argv, nproc, env={"SIIRL_RESTART_COUNT": str(restarts)},
                            heartbeat_timeout_s=config.fault.heartbeat_timeout_s, nnodes=nnodes, node_rank=node_rank,
                            master_addr=master_addr, master_port=master_port)
        if code == 0 or not config.fault.auto_restart or restarts >= config.fault.max_restarts:
            return code
        restarts += 1
        print(f"[siirl_b200] job failed with code {code}; restart {restarts}/{config.fault.max_restarts} from the "
              f"latest checkpoint", file=sys.stderr)


if __name__ == "__main__":
    sys.exit(main())
