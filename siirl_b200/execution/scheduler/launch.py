"""Configuration validation and the multi-process launcher.

``validate_config`` holds the reference's launch-time checks (siirl/execution/scheduler/launch.py:94-308):
micro-batch parameter exclusivity, divisibility of batch sizes by the data-parallel width, ``loss_agg_mode``
whitelist, sequence parallelism requires remove-padding (always true here: the packed layout is native), critic
needed iff the advantage estimator is GAE.

``launch_local`` replaces the Ray actor manager (ray_actor_manager.py:128-286, resource_manager.py:31-132): it spawns
one OS process per GPU on this node with torchrun-style environment variables (RANK, LOCAL_RANK, WORLD_SIZE,
MASTER_ADDR=127.0.0.1, MASTER_PORT), watches child exit codes and a per-rank heartbeat in a TCPStore, and on the
first failure terminates the remaining ranks (fail-fast, as the reference's driver does on ``ActorDiedError``),
optionally restarting the job from the latest complete checkpoint (``fault.auto_restart``)."""
from __future__ import annotations

import os
import socket
import subprocess
import sys
import time
from typing import Dict, List, Optional

_LOSS_AGG_MODES = ("token-mean", "seq-mean-token-sum", "seq-mean-token-mean", "seq-mean-token-sum-norm")


def use_critic(config) -> bool:
    return config.algorithm.adv_estimator in ("gae", "gae_marft")


_WARNED: set = set()


def _warn_once(key: str, message: str) -> None:
    if key not in _WARNED and os.environ.get("RANK", "0") == "0":
        _WARNED.add(key)
        print(f"[siirl_b200] WARNING: {key}: {message}", file=sys.stderr)


def _warn_unsupported_keys(config) -> None:
    """Keys of the reference's configuration that parse but act differently here: say so once instead of silently
    doing something else."""
    arr = config.actor_rollout_ref
    for name, fc in (("actor_rollout_ref.actor", arr.actor.fsdp_config), ("critic", config.critic.fsdp_config)):
        if fc.param_offload:
            _warn_once(f"{name}.fsdp_config.param_offload", "trainable weights stay on the GPU (the rollout engine "
                       "reads them in place); use fsdp_config.sharding=zero3 to cut their footprint, "
                       "optimizer_offload for the Adam state, ref.fsdp_config.param_offload for the frozen policy")
    m = arr.model
    if getattr(m, "use_remove_padding", False) is False and "use_remove_padding" in getattr(config, "_explicit", ()):
        _warn_once("actor_rollout_ref.model.use_remove_padding", "sequences are always packed without padding")
    if getattr(m, "use_fused_kernels", False) is False and "use_fused_kernels" in getattr(config, "_explicit", ()):
        _warn_once("actor_rollout_ref.model.use_fused_kernels", "the fused LM-head log-prob / entropy kernel is "
                   "always used on GPUs")
    if arr.actor.strategy == "megatron" or config.critic.strategy == "megatron":
        mg = arr.actor.megatron
        if int(mg.tensor_model_parallel_size or 1) > 1 and not getattr(mg, "_native_tp", True):
            _warn_once("actor.megatron.tensor_model_parallel_size", "training tensor parallelism is mapped to the "
                       "native column/row-parallel layers")


def validate_config(config, world_size: Optional[int] = None) -> None:
    t = config.trainer
    if int(getattr(config.actor_rollout_ref.actor.megatron, "expert_tensor_parallel_size", 1) or 1) > 1:
        raise ValueError("megatron.expert_tensor_parallel_size > 1 is not supported: experts are whole on one rank "
                         "(expert_model_parallel_size spreads them over the group)")
    world = world_size or t.nnodes * t.n_gpus_per_node
    a, r, rf, c = (config.actor_rollout_ref.actor, config.actor_rollout_ref.rollout, config.actor_rollout_ref.ref,
                   config.critic)
    tp = max(1, r.tensor_model_parallel_size)
    if world % tp:
        raise ValueError(f"world size {world} is not divisible by rollout tensor_model_parallel_size {tp}")
    bs = config.data.gen_batch_size or config.data.train_batch_size
    if bs % (world // tp):
        raise ValueError(f"data batch size {bs} must be divisible by the rollout data-parallel width {world // tp}")

    def check_mutually_exclusive(mbs, mbs_per_gpu, name: str):
        if mbs is not None and mbs_per_gpu is not None and mbs_per_gpu != 1:
            raise ValueError(f"[{name}] You have set both '{name}.micro_batch_size' and "
                             f"'{name}.micro_batch_size_per_gpu'. Please remove '{name}.micro_batch_size' because "
                             f"only '*_micro_batch_size_per_gpu' is supported (the former is deprecated).")

    if not a.use_dynamic_bsz:
        check_mutually_exclusive(a.ppo_micro_batch_size, a.ppo_micro_batch_size_per_gpu, "actor_rollout_ref.actor")
        check_mutually_exclusive(rf.log_prob_micro_batch_size, rf.log_prob_micro_batch_size_per_gpu,
                                 "actor_rollout_ref.ref")
        check_mutually_exclusive(r.log_prob_micro_batch_size, r.log_prob_micro_batch_size_per_gpu,
                                 "actor_rollout_ref.rollout")
        if a.ppo_micro_batch_size_per_gpu is None and a.ppo_micro_batch_size is None:
            raise ValueError("[actor_rollout_ref.actor] set ppo_micro_batch_size_per_gpu or use_dynamic_bsz=True")
        sp = max(1, a.ulysses_sequence_parallel_size)
        if config.data.train_batch_size < a.ppo_mini_batch_size:
            raise ValueError("data.train_batch_size must be >= actor.ppo_mini_batch_size")
        if (a.ppo_mini_batch_size * r.n) % max(world // sp, 1):
            raise ValueError(f"actor.ppo_mini_batch_size * rollout.n ({a.ppo_mini_batch_size * r.n}) must be divisible "
                             f"by the data-parallel width {world // sp}")
    if a.loss_agg_mode not in _LOSS_AGG_MODES:
        raise ValueError(f"Invalid loss_agg_mode: {a.loss_agg_mode}; choose from {_LOSS_AGG_MODES}")
    if use_critic(config):
        if not c.use_dynamic_bsz:
            check_mutually_exclusive(c.ppo_micro_batch_size, c.ppo_micro_batch_size_per_gpu, "critic")
        if c.loss_agg_mode not in _LOSS_AGG_MODES:
            raise ValueError(f"Invalid critic loss_agg_mode: {c.loss_agg_mode}")
    _warn_unsupported_keys(config)
    if config.algorithm.use_kl_in_reward and a.use_kl_loss:
        print("NOTICE: both in-reward KL and KL loss are enabled.", file=sys.stderr)
    if r.multi_turn.enable and r.name not in ("sglang", "native", "vllm"):
        raise ValueError("multi-turn rollout needs an engine with an async generate API")
    if r.val_kwargs.do_sample and r.temperature <= 0:
        raise ValueError("validation sampling needs rollout.temperature > 0")
    if config.algorithm.adv_estimator not in ("gae", "grpo", "cpgd", "gae_marft"):
        from ...dag_worker.core_algos import ADV_ESTIMATOR_REGISTRY
        if config.algorithm.adv_estimator not in ADV_ESTIMATOR_REGISTRY:
            raise ValueError(f"unknown advantage estimator '{config.algorithm.adv_estimator}'")


def find_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def host_store(timeout_s: float = 300.0, attempts: int = 8):
    """A TCPStore server on a free loopback port, owned by the calling process: ``(store, port)``.  Picking a free
    port and binding it later are two steps, and another job on the machine may take the port in between, so the
    bind is retried on a fresh port when it fails."""
    import datetime

    import torch.distributed as dist
    last: Optional[BaseException] = None
    for _ in range(attempts):
        port = find_free_port()
        try:
            store = dist.TCPStore("127.0.0.1", port, is_master=True, wait_for_workers=False,
                                  timeout=datetime.timedelta(seconds=timeout_s))
            return store, port
        except (RuntimeError, OSError) as e:      # address already in use
            last = e
    raise RuntimeError(f"could not bind a rendezvous port after {attempts} attempts: {last}")


HEARTBEAT_EXIT_CODE = 124       # the job was stopped because a rank went silent (same code as timeout(1))


def stale_ranks(store, ranks: List[int], timeout_s: float) -> List[int]:
    """Ranks whose last heartbeat (``hb/<rank>`` = wall-clock seconds, written by ``start_heartbeat``) is older than
    ``timeout_s``.  A rank that has not written yet (still importing, building its model) is not stale."""
    now = time.time()
    out = []
    for r in ranks:
        key = f"hb/{r}"
        try:
            if not store.check([key]):
                continue
            last = float(store.get(key).decode())
        except Exception:  # noqa: BLE001 - a store hiccup must not take the job down
            continue
        if now - last > timeout_s:
            out.append(r)
    return out


class Heartbeat:
    """Daemon thread of a rank that writes ``hb/<rank>`` every ``interval_s`` seconds; ``stop()`` ends it (also what
    the ``drop_heartbeat`` fault injection calls to play a hung rank)."""

    def __init__(self, port: int, rank: int, interval_s: float = 1.0):
        import datetime
        import threading

        import torch.distributed as dist
        self._store = dist.TCPStore("127.0.0.1", port, is_master=False, timeout=datetime.timedelta(seconds=30))
        self._key, self._interval = f"hb/{rank}", max(0.05, float(interval_s))
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="siirl-heartbeat", daemon=True)
        self._thread.start()

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                self._store.set(self._key, repr(time.time()))
            except Exception:  # noqa: BLE001 - the launcher went away; nothing left to report to
                return
            self._stop.wait(self._interval)

    def stop(self) -> None:
        self._stop.set()


_HEARTBEAT: Optional[Heartbeat] = None


def start_heartbeat(interval_s: float = 1.0) -> Optional[Heartbeat]:
    """Called by every rank at start-up; a no-op unless the launcher asked for heartbeats."""
    global _HEARTBEAT
    port = os.environ.get("SIIRL_HEARTBEAT_PORT")
    if port and _HEARTBEAT is None:
        _HEARTBEAT = Heartbeat(int(port), int(os.environ.get("RANK", "0")), interval_s)
    return _HEARTBEAT


def stop_heartbeat() -> None:
    if _HEARTBEAT is not None:
        _HEARTBEAT.stop()


def launch_local(argv: List[str], nproc: int, env: Optional[Dict[str, str]] = None, poll_s: float = 0.5,
                 heartbeat_timeout_s: float = 0.0, module: str = "siirl_b200.main_dag", nnodes: int = 1,
                 node_rank: int = 0, master_addr: str = "127.0.0.1", master_port: int = 0) -> int:
    """Spawn this node's ``nproc`` ranks of ``python -m <module> <argv>`` and babysit them.  Returns the exit code
    (0 when every rank exited 0; otherwise the first non-zero code after the remaining ranks were terminated).

    One node (default): the launcher picks a free loopback port.  Several nodes: the same command runs on every
    node with its ``node_rank``; node 0's launcher hosts the rendezvous store on ``master_port`` (reachable at
    ``master_addr``), the other launchers and all ranks join it as clients.  Global rank = ``node_rank * nproc +
    local rank``.  A launcher that stops its ranks (a failed or silent rank) raises an abort flag in the store; the
    other nodes' launchers see it (or lose the store with node 0) and stop theirs, so a multi-node job ends as a
    whole instead of waiting in a collective."""
    import datetime

    import torch.distributed as dist
    # The launcher hosts the rendezvous store itself (the ranks join as clients, the way torchrun's agent does it):
    # the port is bound here, by the process that chose it, so no other job can take it before rank 0 starts.
    world = nproc * max(1, nnodes)
    if nnodes <= 1:
        rdzv_store, port = host_store()
        master_addr = "127.0.0.1"
    elif node_rank == 0:
        port = int(master_port)
        rdzv_store = dist.TCPStore(master_addr, port, is_master=True, wait_for_workers=False,
                                   timeout=datetime.timedelta(seconds=300))
    else:
        port = int(master_port)
        rdzv_store = dist.TCPStore(master_addr, port, is_master=False, wait_for_workers=False,
                                   timeout=datetime.timedelta(seconds=300))
    abort_key = f"siirl_launcher/abort/{(env or {}).get('SIIRL_RESTART_COUNT', '0')}"
    procs: List[subprocess.Popen] = []
    base = dict(os.environ)
    base.update(env or {})
    base.update({"MASTER_ADDR": master_addr, "MASTER_PORT": str(port), "WORLD_SIZE": str(world),
                 "LOCAL_WORLD_SIZE": str(nproc), "GROUP_RANK": str(node_rank), "SIIRL_LAUNCHED": "1",
                 "TORCHELASTIC_USE_AGENT_STORE": "True"})
    store = None
    if heartbeat_timeout_s > 0:
        store, hb_port = host_store(timeout_s=5.0)
        base["SIIRL_HEARTBEAT_PORT"] = str(hb_port)
    ranks = [node_rank * nproc + r for r in range(nproc)]
    for local, r in enumerate(ranks):
        e = dict(base)
        e.update({"RANK": str(r), "LOCAL_RANK": str(local)})
        procs.append(subprocess.Popen([sys.executable, "-m", module, *argv], env=e))
    code = 0
    try:
        while True:
            states = [p.poll() for p in procs]
            bad = [s for s in states if s not in (None, 0)]
            if bad:
                code = bad[0]
                break
            if all(s == 0 for s in states):
                break
            if store is not None:
                stale = stale_ranks(store, [ranks[i] for i, s in enumerate(states) if s is None], heartbeat_timeout_s)
                if stale:
                    print(f"[siirl_b200] no heartbeat from rank(s) {stale} for {heartbeat_timeout_s:.0f} s: stopping "
                          f"the job", file=sys.stderr)
                    code = HEARTBEAT_EXIT_CODE
                    break
            if nnodes > 1:
                try:
                    if rdzv_store.check([abort_key]):
                        print(f"[siirl_b200] node {node_rank}: another node stopped the job", file=sys.stderr)
                        code = int(rdzv_store.get(abort_key).decode() or 1)
                        break
                except Exception as e:  # noqa: BLE001  (node 0 and its store are gone)
                    print(f"[siirl_b200] node {node_rank}: lost the rendezvous store ({type(e).__name__}): stopping "
                          f"the local ranks", file=sys.stderr)
                    code = 1
                    break
            time.sleep(poll_s)
    finally:
        if code != 0 and nnodes > 1:
            try:
                rdzv_store.set(abort_key, str(code))
            except Exception:  # noqa: BLE001
                pass
        for p in procs:
            if p.poll() is None:
                p.terminate()
        deadline = time.time() + 10
        for p in procs:
            try:
                p.wait(timeout=max(0.1, deadline - time.time()))
            except subprocess.TimeoutExpired:
                p.kill()
        if code != 0 and nnodes > 1 and node_rank == 0:
            time.sleep(2 * poll_s + 0.5)          # the other launchers poll the flag from this process's store
        _ = (store, rdzv_store)
    return code


def node_placement(nnodes: int) -> tuple:
    """``(node_rank, master_addr, master_port)`` of this node from the environment of the usual cluster launchers
    (``NODE_RANK`` / ``GROUP_RANK`` / ``SLURM_NODEID`` / ``OMPI_COMM_WORLD_RANK``; ``MASTER_ADDR``, ``MASTER_PORT``)."""
    if nnodes <= 1:
        return 0, "127.0.0.1", 0
    rank = next((os.environ[k] for k in ("NODE_RANK", "GROUP_RANK", "SLURM_NODEID", "OMPI_COMM_WORLD_RANK")
                 if os.environ.get(k, "") != ""), None)
    addr, port = os.environ.get("MASTER_ADDR"), os.environ.get("MASTER_PORT")
    if rank is None or not addr or not port:
        raise RuntimeError(f"trainer.nnodes={nnodes}: start the same command on every node with NODE_RANK (0 .. "
                           f"{nnodes - 1}), MASTER_ADDR (node 0) and MASTER_PORT set")
    if not 0 <= int(rank) < nnodes:
        raise RuntimeError(f"NODE_RANK={rank} is outside 0 .. {nnodes - 1}")
    return int(rank), addr, int(port)
