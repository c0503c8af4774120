"""DAGWorker: the per-GPU controller.  Every process runs one and walks the same task graph each step
(multi-controller SPMD; no central driver in the data path).

Structure and handler names follow the reference (siirl/dag_worker/dagworker.py:83-1318): ``init_graph`` builds the
distributed groups, tokenizer, dataloader, reward manager and the role workers; ``execute_task_graph`` runs the
training loop; one step is a topological walk over the DAG calling the node functions
``generate / compute_reward / compute_old_log_prob / compute_ref_log_prob / compute_value / compute_advantage /
train_critic / train_actor``; data moves between nodes through an in-process cache when the data-parallel width is
unchanged and through the Data Coordinator otherwise (always for DAPO's filtered samples).

Differences that matter for speed: batches stay on the device between nodes, there is no per-node world barrier
(only one at the step boundary), metrics are reduced with one packed all-reduce per step.
"""
from __future__ import annotations

import os
import sys
import time
from collections import deque
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..data_coordinator import (Batch, DataCoordinator, Dict2Samples, Samples2Dict, init_data_coordinator,
                                preprocess_dataloader)
from ..data_coordinator.dataloader import DataLoaderNode, load_tokenizer
from ..engine.workers import ActorRolloutRefWorker, CriticWorker, RewardModelWorker
from ..execution.dag import Node, NodeRole, NodeType, TaskGraph
from ..execution.scheduler.reward import compute_reward as guarded_compute_reward
from ..execution.scheduler.reward import create_reward_manager
from ..utils.logger.tracking import Tracking
from ..utils.debug.profile import Profiler, mark_end_range, mark_start_range
from ..utils.metrics.metric_utils import (compute_data_metric, compute_throughput_metrics, compute_timing_metrics,
                                          format_core_performance_metrics, reduce_metrics_across_ranks,
                                          write_rank_performance_csv)
from . import core_algos
from .checkpoint_manager import CheckpointManager
from .data_structures import NodeOutput
from .validator import Validator


class _Timer:
    def __init__(self, name: str, sink: Dict[str, float], sync: bool):
        self.name, self.sink, self.sync = name, sink, sync

    def __enter__(self):
        if self.sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        self.sink[self.name] = self.sink.get(self.name, 0.0) + time.perf_counter() - self.t0


class DAGWorker:
    def __init__(self, config, process_group_manager=None, taskgraph_mapping: Optional[Dict[int, TaskGraph]] = None,
                 data_coordinator: Optional[DataCoordinator] = None, device: Optional[torch.device] = None,
                 comm=None, tokenizer=None):
        self.config = config
        self.pgm = process_group_manager
        self._dist = dist.is_available() and dist.is_initialized()
        self._rank = dist.get_rank() if self._dist else 0
        self.world_size = dist.get_world_size() if self._dist else 1
        mapping = taskgraph_mapping or {}
        self.taskgraph: Optional[TaskGraph] = mapping.get(self._rank)
        self.data_coordinator = data_coordinator
        self.comm = comm
        self.tokenizer = tokenizer
        if device is None:
            want_cuda = (config.trainer.device or "cuda") == "cuda" and torch.cuda.is_available()
            device = torch.device("cuda", torch.cuda.current_device()) if want_cuda else torch.device("cpu")
        self.device = torch.device(device)
        self.enable_perf = bool(config.dag.enable_perf or os.environ.get("SIIRL_ENABLE_PERF"))
        self.global_steps = 0
        self.total_training_steps = 0
        self.internal_data_cache: Dict[str, Batch] = {}
        self.workers: Dict[str, Any] = {}
        self._shared_workers: Dict[str, str] = {}
        self.process_groups: Dict[str, Any] = {}
        self.timing_raw: Dict[str, float] = {}
        self.tracker: Optional[Tracking] = None
        self.kl_ctrl_in_reward = None
        self.history: List[Dict[str, float]] = []
        self._dapo_gen_batches = 0
        self.last_step_tokens = self.last_h2d_bytes = self.last_d2h_bytes = 0
        # per-call generation settings that win over the rollout config for the following steps, e.g.
        # {"response_length": 128, "do_sample": False} (read by ``ActorRolloutRefWorker.generate_sequences``)
        self.rollout_meta_overrides: Dict[str, Any] = {}
        self._multi_agent = False
        self.multi_agent_loop = None
        self._agent_ids: List[int] = [0]
        self._initialized = False

    # ================================================================================================
    # initialisation
    # ================================================================================================
    def init_graph(self) -> None:
        if self.taskgraph is None:
            raise RuntimeError(f"rank {self._rank} has no task graph assigned")
        self._setup_distributed_environment()
        if self.tokenizer is None:
            tok_path = self.config.data.tokenizer or self.config.actor_rollout_ref.model.path
            vocab = self._vocab_size_hint()
            self.tokenizer = load_tokenizer(tok_path if not self.config.actor_rollout_ref.model.arch_preset else None,
                                            vocab_size=vocab, model_args=self.config.actor_rollout_ref.model)
        self._import_external_libs()
        self._setup_dataloader()
        self._setup_reward_managers()
        self._bind_default_executables()
        self._initialize_node_workers()
        self._setup_multi_agent_loop()
        if self.config.algorithm.use_kl_in_reward:
            self.kl_ctrl_in_reward = core_algos.get_kl_controller(self.config.algorithm.kl_ctrl)
        if self.data_coordinator is None:
            self.data_coordinator = init_data_coordinator(self.config.trainer.nnodes,
                                                          self.config.actor_rollout_ref.actor.ppo_mini_batch_size,
                                                          self.world_size, group=None, comm=self.comm,
                                                          name=f"dc_rank{self._rank}")
        self.validator = Validator(self)
        # torch.profiler window on the steps / ranks named by ``profiler.*``; node handlers run inside NVTX ranges
        # while it (or ``dag.enable_perf``) is on (reference: dagworker.py:206-212, 421-442)
        self.profiler = Profiler(self.config.profiler, self._rank)
        self.checkpoint_manager = CheckpointManager(self)
        self.global_steps = self.checkpoint_manager.load_checkpoint()
        if self._rank == 0:
            t = self.config.trainer
            self.tracker = Tracking(t.project_name, t.experiment_name, t.logger, config=self.config.to_dict())
        self._initialized = True

    def _vocab_size_hint(self) -> int:
        from ..engine.workers import resolve_model_config
        try:
            return resolve_model_config(self.config.actor_rollout_ref.model).vocab_size
        except Exception:  # noqa: BLE001
            return 1024

    def _setup_distributed_environment(self) -> None:
        """One ``new_group`` per rank tuple the planner derived (every rank creates every group, in the same
        order, as torch.distributed requires)."""
        if not self._dist or self.pgm is None:
            return
        for name in sorted(self.pgm.process_group_spec, key=lambda n: int(n.rsplit("_", 1)[-1])):
            ranks = self.pgm.process_group_spec[name]
            self.process_groups[name] = None if len(ranks) == self.world_size else dist.new_group(ranks)
            if len(ranks) == self.world_size:
                self.process_groups[name] = dist.group.WORLD

    def _node_group(self, node: Node):
        if not self._dist or self.pgm is None:
            return None
        a = self.pgm.get_node_assignment(node.node_id)
        return self.process_groups.get(a["process_group_name"]) if a else dist.group.WORLD

    def _get_node_dp_info(self, node: Node):
        """(dp_size, dp_rank, tp_rank, tp_size): ranks are laid out [DP][PP][TP] with TP fastest
        (reference dagworker.py:1262-1308)."""
        group = self._node_group(node)
        gw = dist.get_world_size(group) if self._dist else 1
        gr = dist.get_rank(group) if self._dist else 0
        tp = 1
        if node.node_role == NodeRole.ROLLOUT:
            tp = max(1, self.config.actor_rollout_ref.rollout.tensor_model_parallel_size)
        elif node.node_role in (NodeRole.ACTOR, NodeRole.REFERENCE):
            # Ulysses peers work on the same micro-batches
            a = self.config.actor_rollout_ref.actor
            tp = max(1, a.ulysses_sequence_parallel_size, int(a.megatron.context_parallel_size or 1),
                     int(a.megatron.pipeline_model_parallel_size or 1),
                     int(a.megatron.tensor_model_parallel_size or 1) if a.strategy == "megatron" else 1)
        elif node.node_role == NodeRole.CRITIC:
            tp = max(1, self.config.critic.ulysses_sequence_parallel_size)
        dp = max(1, gw // tp)
        return dp, gr // tp, gr % tp, tp

    def _setup_dataloader(self) -> None:
        rollout_nodes = self.taskgraph.get_nodes_by_role(NodeRole.ROLLOUT)
        tp = self.config.actor_rollout_ref.rollout.tensor_model_parallel_size
        if rollout_nodes:
            g = self._node_group(rollout_nodes[0])
            gw = dist.get_world_size(g) if self._dist else 1
            gr = dist.get_rank(g) if self._dist else 0
        else:
            gw, gr = self.world_size, self._rank
        self.dataloader = DataLoaderNode(self.config, self.tokenizer, None, gw, gr, tp)
        t = self.config.trainer
        steps = self.dataloader.num_train_batches * t.total_epochs
        self.total_training_steps = t.total_training_steps if t.total_training_steps is not None else steps

    def _setup_reward_managers(self) -> None:
        self.reward_fn = create_reward_manager(self.config, self.tokenizer, num_examine=0,
                                               max_resp_len=self.config.data.max_response_length)
        self.val_reward_fn = create_reward_manager(self.config, self.tokenizer, num_examine=1,
                                                   max_resp_len=self.config.data.max_response_length)

    def _bind_default_executables(self) -> None:
        """Nodes of a declarative (YAML / JSON) workflow name no function: bind the handler their role implies
        (reference: dagworker.py ``_setup_role_worker_mapping`` + node binding in ``_initialize_node_workers``)."""
        by_role = {
            (NodeRole.ROLLOUT, False): self.generate, (NodeRole.ROLLOUT, True): self.generate,
            (NodeRole.REWARD, False): self.compute_reward, (NodeRole.REWARD, True): self.compute_reward,
            (NodeRole.ADVANTAGE, False): self.compute_advantage, (NodeRole.ADVANTAGE, True): self.compute_advantage,
            (NodeRole.ACTOR, True): self.compute_old_log_prob, (NodeRole.ACTOR, False): self.train_actor,
            (NodeRole.REFERENCE, False): self.compute_ref_log_prob, (NodeRole.REFERENCE, True): self.compute_ref_log_prob,
            (NodeRole.CRITIC, True): self.compute_value, (NodeRole.CRITIC, False): self.train_critic,
        }
        for node in self.taskgraph.nodes.values():
            if node.executable is not None or node.node_type == NodeType.BARRIER_SYNC:
                continue
            fn = by_role.get((node.node_role, node.only_forward_compute))
            if fn is None and node.node_role == NodeRole.DYNAMIC_SAMPLING:
                from ..user_interface.filter_interface.dapo import dynamic_sampling
                fn = dynamic_sampling
            if fn is None:
                raise RuntimeError(f"node '{node.node_id}' ({node.node_type.value}/{node.node_role.value}) names no "
                                   f"executable and its role has no default handler")
            node.executable = fn

    @staticmethod
    def _agent_option(node: Optional[Node], key: str, default: Any = None) -> Any:
        opts = getattr(node, "agent_options", None) if node is not None else None
        if opts is None:
            return default
        return opts.get(key, default) if isinstance(opts, dict) else getattr(opts, key, default)

    def _initialize_node_workers(self) -> None:
        """One hybrid worker per agent group for actor/rollout/ref nodes, one critic, one reward model.
        ``agent_options.share_instance: g`` makes a node use agent group g's worker of the same kind."""
        seed = self.config.trainer.seed
        for node in self.taskgraph.nodes.values():
            if node.node_type not in (NodeType.MODEL_TRAIN, NodeType.MODEL_INFERENCE):
                continue
            ag = node.agent_group
            share = self._agent_option(node, "share_instance")
            if share is not None and int(share) != ag:
                kind = "critic" if node.node_role == NodeRole.CRITIC else (
                    "reward" if node.node_role == NodeRole.REWARD else "actor_rollout_ref")
                self._shared_workers[f"{kind}_{ag}"] = f"{kind}_{int(share)}"
                continue
            group = self._node_group(node)
            cfg = node.config.get("intern_config")
            if node.node_role in (NodeRole.ACTOR, NodeRole.ROLLOUT, NodeRole.REFERENCE):
                key = f"actor_rollout_ref_{ag}"
                if key not in self.workers:
                    roles = {n.node_role for n in self.taskgraph.nodes.values() if n.agent_group == ag}
                    need_ref = NodeRole.REFERENCE in roles and (
                        self.config.actor_rollout_ref.actor.use_kl_loss or self.config.algorithm.use_kl_in_reward)
                    role = "actor_rollout_ref" if need_ref else "actor_rollout"
                    w = ActorRolloutRefWorker(cfg or self.config.actor_rollout_ref, role, group, self.device,
                                              self.comm, seed, self.tokenizer)
                    w.total_training_steps = self.total_training_steps
                    w.init_model()
                    self.workers[key] = w
            elif node.node_role == NodeRole.CRITIC:
                key = f"critic_{ag}"
                if key not in self.workers:
                    w = CriticWorker(cfg or self.config.critic, group, self.device, self.comm, seed,
                                     rollout_n=self.config.actor_rollout_ref.rollout.n)
                    w.total_training_steps = self.total_training_steps
                    w.init_model()
                    self.workers[key] = w
            elif node.node_role == NodeRole.REWARD and self.config.reward_model.enable:
                key = f"reward_{ag}"
                if key not in self.workers:
                    w = RewardModelWorker(cfg or self.config.reward_model, group, self.device, self.comm, seed,
                                          input_tokenizer=self.tokenizer)
                    w.init_model()
                    self.workers[key] = w
        if self.config.reward_model.enable and "reward_0" not in self.workers:
            w = RewardModelWorker(self.config.reward_model, None, self.device, self.comm, seed,
                                  input_tokenizer=self.tokenizer)
            w.init_model()
            self.workers["reward_0"] = w
        for alias, target in self._shared_workers.items():
            if alias in self.workers:
                continue       # another node of the group built its own instance
            if target not in self.workers:
                raise RuntimeError(f"share_instance: no worker '{target}' to share as '{alias}'")
            self.workers[alias] = self.workers[target]

    def _arr(self, node: Optional[Node] = None) -> ActorRolloutRefWorker:
        return self.workers[f"actor_rollout_ref_{node.agent_group if node is not None else 0}"]

    # ================================================================================================
    # multi-agent workflows (several agent groups, each with its own policy; MARFT)
    # ================================================================================================
    def _setup_multi_agent_loop(self) -> None:
        """With rollout nodes of more than one agent group, generation is one joint loop over the agents
        (reference: dagworker.py:999-1014 ``_setup_multi_agent_loop``).  Per-agent hooks come from the rollout
        nodes' ``agent_options``: ``process_path`` (a Python file with ``pre_process(tokenizer, prompt_id, obs,
        **kw)`` / ``post_process(tokenizer, prompt_id, response_id, **kw)``), ``pre_process_kwargs``,
        ``post_process_kwargs``, ``env_path: ["file.py:Class"]`` and ``obs_with_env``."""
        model_nodes = [n for n in self.taskgraph.nodes.values()
                       if n.node_type in (NodeType.MODEL_TRAIN, NodeType.MODEL_INFERENCE)]
        self._agent_ids = sorted({n.agent_group for n in model_nodes}) or [0]
        rollout_nodes = sorted(self.taskgraph.get_nodes_by_role(NodeRole.ROLLOUT), key=lambda n: n.agent_group)
        groups = sorted({n.agent_group for n in rollout_nodes})
        if len(groups) < 2:
            return
        from ..execution.rollout_flow.multi_agent.multiagent_generate import MultiAgentLoop
        from ..utils.import_string import import_string, load_module_from_file
        tok = self.tokenizer
        pre, post, env_cls, obs_with_env = {}, {}, None, False
        for node in rollout_nodes:
            k = node.agent_group
            path = self._agent_option(node, "process_path")
            if path:
                mod = load_module_from_file(path)
                pk = dict(self._agent_option(node, "pre_process_kwargs") or {})
                qk = dict(self._agent_option(node, "post_process_kwargs") or {})
                if hasattr(mod, "pre_process"):
                    pre[k] = (lambda ids, obs, agent, turn, _f=mod.pre_process, _kw=pk: _f(tok, list(ids), obs, **_kw))
                if hasattr(mod, "post_process"):
                    post[k] = (lambda ids, resp, agent, turn, _f=mod.post_process, _kw=qk:
                               _f(tok, list(ids), list(resp), **_kw))
            env_path = self._agent_option(node, "env_path")
            if env_path:
                env_cls = import_string(env_path[0] if isinstance(env_path, (list, tuple)) else env_path)
            obs_with_env = obs_with_env or bool(self._agent_option(node, "obs_with_env", False))
        r = self.config.actor_rollout_ref.rollout
        self.multi_agent_loop = MultiAgentLoop(
            {k: self.workers[f"actor_rollout_ref_{k}"] for k in groups}, tok, self.config.data.max_prompt_length,
            max_turns=r.multi_turn.max_assistant_turns or 1, pre_process=pre, post_process=post,
            env_factory=env_cls, colocate=True, group=self._node_group(rollout_nodes[0]),
            use_all_traj=bool(r.multi_turn.use_all_traj), obs_with_env=obs_with_env and env_cls is not None)
        self._multi_agent = True

    def _agent_prefix(self, node: Optional[Node]) -> str:
        """Tensors of every agent but the last travel under ``agent_group_{k}_``; the last agent's are unprefixed."""
        if not self._multi_agent or node is None or node.agent_group == self._agent_ids[-1]:
            return ""
        return f"agent_group_{node.agent_group}_"

    def _on_agent_view(self, batch: Batch, node: Optional[Node], fn) -> Batch:
        """Run ``fn`` (a worker call that reads and writes the plain keys) on agent ``node.agent_group``'s columns."""
        prefix = self._agent_prefix(node)
        if not prefix:
            return fn(batch)
        view = Batch({k[len(prefix):]: v for k, v in batch.tensors.items() if k.startswith(prefix)},
                     batch.non_tensors, dict(batch.meta))
        out = fn(view)
        for k, v in out.tensors.items():
            batch.tensors[prefix + k] = v
        for k, v in out.non_tensors.items():
            if k not in batch.non_tensors:
                batch.non_tensors[k] = v
        batch.meta.update(out.meta)
        return batch

    def _train_cycle_skips(self, node: Optional[Node]) -> bool:
        """``agent_options.train_cycle: c``: the agents take turns being trained, c steps each
        (reference dagworker.py:325-336)."""
        cycle = self._agent_option(node, "train_cycle")
        if not cycle or not self._multi_agent:
            return False
        return (self.global_steps // int(cycle)) % len(self._agent_ids) != self._agent_ids.index(node.agent_group)

    # ================================================================================================
    # node handlers
    # ================================================================================================
    def generate(self, batch: Batch, config=None, **kwargs) -> NodeOutput:
        node = kwargs.get("cur_node")
        batch.meta.update({"eos_token_id": getattr(self.tokenizer, "eos_token_id", None),
                           "pad_token_id": getattr(self.tokenizer, "pad_token_id", 0) or 0,
                           "global_steps": self.global_steps})
        batch.meta.update(self.rollout_meta_overrides)
        if self._multi_agent:
            if batch.meta.get("multi_agent"):
                return NodeOutput(batch, {})          # the first rollout node already ran the joint loop
            out = self.multi_agent_loop.generate_sequence(batch.to("cpu")).to(self.device)
            # turns used per sample = chronological index of its latest turn + 1 (rows are latest turn first)
            first_rows = {}
            for rid, st in zip(out.non_tensors["request_id"], out.non_tensors["traj_step"]):
                first_rows.setdefault(rid, int(st) + 1)
            turns = list(first_rows.values())
            scores = [float(x) for x in out.non_tensors["env_score"]]
            return NodeOutput(out, {"perf/rollout_output_tokens_total": float(out.meta.get("total_output_tokens", 0)),
                                    "num_turns/max": float(max(turns)), "num_turns/mean": sum(turns) / len(turns),
                                    "env/score_mean": sum(scores) / max(len(scores), 1)})
        worker = self._arr(node)
        r = self.config.actor_rollout_ref.rollout
        if (r.multi_turn.enable or r.mode == "async") and worker.engine is not None \
                and getattr(worker, "embodied_rollout", None) is None:
            out = self._generate_with_agent_loops(worker, batch).to(self.device)
        else:
            out = worker.generate_sequences(batch.to(self.device))
        metrics = {"perf/rollout_output_tokens_total": float(out.meta.get("total_output_tokens", 0))}
        if "num_turns" in out.non_tensors:
            turns = [float(t) for t in out.non_tensors["num_turns"]]
            metrics.update({"num_turns/mean": sum(turns) / max(len(turns), 1), "num_turns/max": max(turns, default=0.0)})
        return NodeOutput(out, metrics)

    def _generate_with_agent_loops(self, worker, batch: Batch) -> Batch:
        """Asynchronous rollout: one agent loop per sample (single-turn, tool calling, user interactions) against
        the in-process request server that batches their requests into engine calls
        (reference: dagworker generate -> AgentLoopManager, siirl/execution/rollout_flow/multiturn/agent_loop)."""
        import time as _time
        if getattr(self, "_agent_loops", None) is None:
            from ..engine.rollout.async_server import make_async_server
            from ..execution.rollout_flow.multiturn.agent_loop.agent_loop import AgentLoopManager
            from ..execution.rollout_flow.multiturn.tools.tool_registry import initialize_tools_from_config
            mt = self.config.actor_rollout_ref.rollout.multi_turn
            tools = initialize_tools_from_config(mt.tool_config_path) if mt.tool_config_path else []
            interactions = {}
            if mt.interaction_config_path:
                from ..execution.rollout_flow.multiturn.interactions.base import initialize_interactions_from_config
                interactions = initialize_interactions_from_config(mt.interaction_config_path)
            server = make_async_server(worker.engine, self.tokenizer, self.config.actor_rollout_ref.rollout.agent)
            self._agent_loops = AgentLoopManager(self.config, [server], self.tokenizer, tools, interactions)
        t0 = _time.time()
        worker._full_weights(True)
        worker.engine.wake_up()
        r = self.config.actor_rollout_ref.rollout
        validate = bool(batch.meta.get("validate", False))
        sp = {"seed": (r.seed + 7919 * self.global_steps + 104729 * self._rank) & 0x7FFFFFFF}
        if validate or not r.do_sample:
            sp["temperature"] = r.val_kwargs.temperature if validate else 0.0
        out = self._agent_loops.generate_sequences(batch.to("cpu"), sp)
        if r.free_cache_engine:
            worker.engine.sleep()
            worker._full_weights(False)
        out.meta["timing_generate_s"] = _time.time() - t0
        out.meta["total_output_tokens"] = int(out["attention_mask"][:, -out["responses"].shape[1]:].sum())
        return out

    def compute_reward(self, batch: Batch, config=None, **kwargs) -> NodeOutput:
        metrics: Dict[str, float] = {}
        if self.config.reward_model.enable and "reward_0" in self.workers:
            batch = self.workers["reward_0"].compute_rm_score(batch)
        if self._multi_agent and self.config.actor_rollout_ref.rollout.agent.rewards_with_env \
                and "env_score" in batch.non_tensors:
            # the environment already judged every turn: its score sits on the last response token of the last agent
            m = batch["response_mask"].float()
            last = (m.cumsum(-1) == m.sum(-1, keepdim=True)).float() * m
            score = torch.tensor([float(x) for x in batch.non_tensors["env_score"]], device=m.device)
            reward_tensor, extra = last * score[:, None], {}
        else:
            reward_tensor, extra = guarded_compute_reward(batch, self.reward_fn)
        batch["token_level_scores"] = reward_tensor.to(batch["responses"].device)
        for k, v in (extra or {}).items():
            if isinstance(v, list) and len(v) == batch.batch_size:
                batch.set_non_tensor(k, v)
                if k == "acc":
                    batch["acc"] = torch.tensor([float(x) for x in v])
        if "reward_error" in (extra or {}):
            metrics["reward/errors_total"] = 1.0
        seq = batch["token_level_scores"].sum(-1)
        batch["seq_reward"] = seq
        batch["seq_final_reward"] = seq
        if "acc" not in batch:
            batch["acc"] = (seq > 0).float()
        batch.meta["global_token_num"] = batch["attention_mask"].sum(-1).tolist()
        return NodeOutput(batch, metrics)

    def _sampling_temperature(self, batch: Batch) -> float:
        arr = self.config.actor_rollout_ref
        return arr.embodied.temperature if batch.meta.get("embodied") else arr.rollout.temperature

    def compute_old_log_prob(self, batch: Batch, config=None, **kwargs) -> NodeOutput:
        batch.meta["temperature"] = self._sampling_temperature(batch)
        node = kwargs.get("cur_node")
        out = self._on_agent_view(batch, node, self._arr(node).compute_log_prob)
        metrics = dict(out.meta.pop("metrics", {}))
        out.pop(self._agent_prefix(node) + "entropys")
        if self._agent_prefix(node):
            return NodeOutput(out, {f"agent_{node.agent_group}_{k}": v for k, v in metrics.items()})
        alg = self.config.algorithm
        if alg.rollout_is and "rollout_log_probs" in out and out["responses"].dim() == 2:
            # the engine's sampling distribution differs slightly from the trainer's recomputation (kernel numerics,
            # truncation): weight every token by min(pi_train / pi_rollout, threshold), consumed by the policy loss
            # as ``rollout_is_weights`` (reference: dp_actor.py:444-465 expects them from the trainer)
            m = out["response_mask"].to(out["old_log_probs"].device).float()
            ratio = torch.exp((out["old_log_probs"] - out["rollout_log_probs"].to(out["old_log_probs"].device))
                              .clamp(-20, 20))
            out["rollout_is_weights"] = ratio.clamp(max=alg.rollout_is_threshold) * m
            denom = m.sum().clamp(min=1)
            metrics["actor/rollout_is_ratio_mean"] = float((ratio * m).sum() / denom)
            metrics["actor/rollout_is_truncated_frac"] = float(((ratio > alg.rollout_is_threshold).float() * m).sum()
                                                               / denom)
        return NodeOutput(out, metrics)

    def compute_ref_log_prob(self, batch: Batch, config=None, **kwargs) -> NodeOutput:
        a = self.config.actor_rollout_ref.actor
        if not (a.use_kl_loss or self.config.algorithm.use_kl_in_reward):
            return NodeOutput(batch, {})
        batch.meta["temperature"] = self._sampling_temperature(batch)
        node = kwargs.get("cur_node")
        return NodeOutput(self._on_agent_view(batch, node, self._arr(node).compute_ref_log_prob), {})

    def compute_value(self, batch: Batch, config=None, **kwargs) -> NodeOutput:
        node = kwargs.get("cur_node")
        critic = self.workers[f"critic_{node.agent_group if node else 0}"]
        return NodeOutput(self._on_agent_view(batch, node, critic.compute_values), {})

    def compute_advantage(self, batch: Batch, config=None, **kwargs) -> NodeOutput:
        alg = self.config.algorithm
        metrics: Dict[str, float] = {}
        if "response_mask" not in batch:
            batch["response_mask"] = core_algos.compute_response_mask(batch)
        if alg.use_kl_in_reward and "old_log_probs" in batch and "ref_log_prob" in batch:
            batch, kl_metrics = core_algos.apply_kl_penalty(batch, self.kl_ctrl_in_reward, alg.kl_penalty)
            metrics.update(kl_metrics)
        else:
            batch["token_level_rewards"] = batch["token_level_scores"]
        extra_kw: Dict[str, Any] = {}
        if self._multi_agent:
            # only the last agent is scored; the agents before it share that reward (placed on their own last
            # response token) or get none (reference dagworker.py:586-617)
            pre_ids = self._agent_ids[:-1]
            extra_kw["agent_group_ids"] = pre_ids
            seq = batch["token_level_rewards"].sum(-1)
            for g in pre_ids:
                key = f"agent_group_{g}_token_level_rewards"
                if key not in batch.tensors:
                    m = batch[f"agent_group_{g}_response_mask"].float()
                    last = (m.cumsum(-1) == m.sum(-1, keepdim=True)).float() * m
                    share = seq.to(m.device)[:, None] if alg.share_reward_in_agent else 0.0
                    batch[key] = last * share
                batch[f"agent_group_{g}_token_level_scores"] = batch[key].clone()
        batch = core_algos.compute_advantage(
            batch, alg.adv_estimator, gamma=alg.gamma, lam=alg.lam, **extra_kw,
            norm_adv_by_std_in_grpo=alg.norm_adv_by_std_in_grpo, weight_factor_in_cpgd=alg.weight_factor_in_cpgd,
            use_pf_ppo=alg.use_pf_ppo, pf_ppo_reweight_method=alg.pf_ppo.get("reweight_method", "pow"),
            pf_ppo_weight_pow=alg.pf_ppo.get("weight_pow", 2.0),
            multi_turn=self.config.actor_rollout_ref.rollout.multi_turn.enable)
        return NodeOutput(batch, metrics)

    def train_critic(self, batch: Batch, config=None, **kwargs) -> NodeOutput:
        node = kwargs.get("cur_node")
        if self._train_cycle_skips(node):
            return NodeOutput(batch, {})
        critic = self.workers[f"critic_{node.agent_group if node else 0}"]
        metrics: Dict[str, float] = {}
        self._on_agent_view(batch, node, lambda b: (metrics.update(critic.update_critic(b)), b)[1])
        return NodeOutput(batch, self._agent_metrics(node, metrics))

    def train_actor(self, batch: Batch, config=None, **kwargs) -> NodeOutput:
        if self.config.trainer.critic_warmup > self.global_steps:
            return NodeOutput(batch, {})
        node = kwargs.get("cur_node")
        if self._train_cycle_skips(node):
            return NodeOutput(batch, {})
        batch.meta["temperature"] = self._sampling_temperature(batch)
        metrics: Dict[str, float] = {}
        self._on_agent_view(batch, node, lambda b: (metrics.update(self._arr(node).update_actor(b)), b)[1])
        return NodeOutput(batch, self._agent_metrics(node, metrics))

    def _agent_metrics(self, node: Optional[Node], metrics: Dict[str, float]) -> Dict[str, float]:
        """With several agents every model node's metrics carry ``agent_{k}_`` so that they do not overwrite
        each other (reference dag_utils.py:121-132)."""
        if not self._multi_agent or node is None:
            return metrics
        return {f"agent_{node.agent_group}_{k}": v for k, v in metrics.items()}

    # ================================================================================================
    # data movement between nodes
    # ================================================================================================
    def put_data_to_buffers(self, key: str, data: Batch, source_dp_size: int, dest_dp_size: int,
                            enforce_buffer: bool = False, tp_rank: int = 0) -> None:
        if source_dp_size == dest_dp_size and not enforce_buffer:
            self.internal_data_cache[key] = data
            return
        if tp_rank != 0:
            return      # tensor-parallel peers hold identical data: only the first rank of a TP group publishes
        infos, samples = Dict2Samples(data, key=key)
        for info in infos:
            info.dict_info["source_dp_size"] = source_dp_size
        self.data_coordinator.put_batch(infos, samples, caller_node_id=key)

    def get_data_from_buffers(self, key: str, cur_dp_size: int, cur_dp_rank: int,
                              batch_size: Optional[int] = None) -> Optional[Batch]:
        if key in self.internal_data_cache:
            return self.internal_data_cache.pop(key)
        n = self.config.actor_rollout_ref.rollout.n
        adjusted = batch_size or (self.config.data.train_batch_size * n // max(cur_dp_size, 1))
        flt = lambda info: info.dict_info.get("key") == key  # noqa: E731
        samples = self.data_coordinator.get_batch_collective(adjusted, cur_dp_rank, cur_dp_size, flt) \
            if self._dist and self.world_size > 1 else self.data_coordinator.get_batch(adjusted, 0, flt, None)
        if not samples:
            return None
        return Samples2Dict(samples).to(self.device)

    # ================================================================================================
    # training loop
    # ================================================================================================
    def execute_task_graph(self) -> List[Dict[str, float]]:
        if not self._initialized:
            self.init_graph()
        try:
            self._run_training_loop()
            self.checkpoint_manager.finalize()      # publish a checkpoint that was still being written
        finally:
            if self.tracker is not None:
                self.tracker.finish()
        return self.history

    def _maybe_inject_fault(self, node_id: str) -> None:
        for f in self.config.fault.inject or []:
            if int(f.get("rank", -1)) == self._rank and int(f.get("step", -1)) == self.global_steps \
                    and f.get("node", node_id) == node_id and not f.get("_done") \
                    and int(f.get("restart", 0)) == int(os.environ.get("SIIRL_RESTART_COUNT", "0")):
                f["_done"] = True
                kind = f.get("kind", "raise")
                if kind == "drop_heartbeat":
                    # play a hung rank: stop reporting and stall; the launcher's watchdog has to end the job
                    from ..execution.scheduler.launch import stop_heartbeat
                    stop_heartbeat()
                    time.sleep(float(f.get("seconds", 60.0)))
                if kind == "raise":
                    raise RuntimeError(f"injected fault at rank {self._rank} step {self.global_steps} node {node_id}")
                if kind == "exit":
                    sys.stdout.flush()
                    os._exit(int(f.get("code", 17)))
                if kind == "sleep":
                    time.sleep(float(f.get("seconds", 5.0)))

    def _import_external_libs(self) -> None:
        """``model.external_lib``: modules to import before models and rewards are built, so that user code can
        register architecture presets, reward scorers or pipelines (reference: ``import_external_libs``,
        siirl/utils/extras/import_utils.py, called from the workers' ``init_model``)."""
        import importlib
        libs = self.config.actor_rollout_ref.model.external_lib
        if not libs:
            return
        for name in ([libs] if isinstance(libs, str) else list(libs)):
            for mod in str(name).split(","):
                if mod.strip():
                    importlib.import_module(mod.strip())

    def _start_metric_worker(self) -> None:
        """``trainer.async_metrics``: a collector thread on rank 0 merges the ranks' step metrics out of band."""
        self._metric_client = self._metric_worker = None
        if not getattr(self.config.trainer, "async_metrics", False) or self.world_size <= 1:
            return
        from ..execution.metric_worker.metric_worker import MetricClient, MetricWorker, default_store
        store = default_store()
        if store is None:
            return
        self._metric_client = MetricClient(store, self._rank)
        if self._rank == 0:
            def sink(merged, step):
                merged = dict(merged)
                self._async_history.append(merged)
                if self.tracker is not None:
                    self.tracker.log(merged, step=step)
            self._async_history = []
            self._metric_worker = MetricWorker(store, self.world_size, sink)

    def _run_training_loop(self) -> None:
        self._start_metric_worker()
        try:
            self._training_loop_body()
        except BaseException:
            if getattr(self, "_metric_worker", None) is not None:
                try:                                 # the loop failed: do not wait long for ranks that may be gone
                    self._metric_worker.close(timeout_s=5.0)
                except Exception:  # noqa: BLE001
                    pass
                self._metric_worker = None
            raise
        finally:
            if getattr(self, "_metric_worker", None) is not None:
                self._metric_worker.close()          # deliver what is outstanding to the loggers
                self._metric_worker = None

    def _training_loop_body(self) -> None:
        t = self.config.trainer
        if t.val_before_train and self.validator.enabled and self.global_steps == 0:
            val = self.validator.validate()
            if self._rank == 0 and val and self.tracker:
                self.tracker.log(val, step=0)
            if t.val_only:
                return
        start_step = self.global_steps
        per_epoch = self.dataloader.num_train_batches
        for epoch in range(t.total_epochs):
            for batch_idx in range(per_epoch):
                step_index = epoch * per_epoch + batch_idx
                if step_index < start_step:
                    continue  # already consumed before the checkpoint we resumed from
                if self.global_steps >= self.total_training_steps:
                    return
                self.profiler.start_step(self.global_steps)
                metrics = self._run_training_step(epoch, batch_idx)
                trace = self.profiler.stop_step(self.global_steps)
                if trace and self._rank == 0:
                    print(f"[siirl_b200] profiler trace of step {self.global_steps}: {trace}", file=sys.stderr)
                if metrics is None:
                    continue
                self.global_steps += 1
                is_last = self.global_steps >= self.total_training_steps
                if self.validator.enabled and t.test_freq > 0 and (is_last or self.global_steps % t.test_freq == 0):
                    metrics.update(self.validator.validate() or {})
                if t.save_freq > 0 and (is_last or self.global_steps % t.save_freq == 0):
                    with _Timer("save_checkpoint", self.timing_raw, False):
                        self.checkpoint_manager.save_checkpoint(self.global_steps)
                self.history.append(metrics)
                if getattr(self, "_metric_client", None) is not None:
                    # the step's own metrics reach the loggers through the collector thread; what was added after
                    # the step (validation) is logged here
                    late = {k: v for k, v in metrics.items() if k not in self._posted_keys}
                    if self._rank == 0 and self.tracker is not None and late:
                        self.tracker.log(late, step=self.global_steps)
                elif self._rank == 0 and self.tracker is not None:
                    self.tracker.log(metrics, step=self.global_steps)

    def train_step(self, epoch: int = 0, batch_idx: int = 0) -> Optional[Dict[str, float]]:
        """One training step outside ``execute_task_graph`` (benchmarks, notebooks, tests): next dataloader batch ->
        host-to-device copy -> DAG walk -> metrics on the host.  Returns ``None`` when the step produced too few
        usable samples (DAPO) and has to be repeated with another generation batch."""
        if not self._initialized:
            self.init_graph()
        metrics = self._run_training_step(epoch, batch_idx)
        if metrics is not None:
            self.global_steps += 1
            self.history.append(metrics)
        return metrics

    def _check_kernel_status(self) -> None:
        """Every bounded device-side wait (mbarrier, flag, peer) reports through one status word per GPU; a step whose
        kernels gave up a wait has worked on incomplete data and must not be accepted.  Raises ``KernelStatusError``,
        which ends the rank with a non-zero code so that the launcher's fail-fast / auto-restart takes over."""
        if self.device.type != "cuda":
            return
        from ..ops import lib as _lib
        _lib.check_status(self.device)

    def _run_training_step(self, epoch: int, batch_idx: int) -> Optional[Dict[str, float]]:
        self.timing_raw = {}
        metrics: Dict[str, float] = {}
        n = self.config.actor_rollout_ref.rollout.n
        with _Timer("step", self.timing_raw, True):
            with _Timer("data_loading", self.timing_raw, False):
                batch = self.dataloader.run(epoch=epoch)
                self.last_h2d_bytes = 0
                # group ids unique over ranks and over the generation batches of this run: (draw, rank, prompt)
                self._uid_draw = getattr(self, "_uid_draw", -1) + 1
                batch = preprocess_dataloader(batch, n, uid_offset=(self._uid_draw * max(self.world_size, 1)
                                                                    + self._rank) * batch.batch_size)
                if self.device.type == "cuda":
                    batch = batch.pin_memory()
                    self.last_h2d_bytes = batch.nbytes()
                batch = batch.to(self.device)
            order = self.taskgraph.get_topological_sort()
            queue = deque(order)
            cur: Optional[Batch] = batch
            prev_dp = None
            while queue:
                node = self.taskgraph.nodes[queue.popleft()]
                dp_size, dp_rank, tp_rank, tp_size = self._get_node_dp_info(node)
                if prev_dp is not None:
                    got = self.get_data_from_buffers(node.node_id, dp_size, dp_rank)
                    if got is None:
                        # not enough filtered samples yet (DAPO): roll out another generation batch
                        self._dapo_gen_batches += 1
                        limit = self.config.algorithm.filter_groups.max_num_gen_batches
                        if limit > 0 and self._dapo_gen_batches >= limit:
                            raise RuntimeError(f"{self._dapo_gen_batches} generation batches gave too few usable "
                                               f"groups; check the reward or raise filter_groups.max_num_gen_batches")
                        return None
                    cur = got
                self._maybe_inject_fault(node.node_id)
                nvtx = mark_start_range(node.node_id) if (self.enable_perf or self.profiler.prof is not None) else None
                with _Timer(node.node_id, self.timing_raw, self.enable_perf or node.node_type in (
                        NodeType.MODEL_TRAIN, NodeType.MODEL_INFERENCE)):
                    out = node.run(batch=cur, config=self.config, process_group=self._node_group(node),
                                   agent_group=node.agent_group, cur_tp_rank=tp_rank, tp_size=tp_size, cur_node=node,
                                   _dag_worker_instance=self)
                mark_end_range(nvtx)
                if not isinstance(out, NodeOutput):
                    out = NodeOutput(out if out is not None else cur, {})
                metrics.update(out.metrics or {})
                cur = out.batch
                if cur is None or cur.batch_size == 0:
                    self._dapo_gen_batches += 1
                    return None
                nxt = self.taskgraph.get_dependents(node.node_id)
                enforce = node.node_role == NodeRole.DYNAMIC_SAMPLING or (
                    node.node_role == NodeRole.ROLLOUT and self._dist and self.world_size > 1
                    and bool(getattr(self.config.data, "rebalance_after_rollout", False)))
                for child in nxt:
                    cdp = self._get_node_dp_info(child)[0]
                    self.put_data_to_buffers(child.node_id, cur, dp_size, cdp, enforce_buffer=enforce, tp_rank=tp_rank)
                prev_dp = dp_size
            self._dapo_gen_batches = 0
        self._check_kernel_status()
        final = cur
        use_critic = self.config.algorithm.adv_estimator in ("gae", "gae_marft")
        keep = [k for k in ("response_mask", "attention_mask", "token_level_scores", "token_level_rewards",
                            "advantages", "returns", "values") if k in final.tensors]
        cpu_view = Batch({k: final.tensors[k] for k in keep}, None, final.meta).to("cpu")
        self.last_step_tokens = int(cpu_view["attention_mask"].sum())
        self.last_d2h_bytes = cpu_view.nbytes() + 8 * len(metrics) + sum(
            getattr(w, "engine", None).stats.pop("d2h_bytes", 0) for w in self.workers.values()
            if getattr(w, "engine", None) is not None)
        metrics.update(compute_data_metric(cpu_view, use_critic))
        metrics.update(compute_timing_metrics(cpu_view, self.timing_raw))
        metrics.update(compute_throughput_metrics(cpu_view, self.timing_raw, 1))
        numeric = {k: float(v) for k, v in metrics.items() if isinstance(v, (int, float))}
        if self.enable_perf:
            # every rank's own numbers side by side, before they are reduced (reference: dag_utils.py:684-772)
            model = os.path.basename(os.path.normpath(self.config.actor_rollout_ref.model.path or
                                                      self.config.actor_rollout_ref.model.arch_preset or "model"))
            if getattr(self, "_perf_dir", None) is None:
                self._perf_dir = os.path.join("performance_logs", model, time.strftime("%Y-%m-%d-%H-%M-%S"))
            write_rank_performance_csv(numeric, self.global_steps + 1, self._rank, self.world_size, self._perf_dir)
        if getattr(self, "_metric_client", None) is not None:
            # out-of-band: post and carry on; this rank keeps its own numbers, rank 0's collector merges all ranks'
            step = self.global_steps + 1
            self._metric_client.submit_metric(numeric, step)
            if self._metric_worker is not None:
                self._metric_worker.expect(step, {"training/global_step": step, "training/epoch": epoch})
            metrics = dict(numeric)
            self._posted_keys = set(metrics) | {"training/global_step", "training/epoch"}
        else:
            metrics = reduce_metrics_across_ranks(numeric)
        metrics["training/global_step"] = self.global_steps + 1
        metrics["training/epoch"] = epoch
        if self._rank == 0 and self.config.trainer.logger and "console" in list(self.config.trainer.logger):
            print(format_core_performance_metrics(metrics, self.global_steps + 1, self.enable_perf), flush=True)
        return metrics
