"""Built-in workflows.  Node ids and ordering are the reference's
(siirl/execution/dag/builtin_pipelines.py:27-297) so configs, logs and checkpoints line up:

* GRPO: rollout_actor -> function_reward -> calculate_advantages -> actor_old_log_prob (forward only)
  -> reference_log_prob -> actor_train
* PPO : ... -> compute_value before the advantages, critic_train before actor_train
* DAPO: GRPO plus a dynamic_sampling filter node after the reward
* embodied SRPO: environment rollout, embodied reward/filter, GRPO-style update
"""
from __future__ import annotations

from .node import NodeRole, NodeType
from .pipeline import Pipeline
from .task_graph import TaskGraph

_W = "siirl_b200.dag_worker.dagworker:DAGWorker"


def grpo_pipeline() -> TaskGraph:
    p = Pipeline("grpo_training_pipeline", "Standard GRPO workflow")
    p.add_node("rollout_actor", f"{_W}.generate", [], node_type=NodeType.MODEL_INFERENCE,
               node_role=NodeRole.ROLLOUT)
    p.add_node("function_reward", f"{_W}.compute_reward", ["rollout_actor"], node_type=NodeType.COMPUTE,
               node_role=NodeRole.REWARD)
    p.add_node("calculate_advantages", f"{_W}.compute_advantage", ["function_reward"],
               node_type=NodeType.COMPUTE, node_role=NodeRole.ADVANTAGE)
    p.add_node("actor_old_log_prob", f"{_W}.compute_old_log_prob", ["calculate_advantages"],
               node_type=NodeType.MODEL_TRAIN, node_role=NodeRole.ACTOR, only_forward_compute=True)
    p.add_node("reference_log_prob", f"{_W}.compute_ref_log_prob", ["actor_old_log_prob"],
               node_type=NodeType.MODEL_TRAIN, node_role=NodeRole.REFERENCE)
    p.add_node("actor_train", f"{_W}.train_actor", ["reference_log_prob"], node_type=NodeType.MODEL_TRAIN,
               node_role=NodeRole.ACTOR)
    return p.build()


def ppo_pipeline() -> TaskGraph:
    p = Pipeline("ppo_training_pipeline", "Standard PPO workflow with a critic")
    p.add_node("rollout_actor", f"{_W}.generate", [], node_type=NodeType.MODEL_INFERENCE,
               node_role=NodeRole.ROLLOUT)
    p.add_node("function_reward", f"{_W}.compute_reward", ["rollout_actor"], node_type=NodeType.COMPUTE,
               node_role=NodeRole.REWARD)
    p.add_node("compute_value", f"{_W}.compute_value", ["function_reward"], node_type=NodeType.MODEL_TRAIN,
               node_role=NodeRole.CRITIC, only_forward_compute=True)
    p.add_node("actor_old_log_prob", f"{_W}.compute_old_log_prob", ["compute_value"],
               node_type=NodeType.MODEL_TRAIN, node_role=NodeRole.ACTOR, only_forward_compute=True)
    p.add_node("reference_log_prob", f"{_W}.compute_ref_log_prob", ["actor_old_log_prob"],
               node_type=NodeType.MODEL_TRAIN, node_role=NodeRole.REFERENCE)
    p.add_node("calculate_advantages", f"{_W}.compute_advantage", ["reference_log_prob"],
               node_type=NodeType.COMPUTE, node_role=NodeRole.ADVANTAGE)
    p.add_node("critic_train", f"{_W}.train_critic", ["calculate_advantages"], node_type=NodeType.MODEL_TRAIN,
               node_role=NodeRole.CRITIC)
    p.add_node("actor_train", f"{_W}.train_actor", ["critic_train"], node_type=NodeType.MODEL_TRAIN,
               node_role=NodeRole.ACTOR)
    return p.build()


def dapo_pipeline() -> TaskGraph:
    p = Pipeline("dapo_training_pipeline", "DAPO workflow with dynamic sampling")
    p.add_node("rollout_actor", f"{_W}.generate", [], node_type=NodeType.MODEL_INFERENCE,
               node_role=NodeRole.ROLLOUT)
    p.add_node("function_reward", f"{_W}.compute_reward", ["rollout_actor"], node_type=NodeType.COMPUTE,
               node_role=NodeRole.REWARD)
    p.add_node("dynamic_sampling", "siirl_b200.user_interface.filter_interface.dapo:dynamic_sampling",
               ["function_reward"], node_type=NodeType.COMPUTE, node_role=NodeRole.DYNAMIC_SAMPLING)
    p.add_node("calculate_advantages", f"{_W}.compute_advantage", ["dynamic_sampling"],
               node_type=NodeType.COMPUTE, node_role=NodeRole.ADVANTAGE)
    p.add_node("actor_old_log_prob", f"{_W}.compute_old_log_prob", ["calculate_advantages"],
               node_type=NodeType.MODEL_TRAIN, node_role=NodeRole.ACTOR, only_forward_compute=True)
    p.add_node("reference_log_prob", f"{_W}.compute_ref_log_prob", ["actor_old_log_prob"],
               node_type=NodeType.MODEL_TRAIN, node_role=NodeRole.REFERENCE)
    p.add_node("actor_train", f"{_W}.train_actor", ["reference_log_prob"], node_type=NodeType.MODEL_TRAIN,
               node_role=NodeRole.ACTOR)
    return p.build()


def embodied_srpo_pipeline() -> TaskGraph:
    p = Pipeline("embodied_srpo_pipeline", "Embodied SRPO workflow (environment rollout + GRPO update)")
    p.add_node("rollout_actor", f"{_W}.generate", [], node_type=NodeType.MODEL_INFERENCE,
               node_role=NodeRole.ROLLOUT)
    p.add_node("dynamic_sampling", "siirl_b200.user_interface.filter_interface.embodied:embodied_local_rank_sampling",
               ["rollout_actor"], node_type=NodeType.COMPUTE, node_role=NodeRole.DYNAMIC_SAMPLING)
    p.add_node("function_reward", f"{_W}.compute_reward", ["dynamic_sampling"], node_type=NodeType.COMPUTE,
               node_role=NodeRole.REWARD)
    p.add_node("calculate_advantages", f"{_W}.compute_advantage", ["function_reward"],
               node_type=NodeType.COMPUTE, node_role=NodeRole.ADVANTAGE)
    p.add_node("actor_old_log_prob", f"{_W}.compute_old_log_prob", ["calculate_advantages"],
               node_type=NodeType.MODEL_TRAIN, node_role=NodeRole.ACTOR, only_forward_compute=True)
    p.add_node("reference_log_prob", f"{_W}.compute_ref_log_prob", ["actor_old_log_prob"],
               node_type=NodeType.MODEL_TRAIN, node_role=NodeRole.REFERENCE)
    p.add_node("actor_train", f"{_W}.train_actor", ["reference_log_prob"], node_type=NodeType.MODEL_TRAIN,
               node_role=NodeRole.ACTOR)
    return p.build()


BUILTIN_PIPELINES = {
    "grpo": grpo_pipeline,
    "ppo": ppo_pipeline,
    "dapo": dapo_pipeline,
    "embodied_srpo": embodied_srpo_pipeline,
}
