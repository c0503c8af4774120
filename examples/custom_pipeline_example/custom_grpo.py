"""A user-defined pipeline: GRPO without the reference-policy node, selected with
``dag.custom_pipeline_fn=examples.custom_pipeline_example.custom_grpo:grpo_without_reference``."""
from siirl_b200.execution.dag.node import NodeRole, NodeType
from siirl_b200.execution.dag.pipeline import Pipeline

_W = "siirl_b200.dag_worker.dagworker:DAGWorker"


def grpo_without_reference():
    p = Pipeline("grpo_no_ref", "GRPO without KL to a reference policy")
    p.add_node("rollout_actor", f"{_W}.generate", [], node_type=NodeType.MODEL_INFERENCE, node_role=NodeRole.ROLLOUT)
    p.add_node("function_reward", f"{_W}.compute_reward", ["rollout_actor"], node_type=NodeType.COMPUTE,
               node_role=NodeRole.REWARD)
    p.add_node("calculate_advantages", f"{_W}.compute_advantage", ["function_reward"], node_type=NodeType.COMPUTE,
               node_role=NodeRole.ADVANTAGE)
    p.add_node("actor_old_log_prob", f"{_W}.compute_old_log_prob", ["calculate_advantages"],
               node_type=NodeType.MODEL_TRAIN, node_role=NodeRole.ACTOR, only_forward_compute=True)
    p.add_node("actor_train", f"{_W}.train_actor", ["actor_old_log_prob"], node_type=NodeType.MODEL_TRAIN,
               node_role=NodeRole.ACTOR)
    return p.build()
