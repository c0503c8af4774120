"""Constants of the DAG worker (reference: siirl/dag_worker/constants.py:25-42)."""


class DAGConstants:
    FSDP_STRATEGIES = ("fsdp", "fsdp2")
    MEGATRON_STRATEGIES = ("megatron",)
    NATIVE_STRATEGIES = ("native", "fsdp", "fsdp2", "megatron")  # every name maps to the native sharded runtime
    METRIC_GROUP_ORDER = ("step", "training", "actor", "critic", "perf", "response_length", "prompt_length",
                          "timing_s", "timing_per_token_ms", "val-core", "val-aux", "dapo_sampling", "other")
    WORKER_ROLE_KEYS = ("actor", "rollout", "ref", "critic", "reward")
