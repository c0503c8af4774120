"""Typed configuration tree.  The dotted key names are the reference's public flag surface
(siirl/params/training_args.py:29-102, model_args.py:22-690, data_args.py:23-150, dag_args.py:20-36,
profiler_args.py:20-40, embodied_args.py:19-146) so its launch scripts keep working with only the
module name changed.  Keys that only made sense for FSDP/Megatron/vLLM internals are accepted and
mapped onto this framework's own runtime (see ``siirl_b200.params.parser`` for the loader).
"""
from __future__ import annotations

from dataclasses import dataclass, field, fields, is_dataclass
from typing import Any, Dict, List, Optional


def _dc(cls):
    return field(default_factory=cls)


@dataclass
class MixedPrecisionArguments:
    param_dtype: str = "bfloat16"
    reduce_dtype: str = "float32"
    buffer_dtype: str = "float32"
    keep_low_precision_grads: bool = False
    cast_forward_inputs: bool = False
    cast_root_forward_inputs: bool = True


@dataclass
class FSDPArguments:
    """Sharded-data-parallel knobs.  ``fsdp_size`` = size of the shard group (-1: whole DP group)."""
    wrap_policy: Dict[str, Any] = field(default_factory=dict)
    param_offload: bool = False
    optimizer_offload: bool = False
    fsdp_size: int = -1
    model_dtype: str = "bfloat16"
    mixed_precision: MixedPrecisionArguments = _dc(MixedPrecisionArguments)
    # native runtime: "zero2" keeps bf16 params replicated and shards grads/master/Adam state;
    # "zero3" also shards the bf16 params and gathers them inside the consuming GEMM.
    sharding: str = "zero2"


@dataclass
class MegatronArguments:
    tensor_model_parallel_size: int = 1
    pipeline_model_parallel_size: int = 1
    context_parallel_size: int = 1
    # chunk assignment of ring attention: "zigzag" (rank r holds chunks r and 2n-1-r: equal causal work per rank)
    # or "contiguous" (rank r holds chunk r and does r+1 blocks)
    context_parallel_layout: str = "zigzag"
    expert_model_parallel_size: int = 1
    expert_tensor_parallel_size: int = 1
    virtual_pipeline_model_parallel_size: Optional[int] = None
    sequence_parallel: bool = False
    use_distributed_optimizer: bool = True
    param_dtype: str = "bfloat16"
    seed: int = 1
    param_offload: bool = True
    grad_offload: bool = False
    optimizer_offload: bool = False
    extra: Dict[str, Any] = field(default_factory=dict)
    override_transformer_config: Dict[str, Any] = field(default_factory=dict)
    use_dist_checkpointing: bool = False
    dist_checkpointing_path: str = ""
    override_ddp_config: Dict[str, Any] = field(default_factory=dict)
    use_mbridge: bool = False


@dataclass
class OptimizerArguments:
    lr: float = 1e-6
    lr_warmup_steps_ratio: float = 0.0
    min_lr: float = 0.0
    min_lr_ratio: Optional[float] = 0.0
    warmup_style: str = "constant"
    lr_warmup_init: float = 0.0
    lr_decay_steps: Optional[int] = None
    lr_decay_style: str = "linear"
    weight_decay_incr_style: str = "constant"
    lr_wsd_decay_style: str = "exponential"
    lr_wsd_decay_steps: Optional[int] = None
    use_checkpoint_opt_param_scheduler: bool = False
    total_training_steps: int = 0
    betas: tuple = (0.9, 0.999)
    weight_decay: float = 1e-2
    lr_warmup_steps: int = -1
    clip_grad: float = 1.0
    num_cycles: float = 0.5
    override_optimizer_config: Optional[dict] = None


@dataclass
class ProcessorArguments:
    image_max_pixels: int = 768 * 768
    image_min_pixels: int = 32 * 32
    video_max_pixels: int = 256 * 256
    video_min_pixels: int = 16 * 16
    video_fps: float = 2.0
    video_maxlen: int = 128


@dataclass
class ModelArguments(ProcessorArguments):
    path: str = "~/models/deepseek-llm-7b-chat"
    external_lib: Optional[str] = None
    override_config: Dict[str, Any] = field(default_factory=dict)
    enable_gradient_checkpointing: bool = True
    gradient_checkpointing_kwargs: Dict[str, Any] = field(default_factory=dict)
    use_remove_padding: bool = False
    use_fused_kernels: bool = False
    cache_dir: Optional[str] = None
    model_revision: str = "main"
    trust_remote_code: bool = False
    hf_hub_token: Optional[str] = None
    use_fast_tokenizer: bool = True
    ep_max_tokens: int = 0      # expert parallelism: static per-rank token bound of one forward (0: 8192)
    split_special_tokens: bool = False
    model_max_length: Optional[int] = None
    new_special_tokens: Optional[str] = None
    resize_vocab: bool = False
    use_liger: bool = False
    fsdp_config: FSDPArguments = _dc(FSDPArguments)
    megatron: MegatronArguments = _dc(MegatronArguments)
    input_tokenizer: Optional[str] = None
    rm_tokenizer: Optional[str] = None
    lora_rank: int = 0
    lora_alpha: float = 16
    target_modules: Any = "all-linear"      # "all-linear" or a list of projection names (q_proj, up_proj, ...)
    use_shm: bool = False
    enable_activation_offload: bool = False
    model_type: str = "llm"
    # native additions: build a random-init model from a named architecture preset instead of a
    # checkpoint directory (no network on the build/bench machines)
    arch_preset: Optional[str] = None
    random_init: bool = False


@dataclass
class CheckpointArguments:
    contents: List[str] = field(default_factory=lambda: ["model", "optimizer", "extra"])
    save_contents: List[str] = field(default_factory=lambda: ["model", "optimizer", "extra"])
    load_contents: List[str] = field(default_factory=lambda: ["model", "optimizer", "extra"])
    async_save: bool = False


@dataclass
class PolicyLossArguments:
    loss_mode: str = "vanilla"
    clip_cov_ratio: float = 0.0002
    clip_cov_lb: float = 1.0
    clip_cov_ub: float = 5.0
    kl_cov_ratio: float = 0.0002
    ppo_kl_coef: float = 0.1


@dataclass
class ActorArguments:
    strategy: str = "fsdp"
    ppo_mini_batch_size: int = 256
    ppo_micro_batch_size: Optional[int] = None
    ppo_micro_batch_size_per_gpu: Optional[int] = 1
    use_dynamic_bsz: bool = False
    ppo_max_token_len_per_gpu: int = 16384
    grad_clip: float = 1.0
    clip_ratio: float = 0.2
    clip_ratio_low: float = 0.2
    clip_ratio_high: float = 0.2
    clip_ratio_c: float = 3.0
    entropy_coeff: float = 0.0
    use_kl_loss: bool = False
    kl_loss_coef: float = 0.001
    kl_loss_type: str = "low_var_kl"
    ppo_epochs: int = 1
    shuffle: bool = False
    ulysses_sequence_parallel_size: int = 1
    policy_loss: PolicyLossArguments = _dc(PolicyLossArguments)
    tis_imp_ratio_cap: float = -1
    optim: OptimizerArguments = _dc(OptimizerArguments)
    fsdp_config: FSDPArguments = _dc(FSDPArguments)
    megatron: MegatronArguments = _dc(MegatronArguments)
    use_remove_padding: bool = False
    use_fused_kernels: bool = False
    use_torch_compile: bool = True
    checkpoint: CheckpointArguments = _dc(CheckpointArguments)
    param_offload: bool = False
    grad_offload: bool = False
    optimizer_offload: bool = False
    load_weight: bool = True
    loss_agg_mode: str = "token-mean"
    recompute_old_log_prob: bool = True
    use_cpgd_loss: bool = False
    policy_drift_coeff: float = 0.0
    data_loader_seed: Optional[int] = None
    profile: Dict[str, Any] = field(default_factory=dict)
    entropy_checkpointing: bool = False
    entropy_from_logits_with_chunking: bool = False
    embodied_type: Optional[str] = None
    action_token_len: Optional[int] = None
    action_chunks_len: Optional[int] = None
    traj_mini_batch_size: int = 16


@dataclass
class EvalSamplingArguments:
    top_k: int = -1
    top_p: float = 1.0
    temperature: float = 0
    n: int = 1
    do_sample: bool = False


@dataclass
class LayerNameMapArguments:
    qkv_layer_name: str = "qkv"
    gate_proj_layer_name: str = "linear_fc1.weight"


@dataclass
class MultiTurnArguments:
    use_all_traj: bool = False
    enable: bool = False
    max_assistant_turns: Optional[int] = None
    tool_config_path: Optional[str] = None
    format: str = "hermes"
    max_user_turns: Optional[int] = None
    max_parallel_calls: int = 1
    max_tool_response_length: int = 256
    tool_response_truncate_side: str = "middle"
    interaction_config_path: Optional[str] = None
    completion_callback: Optional[str] = None
    use_inference_chat_template: bool = False
    tokenization_sanity_check_mode: str = "strict"


@dataclass
class CustomAsyncServer:
    path: Optional[str] = None
    name: Optional[str] = None


@dataclass
class AgentArguments:
    agent_name: str = "single_turn_agent"
    num_workers: int = 1
    custom_async_server: Optional[CustomAsyncServer] = None
    train_cycle: Optional[int] = None
    process_path: Optional[str] = None
    pre_process_kwargs: dict = field(default_factory=dict)
    post_process_kwargs: dict = field(default_factory=dict)
    env_path: list = field(default_factory=list)
    obs_with_env: bool = False
    rewards_with_env: bool = False
    share_instance: Optional[int] = None


@dataclass
class EngineArguments:
    vllm: Dict[str, Any] = field(default_factory=dict)
    sglang: Dict[str, Any] = field(default_factory=dict)
    native: Dict[str, Any] = field(default_factory=dict)


@dataclass
class RolloutArguments:
    # "native" is this framework's paged-KV engine; the reference names vllm and sglang map to it, "hf" selects the
    # cache-free engine that generates through the training forward (engine/rollout/recompute_engine.py).
    name: str = "vllm"
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    use_fire_sampling: bool = False
    prompt_length: Optional[int] = None
    response_length: Optional[int] = None
    dtype: str = "bfloat16"
    gpu_memory_utilization: float = 0.5
    ignore_eos: bool = False
    enforce_eager: bool = True
    free_cache_engine: bool = True
    load_format: str = "dummy_dtensor"
    tensor_model_parallel_size: int = 1
    max_num_batched_tokens: int = 8192
    max_model_len: Optional[int] = None
    max_num_seqs: int = 1024
    limit_images: Optional[int] = None
    do_sample: bool = True
    n: int = 1
    log_prob_micro_batch_size: Optional[int] = None
    log_prob_micro_batch_size_per_gpu: Optional[int] = None
    log_prob_max_token_len_per_gpu: int = 16384
    log_prob_use_dynamic_bsz: bool = False
    disable_log_stats: bool = True
    enable_chunked_prefill: bool = True
    enable_prefix_caching: bool = True      # reuse cached full prompt blocks across requests of one rollout phase
    trust_remote_code: bool = True
    val_kwargs: EvalSamplingArguments = _dc(EvalSamplingArguments)
    layer_name_map: LayerNameMapArguments = _dc(LayerNameMapArguments)
    seed: int = 0
    mode: str = "sync"
    kv_borrow_grad_buffer: bool = True     # native: lend the idle fp32 gradient buffer to the KV arena
    multi_turn: MultiTurnArguments = _dc(MultiTurnArguments)
    micro_batch_size: Optional[int] = None
    engine_kwargs: EngineArguments = _dc(EngineArguments)
    calculate_log_probs: bool = False
    agent: AgentArguments = _dc(AgentArguments)
    multi_stage_wake_up: bool = False
    kv_block_size: int = 128


@dataclass
class RefArguments:
    strategy: str = "fsdp"
    fsdp_config: FSDPArguments = _dc(FSDPArguments)
    megatron: MegatronArguments = _dc(MegatronArguments)
    log_prob_micro_batch_size: Optional[int] = None
    log_prob_micro_batch_size_per_gpu: Optional[int] = None
    log_prob_use_dynamic_bsz: bool = False
    log_prob_max_token_len_per_gpu: int = 16384
    ulysses_sequence_parallel_size: int = 1
    use_remove_padding: bool = False
    use_fused_kernels: bool = False
    use_torch_compile: bool = True
    ppo_micro_batch_size: Optional[int] = None
    ppo_micro_batch_size_per_gpu: Optional[int] = None
    param_offload: bool = False
    grad_offload: bool = False
    optimizer_offload: bool = False
    load_weight: bool = True
    profile: Dict[str, Any] = field(default_factory=dict)
    shuffle: bool = False
    data_loader_seed: Optional[int] = None
    recompute_old_log_prob: bool = True
    entropy_checkpointing: bool = False
    entropy_from_logits_with_chunking: bool = False
    embodied_type: Optional[str] = None


@dataclass
class EnvironmentArgs:
    env_type: str = "libero"
    env_name: str = "libero_10"
    num_envs: int = 16
    max_steps: int = 512
    num_trials_per_task: int = 50
    num_steps_wait: int = 10
    model_family: str = "openvla"
    env_kwargs: Dict[str, Any] = field(default_factory=dict)


@dataclass
class EmbodiedArguments:
    env: EnvironmentArgs = _dc(EnvironmentArgs)
    embodied_type: str = "openvla-oft"
    model_path: str = ""
    video_embedding_model_path: str = ""
    action_chunks_len: int = 8
    action_token_len: int = 7
    embedding_img_size: int = 384
    embedding_enable_fp16: bool = True
    embedding_model_class: Optional[str] = None
    embedding_model_offload: bool = False
    num_images_in_input: int = 1
    center_crop: bool = True
    unnorm_key: str = "libero_10_no_noops"
    temperature: float = 1.6
    n_gpus_per_node: int = 8
    policy_image_size: int = 224
    # None: OpenVLA-OFT's one-pass chunk decoding when embodied_type is "openvla-oft" and the policy has the Prismatic
    # backbone, token-by-token decoding otherwise
    parallel_decode: Optional[bool] = None
    video_num_frames: int = 8
    use_video_embedding: bool = True


@dataclass
class EmbodiedSamplingConfig:
    filter_accuracy: bool = False
    accuracy_lower_bound: float = 0.0
    accuracy_upper_bound: float = 1.0
    filter_truncated: bool = False
    oversample_factor: int = 1


@dataclass
class ActorRolloutRefArguments:
    hybrid_engine: bool = True
    model: ModelArguments = _dc(ModelArguments)
    actor: ActorArguments = _dc(ActorArguments)
    ref: RefArguments = _dc(RefArguments)
    rollout: RolloutArguments = _dc(RolloutArguments)
    embodied: EmbodiedArguments = _dc(EmbodiedArguments)


@dataclass
class CriticArguments:
    strategy: str = "fsdp"
    optim: OptimizerArguments = field(default_factory=lambda: OptimizerArguments(lr=1e-5))
    model: ModelArguments = _dc(ModelArguments)
    fsdp_config: FSDPArguments = _dc(FSDPArguments)
    megatron: MegatronArguments = _dc(MegatronArguments)
    ppo_mini_batch_size: int = 256
    ppo_micro_batch_size: Optional[int] = None
    ppo_micro_batch_size_per_gpu: Optional[int] = None
    use_dynamic_bsz: bool = False
    ppo_epochs: int = 1
    shuffle: bool = False
    grad_clip: float = 1.0
    cliprange_value: float = 0.5
    ulysses_sequence_parallel_size: int = 1
    forward_max_token_len_per_gpu: int = 32768
    load_weight: bool = True
    rollout_n: int = 1
    checkpoint: CheckpointArguments = _dc(CheckpointArguments)
    ppo_max_token_len_per_gpu: int = 32768
    loss_agg_mode: str = "token-mean"
    profile: Dict[str, Any] = field(default_factory=dict)
    data_loader_seed: Optional[int] = None


@dataclass
class OverlongBufferArguments:
    enable: bool = False
    len: int = 512
    penalty_factor: float = 1.0
    log: bool = False


@dataclass
class RewardModelArguments:
    enable: bool = False
    strategy: str = "fsdp"
    model: ModelArguments = _dc(ModelArguments)
    fsdp_config: FSDPArguments = _dc(FSDPArguments)
    megatron: MegatronArguments = _dc(MegatronArguments)
    micro_batch_size: Optional[int] = None
    micro_batch_size_per_gpu: Optional[int] = None
    max_length: Optional[int] = None
    ulysses_sequence_parallel_size: int = 1
    use_dynamic_bsz: bool = False
    reward_manager: str = "naive"
    forward_max_token_len_per_gpu: int = 32768
    load_weight: bool = True
    launch_reward_fn_async: bool = False
    reward_kwargs: Dict[str, Any] = field(default_factory=dict)
    sandbox_fusion: Optional[Dict[str, Any]] = None
    overlong_buffer: OverlongBufferArguments = _dc(OverlongBufferArguments)
    profile: Dict[str, Any] = field(default_factory=dict)
    shuffle: bool = False
    data_loader_seed: Optional[int] = None


@dataclass
class KLCtrlArguments:
    type: str = "fixed"
    kl_coef: float = 0.001
    target_kl: Optional[float] = 0.1
    horizon: Optional[float] = 10000


@dataclass
class FilterGroupsArguments:
    enable: bool = False
    metric: str = "seq_final_reward"
    max_num_gen_batches: int = 10


@dataclass
class AlgorithmArguments:
    gamma: float = 1.0
    lam: float = 1.0
    adv_estimator: str = "gae"
    kl_penalty: str = "kl"
    kl_ctrl: KLCtrlArguments = _dc(KLCtrlArguments)
    use_kl_in_reward: bool = False
    share_reward_in_agent: bool = True
    norm_adv_by_std_in_grpo: bool = True
    algorithm_name: str = "grpo"
    weight_factor_in_cpgd: str = "STD_weight"
    workflow_type: str = "default"
    filter_groups: FilterGroupsArguments = _dc(FilterGroupsArguments)
    # native: truncated importance sampling between the rollout engine's and the trainer's log-probs
    rollout_is: bool = False
    rollout_is_threshold: float = 2.0
    use_pf_ppo: bool = False
    pf_ppo: Dict[str, Any] = field(default_factory=dict)
    embodied_sampling: EmbodiedSamplingConfig = _dc(EmbodiedSamplingConfig)


@dataclass
class DataArguments:
    dataset_type: str = "llm"
    tokenizer: Optional[str] = None
    train_files: List[str] = field(default_factory=list)
    val_files: List[str] = field(default_factory=list)
    prompt_key: str = "prompt"
    max_prompt_length: int = 512
    max_response_length: int = 512
    train_batch_size: int = 1024
    gen_batch_size: Optional[int] = None
    val_batch_size: Optional[int] = None
    return_raw_input_ids: bool = False
    return_raw_chat: bool = False
    return_full_prompt: bool = False
    filter_overlong_prompts: bool = False
    shuffle: bool = True
    image_key: str = "images"
    video_key: str = "videos"
    truncation: str = "error"
    train_on_prompt: bool = False
    mask_history: bool = False
    tool_format: Optional[str] = None
    tokenized_path: Optional[str] = None
    dataset_cache_dir: str = "~/.cache/siirl_b200/dataset"
    filter_overlong_prompt: bool = False
    serialize_dataset: bool = False
    streaming: bool = False
    preprocessing_num_workers: Optional[int] = None
    overwrite_cache: bool = False
    preprocessing_batch_size: int = 1000
    mix_strategy: str = "concat"
    interleave_probs: Optional[str] = None
    buffer_size: int = 16384
    cutoff_len: int = 2048
    reward_fn_key: str = "data_source"
    multi_agent: bool = False
    auto_repeat: bool = False
    num_loader_workers: int = 8
    # native addition: after the rollout node the samples go through the data coordinator, which hands every
    # data-parallel rank the same number of whole prompt groups with balanced token counts (ranks that drew long
    # responses otherwise hold up the scoring and training passes of the others)
    rebalance_after_rollout: bool = False
    force_on_the_fly: bool = False
    processor: ProcessorArguments = _dc(ProcessorArguments)
    # native addition: generate a synthetic dataset instead of reading parquet
    # ("arith" = a+b digit prompts, "random" = uniform token ids, "parity" = tiny-model gate)
    synthetic: Optional[str] = None
    synthetic_size: int = 4096
    synthetic_min_prompt: int = 16
    synthetic_max_prompt: int = 32
    synthetic_image_size: int = 448     # side of the random RGB image of the ``vl`` synthetic set


@dataclass
class TrainingArguments:
    total_epochs: int = 30
    total_training_steps: Optional[int] = None
    project_name: str = "siirl_examples"
    experiment_name: str = "gsm8k"
    logger: List[str] = field(default_factory=lambda: ["console"])
    # True: ranks post their step metrics to a collector thread on rank 0 (execution/metric_worker) instead of
    # reducing them with collectives inside the step; the loggers then receive a step's metrics a little later
    async_metrics: bool = False
    log_val_generations: int = 0
    nnodes: int = 1
    n_gpus_per_node: int = 8
    save_freq: int = -1
    resume_mode: str = "auto"
    resume_from_path: Any = False
    test_freq: int = -1
    critic_warmup: int = 0
    default_local_dir: str = "checkpoints/siirl_examples/gsm8k"
    seed: int = 1
    should_log: bool = False
    should_save: bool = True
    val_before_train: bool = True
    default_hdfs_dir: Optional[str] = None
    del_local_ckpt_after_load: bool = False
    val_only: bool = False
    balance_batch: bool = True
    remove_previous_ckpt_in_save: bool = False
    max_actor_ckpt_to_keep: int = 100
    max_critic_ckpt_to_keep: int = 100
    ray_wait_register_center_timeout: int = 300
    validation_data_dir: Optional[str] = None
    rollout_data_dir: Optional[str] = None
    device: Optional[str] = "cuda"


@dataclass
class CustomRewardArguments:
    path: Optional[str] = None
    name: str = "compute_score"
    reward_kwargs: Dict[str, Any] = field(default_factory=dict)


@dataclass
class DagArguments:
    workflow_path: Optional[str] = None
    custom_pipeline_fn: Optional[str] = None
    env_enable: bool = False
    environment_path: Optional[str] = None
    enable_perf: bool = False
    backend_threshold: int = 256


@dataclass
class ProfilerArguments:
    enable: bool = False
    save_path: str = "./prof_data"
    level: str = "level1"
    with_memory: bool = False
    record_shapes: bool = False
    with_npu: bool = True
    with_cpu: bool = False
    with_module: bool = False
    with_stack: bool = False
    analysis: bool = True
    discrete: bool = False
    roles: List[str] = field(default_factory=lambda: ["generate", "compute_reward"])
    all_ranks: bool = False
    ranks: List[int] = field(default_factory=lambda: [0])
    profile_steps: List[int] = field(default_factory=lambda: [0])


@dataclass
class FaultArguments:
    """Host-side fault injection (native addition; the reference is fail-fast only).
    ``inject`` entries look like ``{"rank": 1, "step": 2, "node": "actor_train", "kind": "raise"}``;
    kinds: raise, exit, sleep, drop_heartbeat (the rank stops reporting and stalls for ``seconds``).  An entry fires
    once per launch; ``restart: k`` limits it to the k-th relaunch of ``auto_restart`` (default 0: the first launch).
    ``heartbeat_timeout_s > 0`` makes the launcher stop the job (exit code 124) when a running rank has not reported
    for that long; with ``auto_restart`` a failed job is relaunched from the latest checkpoint up to ``max_restarts``
    times."""
    inject: List[Dict[str, Any]] = field(default_factory=list)
    heartbeat_interval_s: float = 1.0
    heartbeat_timeout_s: float = 0.0
    auto_restart: bool = False
    max_restarts: int = 0


@dataclass
class SiiRLArguments:
    data: DataArguments = _dc(DataArguments)
    actor_rollout_ref: ActorRolloutRefArguments = _dc(ActorRolloutRefArguments)
    critic: CriticArguments = _dc(CriticArguments)
    reward_model: RewardModelArguments = _dc(RewardModelArguments)
    algorithm: AlgorithmArguments = _dc(AlgorithmArguments)
    trainer: TrainingArguments = _dc(TrainingArguments)
    custom_reward_function: CustomRewardArguments = _dc(CustomRewardArguments)
    dag: DagArguments = _dc(DagArguments)
    profiler: ProfilerArguments = _dc(ProfilerArguments)
    fault: FaultArguments = _dc(FaultArguments)

    def to_dict(self) -> Dict[str, Any]:
        return to_dict(self)


def to_dict(obj: Any) -> Any:
    if is_dataclass(obj):
        return {f.name: to_dict(getattr(obj, f.name)) for f in fields(obj)}
    if isinstance(obj, (list, tuple)):
        return [to_dict(v) for v in obj]
    if isinstance(obj, dict):
        return {k: to_dict(v) for k, v in obj.items()}
    return obj
