#!/usr/bin/env bash
# DAPO on a vision-language policy (Qwen2.5-VL-7B, geometry3k): dynamic sampling, clip-higher, token-level loss;
# rollout engines of two GPUs each (tensor parallel), actor and reference weights sharded over the eight ranks.
set -euo pipefail
python3 -m siirl_b200.main_dag \
    algorithm.adv_estimator=grpo algorithm.workflow_type=dapo \
    algorithm.filter_groups.enable=True algorithm.filter_groups.metric=acc algorithm.filter_groups.max_num_gen_batches=10 \
    data.train_files=$HOME/data/geo3k/train.parquet data.val_files=$HOME/data/geo3k/test.parquet \
    data.image_key=images data.train_batch_size=128 data.max_prompt_length=1024 data.max_response_length=2048 \
    actor_rollout_ref.model.path=$HOME/models/Qwen2.5-VL-7B-Instruct \
    actor_rollout_ref.model.enable_gradient_checkpointing=True \
    actor_rollout_ref.actor.optim.lr=1e-6 actor_rollout_ref.actor.ppo_mini_batch_size=128 \
    actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8 \
    actor_rollout_ref.actor.clip_ratio_low=0.2 actor_rollout_ref.actor.clip_ratio_high=0.28 \
    actor_rollout_ref.actor.loss_agg_mode=token-mean actor_rollout_ref.actor.use_kl_loss=False \
    actor_rollout_ref.actor.fsdp_config.sharding=zero3 \
    actor_rollout_ref.rollout.n=8 actor_rollout_ref.rollout.tensor_model_parallel_size=2 \
    actor_rollout_ref.rollout.gpu_memory_utilization=0.6 \
    reward_model.reward_manager=dapo reward_model.overlong_buffer.enable=True reward_model.overlong_buffer.len=512 \
    trainer.n_gpus_per_node=8 trainer.nnodes=1 trainer.total_epochs=15 trainer.save_freq=10 trainer.test_freq=5 \
    trainer.logger="[console,jsonl]" trainer.project_name=siirl_b200 trainer.experiment_name=dapo_qwen2.5_vl_7b "$@"
