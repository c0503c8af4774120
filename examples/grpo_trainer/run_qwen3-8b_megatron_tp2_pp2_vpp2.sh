#!/usr/bin/env bash
# GRPO with the Megatron-style layout: tensor parallel 2 (with sequence parallelism) x pipeline parallel 2 with two
# virtual stages per rank (interleaved 1F1B), data parallel over the remaining ranks; rollout on the trainer's slices.
set -euo pipefail
python3 -m siirl_b200.main_dag \
    algorithm.adv_estimator=grpo \
    data.train_files=$HOME/data/deepscaler/train.parquet data.val_files=$HOME/data/deepscaler/test.parquet \
    data.train_batch_size=256 data.max_prompt_length=2048 data.max_response_length=8192 \
    actor_rollout_ref.model.path=$HOME/models/Qwen3-8B \
    actor_rollout_ref.actor.strategy=megatron actor_rollout_ref.ref.strategy=megatron \
    actor_rollout_ref.actor.megatron.tensor_model_parallel_size=2 \
    actor_rollout_ref.actor.megatron.sequence_parallel=True \
    actor_rollout_ref.actor.megatron.pipeline_model_parallel_size=2 \
    actor_rollout_ref.actor.megatron.virtual_pipeline_model_parallel_size=2 \
    actor_rollout_ref.actor.optim.lr=1e-6 actor_rollout_ref.actor.ppo_mini_batch_size=64 \
    actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=2 actor_rollout_ref.actor.use_kl_loss=True \
    actor_rollout_ref.actor.kl_loss_coef=0.001 actor_rollout_ref.actor.kl_loss_type=low_var_kl \
    actor_rollout_ref.model.override_config="{tie_word_embeddings: False}" \
    actor_rollout_ref.rollout.tensor_model_parallel_size=2 actor_rollout_ref.rollout.n=8 \
    actor_rollout_ref.rollout.gpu_memory_utilization=0.5 \
    trainer.n_gpus_per_node=8 trainer.nnodes=1 trainer.total_epochs=30 trainer.save_freq=10 trainer.test_freq=10 \
    trainer.logger="[console,jsonl]" trainer.project_name=siirl_b200 trainer.experiment_name=grpo_qwen3_8b_tp2_pp2_vpp2 "$@"
