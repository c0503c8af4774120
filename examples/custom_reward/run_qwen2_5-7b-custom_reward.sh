#!/usr/bin/env bash
# GRPO on GSM8K with a user-supplied, batched reward function (examples/custom_reward/rewardfunc_gsm8k.py)
set -euo pipefail
python3 -m siirl_b200.main_dag \
    algorithm.adv_estimator=grpo \
    data.train_files=$HOME/data/gsm8k/train.parquet \
    data.val_files=$HOME/data/gsm8k/test.parquet \
    data.train_batch_size=512 \
    data.max_prompt_length=1024 \
    data.max_response_length=2048 \
    actor_rollout_ref.model.path=$HOME/models/Qwen2.5-7B-Instruct \
    actor_rollout_ref.actor.optim.lr=1e-6 \
    actor_rollout_ref.actor.ppo_mini_batch_size=256 \
    actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8 \
    actor_rollout_ref.actor.use_kl_loss=True \
    actor_rollout_ref.actor.kl_loss_coef=0.001 \
    actor_rollout_ref.rollout.n=8 \
    actor_rollout_ref.rollout.gpu_memory_utilization=0.5 \
    custom_reward_function.path=examples/custom_reward/rewardfunc_gsm8k.py \
    custom_reward_function.name=compute_score \
    reward_model.reward_manager=batch \
    trainer.n_gpus_per_node=8 trainer.nnodes=1 \
    trainer.total_epochs=30 trainer.save_freq=10 trainer.test_freq=10 \
    trainer.logger="[console,jsonl]" trainer.project_name=siirl_b200 \
    trainer.experiment_name=grpo_qwen2.5_7b_custom_reward "$@"
