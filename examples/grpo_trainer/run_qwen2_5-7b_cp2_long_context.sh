#!/usr/bin/env bash
# GRPO on long responses with ring (context-parallel) attention: every sequence is cut into 2 x cp chunks, rank r
# trains on chunks r and 2 cp - 1 - r (zig-zag: equal causal work per rank); K/V travel over peer memory.
set -euo pipefail
python3 -m siirl_b200.main_dag \
    algorithm.adv_estimator=grpo \
    data.train_files=$HOME/data/deepscaler/train.parquet data.val_files=$HOME/data/deepscaler/test.parquet \
    data.train_batch_size=128 data.max_prompt_length=2048 data.max_response_length=30720 \
    actor_rollout_ref.model.path=$HOME/models/Qwen2.5-7B-Instruct \
    actor_rollout_ref.actor.megatron.context_parallel_size=2 \
    actor_rollout_ref.actor.megatron.context_parallel_layout=zigzag \
    actor_rollout_ref.actor.optim.lr=1e-6 actor_rollout_ref.actor.ppo_mini_batch_size=64 \
    actor_rollout_ref.actor.use_dynamic_bsz=True actor_rollout_ref.actor.ppo_max_token_len_per_gpu=65536 \
    actor_rollout_ref.rollout.n=8 actor_rollout_ref.rollout.gpu_memory_utilization=0.6 \
    trainer.n_gpus_per_node=8 trainer.nnodes=1 trainer.total_epochs=30 trainer.save_freq=10 trainer.test_freq=10 \
    trainer.logger="[console,jsonl]" trainer.project_name=siirl_b200 trainer.experiment_name=grpo_qwen2_5_7b_cp2 "$@"
