#!/usr/bin/env bash
# GRPO on Kimi-VL-A3B (MoonViT tower + Moonlight-16B-A3B: multi-head latent attention, 64 routed experts).  Rollout
# decodes against the cache of compressed latents; experts are spread over the 8 GPUs of the node.
set -euo pipefail
python3 -m siirl_b200.main_dag \
    algorithm.adv_estimator=grpo \
    data.train_files=$HOME/data/geo3k/train.parquet data.val_files=$HOME/data/geo3k/test.parquet \
    data.train_batch_size=128 data.max_prompt_length=2048 data.max_response_length=2048 data.image_key=images \
    actor_rollout_ref.model.path=$HOME/models/Kimi-VL-A3B-Instruct \
    actor_rollout_ref.actor.optim.lr=1e-6 actor_rollout_ref.actor.ppo_mini_batch_size=64 \
    actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4 actor_rollout_ref.actor.use_kl_loss=True \
    actor_rollout_ref.actor.kl_loss_coef=0.01 actor_rollout_ref.actor.kl_loss_type=low_var_kl \
    actor_rollout_ref.actor.fsdp_config.sharding=zero3 \
    actor_rollout_ref.rollout.n=5 actor_rollout_ref.rollout.max_num_seqs=128 \
    trainer.n_gpus_per_node=8 trainer.nnodes=1 trainer.total_epochs=15 trainer.save_freq=10 trainer.test_freq=5 \
    trainer.logger="[console,jsonl]" trainer.project_name=siirl_b200 trainer.experiment_name=grpo_kimi_vl_a3b "$@"
