#!/usr/bin/env bash
# MARFT: two Qwen2.5-3B agents (Reasoner -> Actor) trained with multi-agent GAE on a math dataset.
# The agents alternate being trained every `train_cycle` steps (see config/workflow_marft.yaml); one critic serves both.
# Run from the repository root so that the relative paths inside the workflow file resolve.
set -euo pipefail
python3 -m siirl_b200.main_dag \
    dag.workflow_path=examples/experimental/marft/config/workflow_marft.yaml \
    algorithm.adv_estimator=gae_marft \
    algorithm.share_reward_in_agent=True \
    data.train_files=$HOME/data/deepscaler/train.parquet \
    data.val_files=$HOME/data/deepscaler/test.parquet \
    data.train_batch_size=128 \
    data.max_prompt_length=10240 \
    data.max_response_length=2048 \
    data.filter_overlong_prompts=True \
    data.shuffle=False \
    actor_rollout_ref.model.path=$HOME/models/Qwen2.5-3B-Instruct \
    actor_rollout_ref.actor.optim.lr=1e-6 \
    actor_rollout_ref.actor.ppo_mini_batch_size=64 \
    actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4 \
    actor_rollout_ref.actor.use_kl_loss=True \
    actor_rollout_ref.actor.kl_loss_coef=0.01 \
    actor_rollout_ref.actor.kl_loss_type=low_var_kl \
    actor_rollout_ref.actor.grad_clip=0.5 \
    actor_rollout_ref.rollout.n=1 \
    actor_rollout_ref.rollout.gpu_memory_utilization=0.3 \
    actor_rollout_ref.rollout.max_model_len=12288 \
    actor_rollout_ref.rollout.agent.rewards_with_env=True \
    actor_rollout_ref.rollout.multi_turn.max_assistant_turns=3 \
    actor_rollout_ref.rollout.multi_turn.use_all_traj=False \
    critic.model.path=$HOME/models/Qwen2.5-3B-Instruct \
    critic.optim.lr=1e-5 \
    critic.ppo_mini_batch_size=64 \
    critic.ppo_micro_batch_size_per_gpu=4 \
    algorithm.kl_ctrl.kl_coef=0.001 \
    trainer.n_gpus_per_node=8 trainer.nnodes=1 \
    trainer.total_epochs=30 trainer.save_freq=30 trainer.test_freq=10 \
    trainer.logger="[console,jsonl]" trainer.project_name=siirl_b200 \
    trainer.experiment_name=marft_qwen2.5_3b trainer.val_before_train=False "$@"
