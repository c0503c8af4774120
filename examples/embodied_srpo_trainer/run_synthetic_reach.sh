#!/usr/bin/env bash
# Embodied SRPO on the headless synthetic reach environment (CUDA-rasterised 256x256 observations).
# LIBERO suites use env.env_type=libero on machines that have robosuite / MuJoCo with an off-screen GL renderer.
set -euo pipefail
python3 -m siirl_b200.main_dag \
    algorithm.adv_estimator=grpo algorithm.workflow_type=embodied \
    algorithm.embodied_sampling.filter_accuracy=True algorithm.embodied_sampling.accuracy_lower_bound=0.1 \
    algorithm.embodied_sampling.accuracy_upper_bound=0.9 \
    data.synthetic=embodied data.synthetic_size=500 data.train_batch_size=64 \
    actor_rollout_ref.model.path=$HOME/models/Qwen2.5-VL-7B-Instruct \
    actor_rollout_ref.actor.embodied_type=native-vla \
    actor_rollout_ref.embodied.env.env_type=synthetic actor_rollout_ref.embodied.env.num_envs=64 \
    actor_rollout_ref.embodied.env.max_steps=64 actor_rollout_ref.embodied.action_chunks_len=8 \
    actor_rollout_ref.rollout.n=8 reward_model.reward_manager=embodied \
    trainer.n_gpus_per_node=8 trainer.total_epochs=10 "$@"
