#!/usr/bin/env bash
# Embodied SRPO with an OpenVLA-OFT policy (Prismatic DINOv2 + SigLIP towers, Llama-2 7B, one-pass action-chunk
# decoding) on a LIBERO suite.  Needs robosuite / MuJoCo with an off-screen renderer on the machine; SUITE is one of
# libero_goal, libero_spatial, libero_object, libero_10 (the "long" suite).
set -euo pipefail
SUITE=${SUITE:-libero_goal}
python3 -m siirl_b200.main_dag \
    algorithm.adv_estimator=grpo algorithm.workflow_type=embodied \
    algorithm.embodied_sampling.filter_accuracy=True algorithm.embodied_sampling.accuracy_lower_bound=0.1 \
    algorithm.embodied_sampling.accuracy_upper_bound=0.9 algorithm.embodied_sampling.filter_truncated=False \
    data.train_files=$HOME/data/$SUITE/train.parquet data.val_files=$HOME/data/$SUITE/val.parquet \
    data.train_batch_size=64 data.val_batch_size=496 \
    actor_rollout_ref.model.path=$HOME/models/openvla-oft-$SUITE-sft \
    actor_rollout_ref.actor.embodied_type=openvla-oft \
    actor_rollout_ref.actor.optim.lr=5e-6 actor_rollout_ref.actor.ppo_mini_batch_size=32 \
    actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8 actor_rollout_ref.actor.clip_ratio_low=0.2 \
    actor_rollout_ref.actor.clip_ratio_high=0.28 actor_rollout_ref.actor.use_kl_loss=False \
    actor_rollout_ref.embodied.env.env_type=libero actor_rollout_ref.embodied.env.env_name=$SUITE \
    actor_rollout_ref.embodied.env.num_envs=16 actor_rollout_ref.embodied.env.max_steps=512 \
    actor_rollout_ref.embodied.action_chunks_len=8 actor_rollout_ref.embodied.action_token_len=7 \
    actor_rollout_ref.embodied.parallel_decode=True actor_rollout_ref.embodied.center_crop=True \
    actor_rollout_ref.rollout.n=8 actor_rollout_ref.rollout.temperature=1.6 \
    reward_model.reward_manager=embodied \
    trainer.n_gpus_per_node=8 trainer.nnodes=1 trainer.total_epochs=100 trainer.save_freq=5 trainer.test_freq=5 \
    trainer.logger="[console,jsonl]" trainer.project_name=siirl_b200 trainer.experiment_name=srpo_openvla_oft_$SUITE "$@"
