"""Always-on integration gate: tiny Qwen2-style decoder, GRPO on CPU/gloo with world_size=2, 3 steps, then resume.

Model and task of the gate configuration: 2 layers, hidden 128, 4 heads / 2 KV heads, head_dim 32, SwiGLU 352,
vocab 1024; 8 prompts x n=4 per step, prompt lengths 16-32, max response 32, reward 1 if the last generated token
id is even; group-normalised advantages, clip 0.2, KL coefficient 0.001 to a frozen reference copy, lr 1e-5."""
import json
import os
import subprocess
import sys

import pytest

ARGS = [
    "algorithm.adv_estimator=grpo", "data.synthetic=parity", "data.synthetic_size=64", "data.synthetic_min_prompt=16",
    "data.synthetic_max_prompt=32", "data.max_prompt_length=32", "data.max_response_length=32",
    "data.train_batch_size=8", "actor_rollout_ref.model.arch_preset=tiny", "actor_rollout_ref.rollout.n=4",
    "actor_rollout_ref.rollout.max_num_seqs=16", "actor_rollout_ref.actor.ppo_mini_batch_size=8",
    "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4", "actor_rollout_ref.actor.use_kl_loss=True",
    "actor_rollout_ref.actor.kl_loss_coef=0.001", "actor_rollout_ref.actor.clip_ratio=0.2",
    "actor_rollout_ref.actor.optim.lr=1e-5", "trainer.n_gpus_per_node=2", "trainer.device=cpu",
    "trainer.val_before_train=False", "trainer.logger=['jsonl']",
]


def _run(extra, log_dir, timeout=900):
    env = dict(os.environ, OMP_NUM_THREADS="2", SIIRL_LOG_DIR=str(log_dir))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    return subprocess.run([sys.executable, "-m", "siirl_b200.main_dag", *ARGS, *extra], env=env, cwd=root,
                          capture_output=True, text=True, timeout=timeout)


def _metrics(log_dir):
    with open(os.path.join(log_dir, "metrics.jsonl")) as f:
        return [json.loads(line) for line in f]


def test_grpo_two_ranks_three_steps_and_resume(tmp_path):
    ck = tmp_path / "ckpt"
    remote = tmp_path / "remote"        # stands in for an hdfs:// directory (the copy helper takes local paths too)
    out = _run([f"trainer.default_local_dir={ck}", "trainer.total_training_steps=3", "trainer.save_freq=2",
                "actor_rollout_ref.actor.checkpoint.async_save=True", f"trainer.default_hdfs_dir={remote}"],
               tmp_path / "log1")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log1")
    assert [r["step"] for r in m] == [1, 2, 3]
    for r in m:
        assert 0.0 <= r["critic/score/mean"] <= 1.0
        assert r["actor/grad_norm"] > 0 and r["actor/grad_norm"] == r["actor/grad_norm"]
        assert abs(r["critic/advantages/mean"]) < 0.2
        assert r["perf/total_num_tokens"] > 8 * 4 * 17          # summed over both ranks
        assert r["response_length/max"] <= 32
    assert (ck / "latest_checkpointed_iteration.txt").read_text().strip() == "3"
    step3 = ck / "global_step_3" / "actor_agent_0"
    assert (step3 / "manifest.json").exists() and (step3 / "model_world_size_2_rank_1.pt").exists()
    assert (ck / "global_step_3" / "data_dp_rank_1.pt").exists()
    # the asynchronous writers were joined before the tracker was written, and every file went to the remote copy
    from siirl_b200.utils.checkpoint.checkpoint_manager import checkpoint_problems
    assert checkpoint_problems(str(ck / "global_step_3")) == []
    assert (remote / "latest_checkpointed_iteration.txt").read_text().strip() == "3"
    assert checkpoint_problems(str(remote / "global_step_3")) == []
    # resume on a machine with an empty local directory: the tracked step is fetched from the remote copy;
    # continues at step 4 and stops at 4
    fresh = tmp_path / "fresh"
    out = _run([f"trainer.default_local_dir={fresh}", f"trainer.default_hdfs_dir={remote}",
                "trainer.total_training_steps=4", "trainer.resume_mode=auto"], tmp_path / "log2")
    assert out.returncode == 0, out.stderr[-4000:]
    assert [r["step"] for r in _metrics(tmp_path / "log2")] == [4]
    # an explicit step directory instead of the tracker's latest one
    out = _run([f"trainer.default_local_dir={tmp_path / 'other'}", "trainer.total_training_steps=3",
                "trainer.resume_mode=resume_path", f"trainer.resume_from_path={ck / 'global_step_2'}"], tmp_path / "log3")
    assert out.returncode == 0, out.stderr[-4000:]
    assert [r["step"] for r in _metrics(tmp_path / "log3")] == [3]


def test_grpo_with_sharded_parameters(tmp_path):
    """``fsdp_config.sharding=zero3``: actor and reference weights sharded over the two ranks, gathered layer by layer
    for scoring and training and regathered whole for the rollout engine; save and resume included."""
    ck = tmp_path / "c"
    extra = ["actor_rollout_ref.actor.fsdp_config.sharding=zero3",
             "actor_rollout_ref.model.enable_gradient_checkpointing=True", "data.max_response_length=16",
             "actor_rollout_ref.actor.checkpoint.contents=[model,optimizer,extra,hf_model]"]
    out = _run([f"trainer.default_local_dir={ck}", "trainer.total_training_steps=2", "trainer.save_freq=2", *extra],
               tmp_path / "log1")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log1")
    assert [r["step"] for r in m] == [1, 2]
    assert all(r["actor/grad_norm"] > 0 for r in m)
    role = ck / "global_step_2" / "actor_agent_0"
    assert (role / "experts_world_size_2_rank_1.pt").exists()
    # every layer's flat unit is split over the ranks: the offline exporter puts the pieces back together, and its
    # output equals the Hugging Face directory the training job wrote itself
    import torch
    from safetensors.torch import load_file

    from siirl_b200.utils.checkpoint.export_hf import main as export_main
    assert export_main(["--checkpoint", str(role), "--out", str(tmp_path / "hf"), "--dtype", "float32"]) == 0
    want = load_file(str(role / "huggingface" / "model.safetensors"))
    got = load_file(str(tmp_path / "hf" / "model.safetensors"))
    assert set(want) == set(got) and all(torch.equal(want[k], got[k]) for k in want)
    out = _run([f"trainer.default_local_dir={ck}", "trainer.total_training_steps=3", "trainer.resume_mode=auto",
                *extra], tmp_path / "log2")
    assert out.returncode == 0, out.stderr[-4000:]
    assert [r["step"] for r in _metrics(tmp_path / "log2")] == [3]


def test_grpo_with_megatron_tensor_and_sequence_parallel_training(tmp_path):
    """``strategy=megatron`` with tensor_model_parallel_size=2 and sequence_parallel: both ranks hold half of every
    projection, train and score on the slices, the rollout engine decodes on the same slices; save and resume."""
    ck = tmp_path / "c"
    extra = ["actor_rollout_ref.actor.strategy=megatron",
             "actor_rollout_ref.actor.megatron.tensor_model_parallel_size=2",
             "actor_rollout_ref.actor.megatron.sequence_parallel=True",
             "actor_rollout_ref.rollout.tensor_model_parallel_size=2", "data.max_response_length=16"]
    out = _run([f"trainer.default_local_dir={ck}", "trainer.total_training_steps=2", "trainer.save_freq=2", *extra],
               tmp_path / "log1")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log1")
    assert [r["step"] for r in m] == [1, 2]
    assert all(r["actor/grad_norm"] > 0 and r["actor/grad_norm"] == r["actor/grad_norm"] for r in m)
    assert (ck / "global_step_2" / "actor_agent_0" / "tp_rank_1" / "manifest.json").exists()
    out = _run([f"trainer.default_local_dir={ck}", "trainer.total_training_steps=3", "trainer.resume_mode=auto",
                *extra], tmp_path / "log2")
    assert out.returncode == 0, out.stderr[-4000:]
    assert [r["step"] for r in _metrics(tmp_path / "log2")] == [3]


def test_injected_rank_failure_stops_the_job(tmp_path):
    out = _run([f"trainer.default_local_dir={tmp_path / 'c'}", "trainer.total_training_steps=2",
                "fault.inject=[{rank: 1, step: 0, node: function_reward, kind: exit, code: 17}]"], tmp_path / "log",
               timeout=600)
    assert out.returncode == 17
    assert not (tmp_path / "c" / "latest_checkpointed_iteration.txt").exists()


@pytest.mark.parametrize("preset", ["tiny-moe", "tiny-deepseek-v3"])
def test_moe_expert_parallel_two_ranks(tmp_path, preset):
    """Qwen3-MoE-style tiny model, experts split over two gloo ranks: dispatch / combine across ranks in training,
    scoring and the lock-step rollout; the dense part in the sharded-state store, the experts in a rank-local one.
    ``tiny-deepseek-v3``: the same with multi-head latent attention, whose rollout is the latent-cache engine running
    in lock-step rounds (responses stop at EOS at different lengths on the two ranks)."""
    out = _run([f"actor_rollout_ref.model.arch_preset={preset}", "actor_rollout_ref.model.ep_max_tokens=512",
                "actor_rollout_ref.actor.megatron.expert_model_parallel_size=2", "data.max_response_length=16",
                "actor_rollout_ref.rollout.n=2", "actor_rollout_ref.rollout.max_num_seqs=16",
                "actor_rollout_ref.actor.use_kl_loss=False", f"trainer.default_local_dir={tmp_path / 'c'}",
                "trainer.total_training_steps=2", "trainer.save_freq=2"], tmp_path / "log")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log")
    assert [r["step"] for r in m] == [1, 2]
    assert all(r["actor/grad_norm"] > 0 for r in m)
    d = tmp_path / "c" / "global_step_2" / "actor_agent_0"
    assert (d / "experts_world_size_2_rank_0.pt").exists() and (d / "experts_world_size_2_rank_1.pt").exists()


def test_ulysses_and_tensor_parallel_rollout_two_ranks(tmp_path):
    """Two ranks as ONE data-parallel replica: tensor-parallel rollout (TP=2), then Ulysses sequence-parallel
    scoring and training (SP=2).  The generation batch is published by the first TP rank only and both SP ranks
    receive the same micro-batches."""
    out = _run(["actor_rollout_ref.rollout.tensor_model_parallel_size=2", "actor_rollout_ref.rollout.max_num_seqs=32",
                "actor_rollout_ref.actor.ulysses_sequence_parallel_size=2", f"trainer.default_local_dir={tmp_path / 'c'}",
                "trainer.total_training_steps=2", "trainer.save_freq=-1"], tmp_path / "log")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log")
    assert [r["step"] for r in m] == [1, 2]
    for r in m:
        assert r["actor/grad_norm"] > 0 and 0.0 <= r["critic/score/mean"] <= 1.0
        assert r["perf/total_num_tokens"] > 8 * 4 * 17


def test_lora_adapters_train_against_the_frozen_base(tmp_path):
    """Two ranks decode as one tensor-parallel engine whose weight slices have the adapters folded in (the
    single-rank engine is covered by the target-modules test below)."""
    _lora_run(tmp_path, 2, [])


def test_lora_target_modules_select_the_adapted_projections(tmp_path):
    """peft-style ``target_modules``: adapters on the attention projections only."""
    _lora_run(tmp_path, 1, ["actor_rollout_ref.model.target_modules=[q_proj,v_proj,o_proj]"])
    from siirl_b200.engine.workers import lora_targets
    assert lora_targets("all-linear") is None and lora_targets(["q_proj", "v_proj", "o_proj"]) == ("qkv_proj", "o_proj")
    assert lora_targets("up_proj") == ("gate_up_proj",)
    with pytest.raises(ValueError):
        lora_targets(["lm_head"])


def _lora_run(tmp_path, rollout_tp, more):
    """LoRA: only the adapters are in the optimizer store; the reference policy is the same model with the
    adapters switched off, so the KL term starts at zero and becomes positive once the adapters move.  With
    ``rollout_tp=2`` two ranks decode as one tensor-parallel engine whose weight slices have the adapters folded in."""
    out = _run(["actor_rollout_ref.model.lora_rank=8", "actor_rollout_ref.model.lora_alpha=16",
                "actor_rollout_ref.actor.optim.lr=1e-3", f"trainer.n_gpus_per_node={rollout_tp}",
                f"actor_rollout_ref.rollout.tensor_model_parallel_size={rollout_tp}",
                f"trainer.default_local_dir={tmp_path / 'c'}", "trainer.total_training_steps=3",
                "trainer.save_freq=-1", *more], tmp_path / "log")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log")
    assert [r["step"] for r in m] == [1, 2, 3]
    assert m[0]["actor/kl_loss"] == 0.0 and m[2]["actor/kl_loss"] > 0.0
    assert all(r["actor/grad_norm"] > 0 for r in m)


def test_context_parallel_ring_attention_two_ranks(tmp_path):
    """Two ranks as one replica with ring (context-parallel) attention in scoring and training: every sequence is cut
    in two chunks, K/V of the first chunk travel to the second rank, log-probs are summed over the group."""
    out = _run(["actor_rollout_ref.actor.megatron.context_parallel_size=2", "actor_rollout_ref.rollout.max_num_seqs=32",
                f"trainer.default_local_dir={tmp_path / 'c'}", "trainer.total_training_steps=2", "trainer.save_freq=-1"],
               tmp_path / "log")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log")
    assert [r["step"] for r in m] == [1, 2]
    for r in m:
        assert r["actor/grad_norm"] > 0 and abs(r["actor/ppo_kl"]) < 1e-3       # on-policy: same log-probs twice


@pytest.mark.parametrize("virtual", [1, 2])
def test_pipeline_parallel_two_stages(tmp_path, virtual):
    """Two ranks as one two-stage pipeline (layers split, activations and their gradients sent point to point, trained
    stage weights re-broadcast after the update so the rollout engines keep whole, identical replicas); with
    ``virtual=2`` every stage holds two model chunks and training runs the interleaved schedule."""
    out = _run(["actor_rollout_ref.actor.megatron.pipeline_model_parallel_size=2",
                f"actor_rollout_ref.actor.megatron.virtual_pipeline_model_parallel_size={virtual}",
                "actor_rollout_ref.model.override_config={tie_word_embeddings: False, num_layers: 4}",
                "actor_rollout_ref.rollout.max_num_seqs=32", f"trainer.default_local_dir={tmp_path / 'c'}",
                "trainer.total_training_steps=2", "trainer.save_freq=-1"], tmp_path / "log")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log")
    assert [r["step"] for r in m] == [1, 2]
    for r in m:
        assert r["actor/grad_norm"] > 0 and abs(r["actor/ppo_kl"]) < 1e-3


def test_rollout_importance_weights(tmp_path):
    """algorithm.rollout_is: per-token weights min(pi_train / pi_rollout, threshold) reach the policy loss; engine and
    trainer agree on CPU, so the ratio is 1 and nothing is truncated."""
    out = _run(["algorithm.rollout_is=True", "trainer.n_gpus_per_node=1", f"trainer.default_local_dir={tmp_path / 'c'}",
                "trainer.total_training_steps=1", "trainer.save_freq=-1"], tmp_path / "log")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log")[0]
    assert abs(m["actor/rollout_is_ratio_mean"] - 1.0) < 1e-3 and m["actor/rollout_is_truncated_frac"] == 0.0
    assert m["actor/grad_norm"] > 0


_SMALL = ["data.max_response_length=16", "trainer.total_training_steps=2"]


def test_ppo_with_critic_and_warmup(tmp_path):
    """GAE pipeline: value model scored before the update, critic trained every step, the actor only after
    ``trainer.critic_warmup`` steps; KL to the reference folded into the reward."""
    out = _run(["algorithm.adv_estimator=gae", "critic.model.arch_preset=tiny", "critic.ppo_mini_batch_size=8",
                "critic.ppo_micro_batch_size_per_gpu=4", "algorithm.use_kl_in_reward=True",
                "actor_rollout_ref.actor.use_kl_loss=False", "actor_rollout_ref.rollout.n=2",
                "trainer.critic_warmup=1", f"trainer.default_local_dir={tmp_path / 'c'}", "trainer.save_freq=2",
                *_SMALL], tmp_path / "log")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log")
    assert [r["step"] for r in m] == [1, 2]
    assert "actor/grad_norm" not in m[0] and m[1]["actor/grad_norm"] > 0
    for r in m:
        assert r["critic/vf_loss"] > 0 and "critic/values/mean" in r and "actor/reward_kl_penalty" in r
    assert (tmp_path / "c" / "global_step_2" / "critic_agent_0" / "manifest.json").exists()


def test_dapo_dynamic_sampling_and_overlong_penalty(tmp_path):
    out = _run(["algorithm.workflow_type=dapo", "algorithm.filter_groups.enable=True",
                "algorithm.filter_groups.metric=seq_reward", "algorithm.filter_groups.max_num_gen_batches=8",
                "reward_model.reward_manager=dapo", "reward_model.overlong_buffer.enable=True",
                "reward_model.overlong_buffer.len=4", "actor_rollout_ref.actor.clip_ratio_low=0.2",
                "actor_rollout_ref.actor.clip_ratio_high=0.28", "data.gen_batch_size=12",
                "actor_rollout_ref.actor.use_kl_loss=False", f"trainer.default_local_dir={tmp_path / 'c'}", *_SMALL],
               tmp_path / "log")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log")
    assert [r["step"] for r in m] == [1, 2]
    for r in m:
        assert 0 < r["dapo_sampling/kept_trajectories_ratio"] <= 1.0
        assert r["dapo_sampling/final_trajectories"] <= r["dapo_sampling/initial_trajectories"]
        assert r["critic/score/min"] < 0          # the overlong penalty makes full-length responses negative
        assert r["actor/grad_norm"] > 0


@pytest.mark.parametrize("variant", [["actor_rollout_ref.actor.policy_loss.loss_mode=gspo"],
                                     ["algorithm.adv_estimator=cpgd"]], ids=["gspo", "cpgd"])
def test_gspo_and_cpgd_variants(tmp_path, variant):
    # a loss-mode variant does not depend on the number of ranks: one rank keeps the job short
    out = _run([*variant, f"trainer.default_local_dir={tmp_path / 'c'}", *_SMALL, "trainer.n_gpus_per_node=1"],
               tmp_path / "log")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log")
    assert [r["step"] for r in m] == [1, 2]
    assert all(r["actor/grad_norm"] > 0 for r in m)


def test_silent_rank_is_detected_by_the_heartbeat_watchdog(tmp_path):
    """Rank 1 stops reporting and stalls before the reward node: the launcher ends the job with code 124 long before
    the stall (60 s) is over."""
    import time
    t0 = time.time()
    out = _run([f"trainer.default_local_dir={tmp_path / 'c'}", "trainer.total_training_steps=2",
                "fault.heartbeat_timeout_s=3", "fault.heartbeat_interval_s=0.5",
                "fault.inject=[{rank: 1, step: 0, node: function_reward, kind: drop_heartbeat, seconds: 60}]",
                *_SMALL], tmp_path / "log", timeout=600)
    assert out.returncode == 124, out.stdout[-1000:] + out.stderr[-3000:]
    assert "no heartbeat from rank(s) [1]" in out.stderr
    assert time.time() - t0 < 55


def test_auto_restart_resumes_from_the_latest_checkpoint(tmp_path):
    """Rank 0 exits at step 2 of the first launch; the job is relaunched once, resumes at step 2 and finishes."""
    ck = tmp_path / "c"
    out = _run([f"trainer.default_local_dir={ck}", "trainer.total_training_steps=3", "trainer.save_freq=1",
                "fault.auto_restart=True", "fault.max_restarts=1",
                "fault.inject=[{rank: 0, step: 2, node: actor_train, kind: exit, code: 9}]",
                "data.max_response_length=16"], tmp_path / "log", timeout=900)
    assert out.returncode == 0, out.stdout[-1000:] + out.stderr[-3000:]
    assert "restart 1/1" in out.stderr
    steps = [r["step"] for r in _metrics(tmp_path / "log")]
    assert steps[-1] == 3 and steps.count(3) == 1 and 1 in steps and 2 in steps
    assert (ck / "latest_checkpointed_iteration.txt").read_text().strip() == "3"


def test_resume_falls_back_when_the_latest_checkpoint_is_damaged(tmp_path):
    from siirl_b200.utils.checkpoint.checkpoint_manager import checkpoint_problems, find_latest_complete_ckpt_path
    ck = tmp_path / "c"
    out = _run([f"trainer.default_local_dir={ck}", "trainer.total_training_steps=2", "trainer.save_freq=1",
                "data.max_response_length=16"], tmp_path / "log1")
    assert out.returncode == 0, out.stderr[-3000:]
    assert checkpoint_problems(str(ck / "global_step_2")) == []
    shard = ck / "global_step_2" / "actor_agent_0" / "model_world_size_2_rank_1.pt"
    data = shard.read_bytes()
    shard.write_bytes(data[:len(data) // 2])                       # cut short, as after a crash or a full disk
    probs = checkpoint_problems(str(ck / "global_step_2"))
    assert len(probs) == 1 and "model_world_size_2_rank_1.pt" in probs[0]
    assert find_latest_complete_ckpt_path(str(ck), log=lambda *_: None) == str(ck / "global_step_1")
    # an optimizer shard that is absent is a problem too (the other ranks would load theirs)
    optim = ck / "global_step_1" / "actor_agent_0" / "optim_world_size_2_rank_0.pt"
    kept = optim.read_bytes()
    optim.unlink()
    assert any("optim" in p for p in checkpoint_problems(str(ck / "global_step_1")))
    assert find_latest_complete_ckpt_path(str(ck), log=lambda *_: None) is None
    optim.write_bytes(kept)
    # without the tracker file no save ever completed: nothing is resumed
    tracker = ck / "latest_checkpointed_iteration.txt"
    text = tracker.read_text()
    tracker.unlink()
    assert find_latest_complete_ckpt_path(str(ck), log=lambda *_: None) is None
    tracker.write_text(text)
    out = _run([f"trainer.default_local_dir={ck}", "trainer.total_training_steps=3", "trainer.resume_mode=auto",
                "data.max_response_length=16"], tmp_path / "log2")
    assert out.returncode == 0, out.stderr[-3000:]
    assert [r["step"] for r in _metrics(tmp_path / "log2")] == [2, 3]      # continued after step 1


def test_grpo_with_hybrid_sharding(tmp_path):
    """``fsdp_config.fsdp_size=2`` on four ranks (FSDP's HYBRID_SHARD): state sharded inside blocks of two ranks and
    replicated across the blocks, with the replicated-weights store and with the parameter-sharded one; save and
    resume.  (That the stores compute the same update as four-way sharding is checked on the stores directly.)"""
    base = ["trainer.n_gpus_per_node=4", "data.max_response_length=16",
            "actor_rollout_ref.model.enable_gradient_checkpointing=True",
            "actor_rollout_ref.actor.fsdp_config.fsdp_size=2"]
    # the first job also decodes with tensor-parallel engines of two ranks each: rollout data-parallel width 2,
    # training width 4, so the samples are redistributed (whole prompt groups, ids unique over the producers)
    out = _run([*base, "trainer.total_training_steps=1", "actor_rollout_ref.rollout.tensor_model_parallel_size=2",
                "data.train_batch_size=16", "actor_rollout_ref.actor.ppo_mini_batch_size=16"], tmp_path / "zero2")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m0 = _metrics(tmp_path / "zero2")[0]
    assert m0["actor/grad_norm"] > 0 and abs(m0["actor/ppo_kl"]) < 1e-3 and abs(m0["critic/advantages/mean"]) < 0.2
    z3 = [*base, "actor_rollout_ref.actor.fsdp_config.sharding=zero3", f"trainer.default_local_dir={tmp_path / 'c'}"]
    out = _run([*z3, "trainer.total_training_steps=2", "trainer.save_freq=2"], tmp_path / "zero3")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "zero3")
    assert [r["step"] for r in m] == [1, 2] and all(r["actor/grad_norm"] > 0 for r in m)
    out = _run([*z3, "trainer.total_training_steps=3", "trainer.resume_mode=auto"], tmp_path / "resume")
    assert out.returncode == 0, out.stderr[-4000:]
    assert [r["step"] for r in _metrics(tmp_path / "resume")] == [3]


def test_grpo_with_deepseek_v3_family(tmp_path):
    """Multi-head latent attention + DeepSeek-V3 routing (sigmoid scores, selection bias, expert groups, shared expert,
    a dense first layer) through rollout (cache-free engine), scoring and training on two ranks; save and resume."""
    ck = tmp_path / "c"
    extra = ["actor_rollout_ref.model.arch_preset=tiny-deepseek-v3", "data.max_response_length=8",
             f"trainer.default_local_dir={ck}"]
    out = _run([*extra, "trainer.total_training_steps=2", "trainer.save_freq=2"], tmp_path / "log1")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log1")
    assert [r["step"] for r in m] == [1, 2]
    assert all(r["actor/grad_norm"] > 0 and r["actor/grad_norm"] == r["actor/grad_norm"] for r in m)
    out = _run([*extra, "trainer.total_training_steps=3", "trainer.resume_mode=auto"], tmp_path / "log2")
    assert out.returncode == 0, out.stderr[-4000:]
    assert [r["step"] for r in _metrics(tmp_path / "log2")] == [3]



def _spawn_node(args, log_dir, node_rank, port):
    env = dict(os.environ, OMP_NUM_THREADS="2", SIIRL_LOG_DIR=str(log_dir), NODE_RANK=str(node_rank),
               MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    return subprocess.Popen([sys.executable, "-m", "siirl_b200.main_dag", *ARGS, *args], env=env, cwd=root,
                            stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)


def test_two_node_launch_on_one_host(tmp_path):
    """``trainer.nnodes=2``: the same command on two "nodes" (here: two launchers on one host) with NODE_RANK /
    MASTER_ADDR / MASTER_PORT; node 0 hosts the rendezvous, each launcher spawns its own ranks."""
    from siirl_b200.execution.scheduler.launch import find_free_port
    port = find_free_port()
    args = ["trainer.nnodes=2", "trainer.n_gpus_per_node=1", f"trainer.default_local_dir={tmp_path / 'c'}",
            "trainer.total_training_steps=2", "trainer.save_freq=-1"]
    nodes = [_spawn_node(args, tmp_path / "log", r, port) for r in (0, 1)]
    outs = [p.communicate(timeout=600) for p in nodes]
    assert [p.returncode for p in nodes] == [0, 0], outs[0][1][-3000:] + outs[1][1][-3000:]
    m = _metrics(tmp_path / "log")
    assert [r["step"] for r in m] == [1, 2] and all(r["actor/grad_norm"] > 0 for r in m)


def test_two_node_job_stops_as_a_whole_when_one_node_fails(tmp_path):
    """A rank of node 1 raises at step 1: node 1's launcher flags the abort in the rendezvous store, node 0's launcher
    sees it and stops its ranks; both commands return non-zero instead of waiting in a collective."""
    from siirl_b200.execution.scheduler.launch import find_free_port
    port = find_free_port()
    args = ["trainer.nnodes=2", "trainer.n_gpus_per_node=1", f"trainer.default_local_dir={tmp_path / 'c'}",
            "trainer.total_training_steps=3", "trainer.save_freq=-1",
            "fault.inject=[{rank: 1, step: 1, node: function_reward, kind: exit, code: 23}]"]
    nodes = [_spawn_node(args, tmp_path / "log", r, port) for r in (0, 1)]
    outs = [p.communicate(timeout=300) for p in nodes]
    assert nodes[1].returncode == 23, outs[1][1][-3000:]
    assert nodes[0].returncode != 0, outs[0][1][-3000:]
    assert "another node stopped the job" in outs[0][1] or nodes[0].returncode == 23


def test_optional_step_features_two_ranks(tmp_path):
    """One two-rank job with the optional paths of a step switched on together:

    * ``trainer.async_metrics``: ranks post their step metrics to the collector thread on rank 0; the log holds one
      merged record per step with the keys of the in-band reduction (token counts summed over the ranks);
    * ``data.rebalance_after_rollout``: after generation the ranks exchange whole prompt groups; group-relative
      advantages still see complete groups (mean advantage ~ 0, on-policy ratio 1);
    * ``trainer.rollout_data_dir``: each rank writes ``step_<N>_rank_<r>.json`` with the generations it validated;
    * the checkpoint written by the two ranks (one parameter slice each) is reassembled offline in one process and
      written as a Hugging Face directory that loads back into the same weights."""
    import torch

    from siirl_b200.models.config import DecoderConfig, get_config
    from siirl_b200.models.decoder import build_model
    from siirl_b200.models.hf_io import load_hf_weights
    from siirl_b200.utils.checkpoint.export_hf import main as export_main
    out = _run(["trainer.async_metrics=True", "data.rebalance_after_rollout=True", "trainer.test_freq=1",
                f"trainer.rollout_data_dir={tmp_path / 'dump'}", f"trainer.default_local_dir={tmp_path / 'c'}",
                "trainer.total_training_steps=2", "trainer.save_freq=2"], tmp_path / "log")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log")
    steps = [r for r in m if "actor/pg_loss" in r]                 # the collector's records (validation logs its own)
    assert [r["step"] for r in steps] == [1, 2]
    for k, r in enumerate(steps):
        assert r["training/global_step"] == k + 1
        # 8 prompts x 4 samples over both ranks, prompts of 16-32 and responses of up to 32 tokens: a sum, not a mean
        assert 32 * 17 <= r["perf/total_num_tokens"] <= 32 * 64
        assert 0.0 <= r["critic/score/mean"] <= 1.0 and r["actor/grad_norm"] > 0
        assert {"timing_s/step", "response_length/mean", "perf/throughput"} <= set(r)
        assert abs(r["critic/advantages/mean"]) < 0.2 and abs(r["actor/ppo_kl"]) < 1e-3
    assert any("val-core/all/reward/mean" in r for r in m)
    files = sorted(os.listdir(tmp_path / "dump"))
    assert files == ["step_1_rank_0.json", "step_1_rank_1.json", "step_2_rank_0.json", "step_2_rank_1.json"], files
    rows = json.load(open(tmp_path / "dump" / files[1]))
    assert rows and rows[0]["rank"] == 1 and {"data_source", "input", "output", "score", "global_step"} <= set(rows[0])
    role = tmp_path / "c" / "global_step_2" / "actor_agent_0"
    assert (role / "model_world_size_2_rank_1.pt").exists()
    assert export_main(["--checkpoint", str(role), "--out", str(tmp_path / "hf"), "--dtype", "float32"]) == 0
    cfg = DecoderConfig.from_hf_config(json.load(open(tmp_path / "hf" / "config.json")))
    assert cfg.hidden_size == get_config("tiny").hidden_size
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=123)
    load_hf_weights(model, str(tmp_path / "hf"))
    flat = torch.cat([torch.load(role / f"model_world_size_2_rank_{r}.pt", weights_only=False)["flat"].float()
                      for r in range(2)])
    manifest = json.load(open(role / "manifest.json"))
    for name, p in model.named_parameters():
        o, k, shape = manifest["offsets"][name]
        assert torch.allclose(p.detach().float().reshape(-1), flat[o:o + k], atol=1e-6), name
    os.remove(role / "model_world_size_2_rank_1.pt")
    with pytest.raises(FileNotFoundError):
        export_main(["--checkpoint", str(role), "--out", str(tmp_path / "hf2")])



def test_grpo_with_a_reward_model_worker(tmp_path):
    """``reward_model.enable``: a model with a scalar head scores the responses inside the reward node (its score is
    added to the rule-based one); the worker lives on the same ranks as the policy."""
    out = _run(["reward_model.enable=True", "reward_model.model.arch_preset=tiny", "reward_model.model.random_init=True",
                "reward_model.micro_batch_size_per_gpu=8", "trainer.n_gpus_per_node=1",
                f"trainer.default_local_dir={tmp_path / 'c'}", "trainer.total_training_steps=1", "trainer.save_freq=-1"],
               tmp_path / "log")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log")[0]
    assert m["actor/grad_norm"] > 0
    # the rule scores are 0 / 1; a random scalar head adds real-valued scores, so the mean is no multiple of 1/32
    assert abs(m["critic/score/mean"] * 32 - round(m["critic/score/mean"] * 32)) > 1e-6


def test_custom_pipeline_with_dynamic_batches_and_several_epochs(tmp_path):
    """A user pipeline function (GRPO without the reference node), token-budget micro-batches, two passes over two
    mini-batches per step (so the second pass is off-policy against the stored old log-probs), Adam moments parked in
    host memory between steps."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env_path = os.path.join(root, "examples", "custom_pipeline_example")
    old = os.environ.get("PYTHONPATH", "")
    os.environ["PYTHONPATH"] = env_path + os.pathsep + old
    try:
        out = _run(["dag.custom_pipeline_fn=custom_grpo:grpo_without_reference",
                    "actor_rollout_ref.actor.use_kl_loss=False",
                    "actor_rollout_ref.actor.use_dynamic_bsz=True", "actor_rollout_ref.actor.ppo_max_token_len_per_gpu=160",
                    "actor_rollout_ref.rollout.log_prob_use_dynamic_bsz=True",
                    "actor_rollout_ref.rollout.log_prob_max_token_len_per_gpu=160",
                    "actor_rollout_ref.actor.ppo_epochs=2", "actor_rollout_ref.actor.ppo_mini_batch_size=4",
                    "actor_rollout_ref.actor.shuffle=True", "actor_rollout_ref.actor.fsdp_config.optimizer_offload=True",
                    f"trainer.default_local_dir={tmp_path / 'c'}", "trainer.total_training_steps=2",
                    "trainer.save_freq=-1"], tmp_path / "log")
    finally:
        os.environ["PYTHONPATH"] = old
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log")
    assert [r["step"] for r in m] == [1, 2]
    for r in m:
        assert r["actor/grad_norm"] > 0 and "timing_s/reference_log_prob" not in r
        assert 0.0 < abs(r["actor/ppo_kl"]) < 0.05          # the policy moved between the passes, a little


@pytest.mark.parametrize("manager", ["naive", "batch"])
def test_user_reward_function_from_a_file(tmp_path, manager):
    """``custom_reward_function.path / name``: per-sample signature with the ``naive`` manager, one call per batch with
    the ``batch`` manager; the scores the file returns are the ones that reach the metrics."""
    f = tmp_path / "my_reward.py"
    f.write_text(
        "def per_sample(data_source, solution_str, ground_truth, extra_info=None):\n"
        "    return 0.25\n\n"
        "def per_batch(data_sources, solution_strs, ground_truths, extra_infos=None):\n"
        "    assert len(data_sources) == len(solution_strs) == len(ground_truths) > 1\n"
        "    return [0.75] * len(solution_strs)\n")
    name, want = ("per_sample", 0.25) if manager == "naive" else ("per_batch", 0.75)
    out = _run([f"custom_reward_function.path={f}", f"custom_reward_function.name={name}",
                f"reward_model.reward_manager={manager}", "trainer.n_gpus_per_node=1",
                f"trainer.default_local_dir={tmp_path / 'c'}", "trainer.total_training_steps=1", "trainer.save_freq=-1"],
               tmp_path / "log")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log")[0]
    assert m["critic/score/mean"] == pytest.approx(want) and m["critic/score/max"] == pytest.approx(want)


def test_validation_only_run(tmp_path):
    """``trainer.val_only`` with ``val_before_train``: the job validates once, logs the validation metrics at step 0
    and stops without a training step."""
    out = _run(["trainer.val_before_train=True", "trainer.val_only=True", "trainer.test_freq=1",
                "trainer.n_gpus_per_node=1", f"trainer.default_local_dir={tmp_path / 'c'}",
                "trainer.total_training_steps=3", "trainer.save_freq=-1"], tmp_path / "log")
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    m = _metrics(tmp_path / "log")
    assert len(m) == 1 and m[0]["step"] == 0 and "val-core/all/reward/mean" in m[0] and "actor/pg_loss" not in m[0]
