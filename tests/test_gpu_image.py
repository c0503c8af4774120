"""CUDA image kernels of the embodied path against their numpy twins, and a multimodal rollout on the GPU."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_resize_bilinear_matches_numpy_twin():
    from siirl_b200.ops.image import center_crop_box, resize_bilinear, resize_bilinear_reference
    img = np.random.RandomState(0).randint(0, 256, (5, 256, 256, 3), dtype=np.uint8)
    for out_hw, crop in (((224, 224), None), ((224, 224), center_crop_box(256, 256, 0.9)), ((96, 160), None)):
        want = resize_bilinear_reference(img, out_hw, crop)
        got = resize_bilinear(torch.from_numpy(img).cuda(), out_hw, crop).cpu().numpy()
        diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
        assert diff.max() <= 1 and (diff > 0).mean() < 0.05          # rounding of .5 may differ by one level


def test_raster_matches_numpy_twin():
    from siirl_b200.ops.image import raster_synth_env, raster_synth_env_reference
    rs = np.random.RandomState(1)
    st = np.zeros((7, 8), dtype=np.float32)
    st[:, :4] = rs.uniform(0.1, 0.9, (7, 4))
    st[:, 4] = rs.randint(0, 2, 7)
    want = raster_synth_env_reference(st, 256, 256)
    got = raster_synth_env(torch.from_numpy(st).cuda(), 256, 256).cpu().numpy()
    diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert (diff > 1).mean() < 1e-3                                  # edge pixels of the discs may flip


def test_embodied_rollout_on_gpu_and_logprob_consistency():
    """Closed-loop episodes with the tiny VL policy; log-probs recomputed by the training path on the executed calls
    must match the rollout's (same multimodal rope layout, same image patches)."""
    from siirl_b200.data_coordinator.protocol import Batch
    from siirl_b200.engine.workers import ActorRolloutRefWorker
    from siirl_b200.params.parser import parse_config
    cfg = parse_config(["actor_rollout_ref.model.arch_preset=tiny-vl-gpu", "actor_rollout_ref.rollout.n=1",
                        "actor_rollout_ref.rollout.max_num_seqs=16", "actor_rollout_ref.actor.embodied_type=native-vla",
                        "actor_rollout_ref.embodied.env.env_type=synthetic", "actor_rollout_ref.embodied.env.num_envs=4",
                        "actor_rollout_ref.embodied.env.max_steps=6", "actor_rollout_ref.embodied.action_chunks_len=2",
                        "actor_rollout_ref.embodied.policy_image_size=112", "actor_rollout_ref.embodied.temperature=1.0",
                        "actor_rollout_ref.embodied.video_num_frames=2", "actor_rollout_ref.embodied.embedding_img_size=64",
                        "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8",
                        "actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=8", "trainer.n_gpus_per_node=1"])
    w = ActorRolloutRefWorker(cfg.actor_rollout_ref, "actor_rollout", None, torch.device("cuda"), None, 1, None)
    w.init_model()
    prompts = Batch({"task_id": torch.arange(4), "trial_id": torch.zeros(4, dtype=torch.long)}, {}, {"global_steps": 0})
    out = w.generate_sequences(prompts)
    B, L, A = out["responses"].shape
    assert (B, L, A) == (4, 3, 14) and out["images"].shape == (4, 3, 112, 112, 3)
    assert out["vjepa_embedding"].shape[0] == 4 and torch.isfinite(out["vjepa_embedding"]).all()
    assert int(out["images"][0, 0].float().std()) > 0                    # frames were rendered and resized
    out.meta["temperature"] = 1.0
    out = w.compute_log_prob(out)
    m = out["response_mask"].bool()
    d = (out["old_log_probs"] - out["rollout_log_probs"])[m].abs()
    assert float(d.mean()) < 0.05 and float(d.max()) < 0.5, (float(d.mean()), float(d.max()))
