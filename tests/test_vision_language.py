"""Vision-language path on CPU: image processor, placeholder expansion, multimodal rope in the rollout engine and
in the training forward (their log-probs must agree), and a GRPO step with image prompts."""
import json
import os
import subprocess
import sys

import pytest
import torch

from siirl_b200.models.config import get_config
from siirl_b200.models.vision_processor import VLProcessor, smart_resize


def test_smart_resize_bounds_and_multiples():
    for h, w in ((448, 448), (100, 37), (2000, 3000), (20, 20)):
        h2, w2 = smart_resize(h, w, 28, 32 * 32, 768 * 768)
        assert h2 % 28 == 0 and w2 % 28 == 0 and 32 * 32 <= h2 * w2 <= 768 * 768 + 28 * 28
    assert smart_resize(448, 448, 28, 1024, 768 * 768) == (448, 448)


def test_processor_expands_placeholders_and_orders_patches():
    cfg = get_config("tiny-vl")
    proc = VLProcessor(cfg, 28 * 28, 112 * 112)
    img = torch.arange(56 * 84 * 3, dtype=torch.float32).reshape(56, 84, 3) % 255
    out = proc([5, cfg.image_token_id, 6], [img.to(torch.uint8)])
    gh, gw = out["image_grid_thw"][0, 1:].tolist()
    assert (gh, gw) == (4, 6) and out["pixel_values"].shape == (24, 3 * 2 * 14 * 14)
    n_img = gh * gw // 4
    assert out["input_ids"] == [5] + [cfg.image_token_id] * n_img + [6]
    # first four patches are the 2x2 merge unit of the top-left corner: rows 0..27, columns 0..27
    p = out["pixel_values"].reshape(24, 3, 2, 14, 14)
    assert torch.equal(p[:, :, 0], p[:, :, 1])                      # still images: the frame is duplicated in time
    pos, delta = proc.rope(torch.tensor(out["input_ids"]), out["image_grid_thw"])
    assert pos.shape == (3, len(out["input_ids"])) and delta == n_img - max(gh, gw) // 2


def test_vl_rollout_and_training_logprobs_agree():
    from siirl_b200.data_coordinator import preprocess_dataloader
    from siirl_b200.data_coordinator.dataloader import DataLoaderNode, load_tokenizer
    from siirl_b200.engine.workers import ActorRolloutRefWorker
    from siirl_b200.params.parser import parse_config
    cfg = parse_config(["data.synthetic=vl", "data.synthetic_image_size=84", "data.synthetic_size=16",
                        "data.synthetic_min_prompt=8", "data.synthetic_max_prompt=16", "data.max_prompt_length=64",
                        "data.max_response_length=12", "data.train_batch_size=4",
                        "actor_rollout_ref.model.arch_preset=tiny-vl", "actor_rollout_ref.rollout.n=2",
                        "actor_rollout_ref.rollout.max_num_seqs=16", "actor_rollout_ref.rollout.prompt_length=64",
                        "actor_rollout_ref.rollout.response_length=12",
                        "actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=8", "trainer.n_gpus_per_node=1",
                        "trainer.device=cpu"])
    tok = load_tokenizer(None, 1024)
    batch = preprocess_dataloader(DataLoaderNode(cfg, tok, None, 1, 0, 1).run(), 2)
    assert len(batch.non_tensors["multi_modal_inputs"]) == 8
    w = ActorRolloutRefWorker(cfg.actor_rollout_ref, "actor_rollout", None, torch.device("cpu"), None, 1, tok)
    w.init_model()
    batch.meta.update({"eos_token_id": None, "pad_token_id": 0, "global_steps": 0})
    out = w.generate_sequences(batch)
    out.meta["temperature"] = 1.0
    out = w.compute_log_prob(out)
    m = out["response_mask"].bool()
    assert (out["old_log_probs"] - out["rollout_log_probs"])[m].abs().max().item() < 1e-4


@pytest.mark.parametrize("ulysses", [1, 2])
def test_vl_grpo_pipeline(tmp_path, ulysses):
    """GRPO on the vision-language decoder; with ``ulysses=2`` two ranks share every packed stream (image features
    are written over the whole stream on both ranks before the rows are divided)."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, OMP_NUM_THREADS="2", SIIRL_LOG_DIR=str(tmp_path / "log"))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    args = ["algorithm.adv_estimator=grpo", "data.synthetic=vl", "data.synthetic_image_size=56", "data.synthetic_size=64",
            "data.synthetic_min_prompt=8", "data.synthetic_max_prompt=16", "data.max_prompt_length=48",
            "data.max_response_length=16", "data.train_batch_size=4", "actor_rollout_ref.model.arch_preset=tiny-vl",
            "actor_rollout_ref.rollout.n=4", "actor_rollout_ref.rollout.max_num_seqs=16",
            "actor_rollout_ref.actor.ppo_mini_batch_size=4", "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8",
            "actor_rollout_ref.actor.use_kl_loss=True", f"trainer.n_gpus_per_node={ulysses}", "trainer.device=cpu",
            f"actor_rollout_ref.actor.ulysses_sequence_parallel_size={ulysses}",
            "trainer.val_before_train=False", "trainer.logger=['jsonl']", "trainer.total_training_steps=2",
            "trainer.save_freq=-1"]
    out = subprocess.run([sys.executable, "-m", "siirl_b200.main_dag", *args], env=env, cwd=root, capture_output=True,
                         text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    with open(tmp_path / "log" / "metrics.jsonl") as f:
        m = [json.loads(line) for line in f]
    assert [r["step"] for r in m] == [1, 2] and any(r["actor/grad_norm"] > 0 for r in m)
    assert abs(m[0]["actor/ppo_kl"]) < 1e-3          # training forward = scoring forward on the first, on-policy step


def test_video_inputs_sampling_patching_and_forward():
    """Videos: frame sampling rules, resize to multiples of 28, temporal patches (grid t > 1), placeholder expansion,
    3-row rope positions over the (t, h, w) grid, and a forward pass through the vision tower and the decoder."""
    import numpy as np

    from siirl_b200.data_coordinator.dataloader.vision_utils import process_image, process_video, sample_frame_indices
    from siirl_b200.models.config import get_config
    from siirl_b200.models.decoder import build_model
    from siirl_b200.models.vision_processor import VLProcessor
    from siirl_b200.ops.attention import SeqInfo
    frames = [np.random.randint(0, 255, (60, 90, 3), dtype=np.uint8) for _ in range(5)]
    v = process_video({"video": frames}, min_pixels=28 * 28, max_pixels=56 * 56)
    assert v.shape[0] == 6 and v.shape[2] % 28 == 0 and v.shape[3] % 28 == 0       # odd frame count is padded to even
    clip = np.random.rand(40, 3, 64, 64).astype(np.float32)
    v2 = process_video({"video": clip, "nframes": 8}, min_pixels=28 * 28, max_pixels=56 * 56)
    assert tuple(v2.shape) == (8, 3, 56, 56)
    idx = sample_frame_indices(300, 30.0, fps=2.0)                                  # 10 s at 2 frames per second
    assert len(idx) == 20 and idx[0] == 0 and idx[-1] == 299
    assert len(sample_frame_indices(30, 30.0, fps=2.0)) == 4                        # never fewer than min_frames
    with pytest.raises(ValueError):
        process_video({"video": clip}, nframes=4, fps=1.0)
    img = process_image(np.random.randint(0, 255, (100, 37, 3), dtype=np.uint8), max_pixels=56 * 56, min_pixels=28 * 28)
    assert img.shape[1] % 28 == 0 and img.shape[2] % 28 == 0 and float(img.max()) <= 1.0
    cfg = get_config("tiny-vl")
    proc = VLProcessor(cfg, 28 * 28, 56 * 56)
    out = proc([5, 6, cfg.image_token_id, 7], [], [v2])
    t, gh, gw = out["image_grid_thw"][0].tolist()
    assert t == 8 // cfg.vision.temporal_patch_size and out["pixel_values"].shape[0] == t * gh * gw
    assert len(out["input_ids"]) == 3 + t * gh * gw // cfg.vision.spatial_merge_size ** 2
    ids = torch.tensor(out["input_ids"])
    pos, delta = proc.rope(ids, out["image_grid_thw"])
    assert pos.shape == (3, ids.numel()) and int(pos[0].max()) < ids.numel()       # the time row advances per grid t
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=0)
    h = model.forward_hidden(ids, pos, SeqInfo([ids.numel()]), pixel_values=out["pixel_values"],
                             image_grid_thw=out["image_grid_thw"])
    assert h.shape == (ids.numel(), cfg.hidden_size) and torch.isfinite(h).all()
