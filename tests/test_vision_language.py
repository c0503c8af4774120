"""Vision-language path on CPU: image processor, placeholder expansion, multimodal rope in the rollout engine and
in the training forward (their log-probs must agree), and a GRPO step with image prompts."""
import json
import os
import subprocess
import sys

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


def test_vl_grpo_pipeline(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, OMP_NUM_THREADS="2", SIIRL_LOG_DIR=str(tmp_path / "log"))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    args = ["algorithm.adv_estimator=grpo", "data.synthetic=vl", "data.synthetic_image_size=56", "data.synthetic_size=64",
            "data.synthetic_min_prompt=8", "data.synthetic_max_prompt=16", "data.max_prompt_length=48",
            "data.max_response_length=16", "data.train_batch_size=4", "actor_rollout_ref.model.arch_preset=tiny-vl",
            "actor_rollout_ref.rollout.n=4", "actor_rollout_ref.rollout.max_num_seqs=16",
            "actor_rollout_ref.actor.ppo_mini_batch_size=4", "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8",
            "actor_rollout_ref.actor.use_kl_loss=True", "trainer.n_gpus_per_node=1", "trainer.device=cpu",
            "trainer.val_before_train=False", "trainer.logger=['jsonl']", "trainer.total_training_steps=2",
            "trainer.save_freq=-1"]
    out = subprocess.run([sys.executable, "-m", "siirl_b200.main_dag", *args], env=env, cwd=root, capture_output=True,
                         text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    with open(tmp_path / "log" / "metrics.jsonl") as f:
        m = [json.loads(line) for line in f]
    assert [r["step"] for r in m] == [1, 2] and any(r["actor/grad_norm"] > 0 for r in m)
