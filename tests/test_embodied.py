"""Embodied path on CPU: action tokens, image twins, synthetic environment, vector envs, reward shaping,
trajectory <-> row views, and the embodied pipeline end to end on one rank."""
import asyncio
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from siirl_b200.data_coordinator.protocol import Batch
from siirl_b200.engine.actor.embodied_actor import (executed_calls, flatten_trajectories, scatter_steps,
                                                    trajectory_response_mask)
from siirl_b200.environment.embodied import DummyVectorEnv, SubprocVectorEnv, make_environment
from siirl_b200.models.embodied.vla import ActionTokenizer
from siirl_b200.ops.image import (center_crop_box, raster_synth_env_reference, resize_bilinear_reference)
from siirl_b200.utils.reward_score.embodied import compute_embodied_reward, dbscan


def test_action_tokenizer_roundtrip_and_clamp():
    tok = ActionTokenizer(vocab_size=1024)
    a = torch.linspace(-1, 1, 101)
    ids = tok.encode(a)
    assert ids.min() >= tok.first_action_token and ids.max() <= 1023
    back = tok.decode(ids)
    assert (back - a).abs().max() <= 2.0 / 255 + 1e-6
    assert -1.0 <= float(tok.decode(torch.tensor([5]))) <= 1.0           # non-action ids clamp into the range


def test_resize_identity_and_crop_box():
    img = np.random.RandomState(0).randint(0, 255, (2, 16, 16, 3), dtype=np.uint8)
    assert np.array_equal(resize_bilinear_reference(img, (16, 16)), img)
    flat = np.full((1, 32, 32, 3), 77, dtype=np.uint8)
    assert (resize_bilinear_reference(flat, (8, 8), center_crop_box(32, 32, 0.9)) == 77).all()
    y0, x0, h, w = center_crop_box(100, 200, 0.81)
    assert abs(h - 90) < 1e-4 and abs(w - 180) < 1e-4 and abs(y0 - 5) < 1e-4 and abs(x0 - 10) < 1e-4


def test_raster_places_goal_and_gripper():
    st = np.array([[0.25, 0.25, 0.75, 0.75, 1.0, 0, 0, 0]], dtype=np.float32)
    img = raster_synth_env_reference(st, 64, 64)[0]
    assert tuple(img[48, 48]) == (30, 200, 60)            # goal centre (u = v = 0.75)
    assert img[16, 16, 0] > 150 and img[16, 16, 1] < 80   # gripper is red
    assert img[2, 60, 0] < 80                             # background


def test_synthetic_env_reaches_goal_with_oracle_policy():
    env = make_environment("synthetic", num_envs=4, max_steps=40, image_size=32)
    obs = asyncio.new_event_loop().run_until_complete(env.reset([0, 1, 2, 3], [0, 0, 0, 0]))
    assert obs[0]["image"].shape == (32, 32, 3) and "target" in obs[0]["task_description"]
    loop = asyncio.new_event_loop()
    for _ in range(40):
        d = env.state[:, 2:4] - env.state[:, :2]
        act = np.zeros((4, 7), dtype=np.float32)
        act[:, :2] = np.clip(d / env.action_scale, -1, 1)
        obs = loop.run_until_complete(env.step(act))
        if all(o["done"] for o in obs):
            break
    assert all(o["success"] for o in obs) and max(o["step"] for o in obs) < 40
    # same (task, trial) -> same layout
    a = loop.run_until_complete(env.reset([3, 3, 3, 3], [1, 1, 2, 2]))
    assert np.allclose(a[0]["state"], a[1]["state"]) and not np.allclose(a[1]["state"], a[2]["state"])


class _Counter:
    def __init__(self, start):
        self.x = start

    def reset(self):
        return {"x": self.x}

    def step(self, a):
        self.x += int(a)
        return {"x": self.x}, float(self.x), self.x >= 5, {}


def _make_counter(start):
    return _Counter(start)


def test_vector_envs_agree():
    import functools
    fns = [functools.partial(_make_counter, s) for s in (0, 3)]
    for cls in (DummyVectorEnv, SubprocVectorEnv):
        v = cls(fns)
        assert [o["x"] for o in v.reset()] == [0, 3]
        obs, rew, done, info = v.step([2, 2])
        assert [o["x"] for o in obs] == [2, 5] and rew.tolist() == [2.0, 5.0] and done.tolist() == [False, True]
        obs, rew, done, info = v.step([1], ids=[0])
        assert obs[0]["x"] == 3
        v.close()


def test_dbscan_and_shaped_reward():
    x = np.array([[0, 0], [0.1, 0], [0, 0.1], [5, 5], [5.1, 5], [20, 20]], dtype=np.float64)
    lab = dbscan(x, eps=0.5, min_samples=2)
    assert lab[0] == lab[1] == lab[2] and lab[3] == lab[4] and lab[0] != lab[3] and lab[5] == -1
    emb = torch.tensor([[0.0, 0.0], [0.1, 0.0], [0.2, 0.1], [3.0, 3.0], [9.0, 9.0]])
    ok = torch.tensor([1, 1, 0, 0, 0])
    s = compute_embodied_reward(emb, ok, ["t"] * 5)
    assert s[0] == s[1] == 1.0 and 0.0 < s[4] < s[3] < s[2] <= 0.6
    assert compute_embodied_reward(emb, torch.zeros(5), ["t"] * 5) == [0.0] * 5     # no success: no shaping


def test_flatten_and_scatter_trajectories():
    B, L, chunk, atl, P = 3, 4, 2, 7, 5
    A = chunk * atl
    finish = torch.tensor([8, 3, 1])
    assert executed_calls(finish, L, chunk).sum(1).tolist() == [4, 2, 1]
    mask = trajectory_response_mask(finish, L, chunk, atl)
    assert mask.sum(1).tolist() == [56, 21, 7]
    data = Batch({"responses": torch.arange(B * L * A).reshape(B, L, A),
                  "step_input_ids": torch.ones(B, L, P, dtype=torch.long),
                  "step_attention_mask": torch.ones(B, L, P, dtype=torch.long),
                  "images": torch.zeros(B, L, 4, 4, 3, dtype=torch.uint8), "finish_step": finish,
                  "response_mask": mask, "advantages": torch.randn(B, L * A)})
    rows, bi, li = flatten_trajectories(data, chunk)
    assert rows.batch_size == 7 and rows["input_ids"].shape == (7, P + A)
    assert rows["response_mask"][5].tolist() == [1] * 7 + [0] * 7       # trajectory 1, call 1: second action not run
    back = scatter_steps(rows["advantages"], bi, li, B, L)
    run_tok = executed_calls(finish, L, chunk).repeat_interleave(A, 1)
    assert torch.equal(back[run_tok], data["advantages"][run_tok]) and float(back[~run_tok].abs().sum()) == 0


@pytest.mark.parametrize("policy,cameras", [("native-vla", 1), ("openvla-oft", 1), ("openvla-oft", 2)])
def test_embodied_pipeline_two_steps(tmp_path, policy, cameras):
    """``native-vla``: the framework's VL decoder decoding action tokens one by one; ``openvla-oft``: the Prismatic
    backbone (DINOv2 + SigLIP towers) with one-pass chunk decoding and scoring over the action bins.  ``cameras=2``:
    third-person and wrist view per step (``num_images_in_input``)."""
    preset = "tiny-vl" if policy == "native-vla" else "tiny-openvla"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, OMP_NUM_THREADS="2", SIIRL_LOG_DIR=str(tmp_path / "log"))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    args = ["algorithm.adv_estimator=grpo", "algorithm.workflow_type=embodied", "data.synthetic=embodied",
            "data.synthetic_size=32", "data.max_prompt_length=32", "data.max_response_length=32",
            f"actor_rollout_ref.embodied.num_images_in_input={cameras}",
            "data.train_batch_size=4", f"actor_rollout_ref.model.arch_preset={preset}", "actor_rollout_ref.rollout.n=4",
            f"actor_rollout_ref.embodied.embodied_type={policy}",
            "actor_rollout_ref.rollout.max_num_seqs=16", "actor_rollout_ref.actor.ppo_mini_batch_size=4",
            "actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=8", f"actor_rollout_ref.actor.embodied_type={policy}",
            "actor_rollout_ref.embodied.env.env_type=synthetic", "actor_rollout_ref.embodied.env.num_envs=8",
            "actor_rollout_ref.embodied.env.max_steps=8", "actor_rollout_ref.embodied.env.env_kwargs={success_radius: 0.3}",
            "actor_rollout_ref.embodied.action_chunks_len=2", "actor_rollout_ref.embodied.policy_image_size=56",
            "actor_rollout_ref.embodied.video_num_frames=2", "actor_rollout_ref.embodied.embedding_img_size=64",
            "reward_model.reward_manager=embodied", "trainer.n_gpus_per_node=1", "trainer.device=cpu",
            "trainer.val_before_train=False", "trainer.logger=['jsonl']", "trainer.total_training_steps=2",
            "trainer.save_freq=-1"]
    out = subprocess.run([sys.executable, "-m", "siirl_b200.main_dag", *args], env=env, cwd=root, capture_output=True,
                         text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    with open(tmp_path / "log" / "metrics.jsonl") as f:
        m = [json.loads(line) for line in f]
    assert [r["step"] for r in m] == [1, 2]
    assert all(0.0 <= r["critic/score/mean"] <= 1.0 for r in m)
    assert any(r["actor/grad_norm"] > 0 for r in m)          # some group mixes successes and failures
    assert m[0]["embodied_sampling/initial_trajectories"] == 16.0
    assert m[0]["response_length/max"] <= 8 * 7
    assert abs(m[0]["actor/ppo_kl"]) < 1e-3                  # scoring sees the same images in the same layout as rollout


@pytest.mark.parametrize("preset", ["tiny-openvla", "tiny-vl"])
def test_oft_l1_regression_head_and_proprio(preset):
    """OpenVLA-OFT's continuous path: the proprioception pseudo-token changes the prediction, the head learns a fixed
    target through an L1 loss (gradients reach head, projector and decoder), and un-normalisation follows the dataset
    statistics."""
    from siirl_b200.models.config import get_config
    from siirl_b200.models.decoder import build_model
    from siirl_b200.models.embodied.action_heads import (L1RegressionActionHead, ProprioProjector, normalize_proprio,
                                                        unnormalize_actions)
    from siirl_b200.models.embodied.vla import VLAProcessor, oft_action_hidden, oft_continuous_actions

    class Tok:
        def encode(self, s):
            return [5 + (ord(c) % 50) for c in s][:12]

    cfg = get_config(preset)
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=2)
    proc = VLAProcessor(cfg, Tok(), image_size=56)
    N, chunk, adim, pdim = 2, 3, 7, 8
    head = L1RegressionActionHead(cfg.hidden_size, adim, head_hidden=64, blocks=2, dtype=torch.float32, seed=1)
    proj = ProprioProjector(pdim, cfg.hidden_size, dtype=torch.float32, seed=2)
    g = torch.Generator().manual_seed(0)
    images = torch.randint(0, 255, (N, proc.image_size, proc.image_size, 3), generator=g, dtype=torch.uint8)
    prompts = [proc.prompt_ids("pick up the block"), proc.prompt_ids("open the drawer")]
    stats = {"q01": [-2.0] * adim, "q99": [2.0] * adim, "mask": [True] * (adim - 1) + [False]}
    state = normalize_proprio(torch.randn(N, pdim, generator=g) * 3, {"q01": [-3.0] * pdim, "q99": [3.0] * pdim})
    assert state.abs().max() <= 1.0
    a0 = oft_continuous_actions(model, proc, prompts, images, head, chunk)
    a1 = oft_continuous_actions(model, proc, prompts, images, head, chunk, proprio=state, proprio_projector=proj)
    assert a0.shape == (N, chunk, adim) and (a0 - a1).abs().max() > 1e-6          # the state token is seen
    un = oft_continuous_actions(model, proc, prompts, images, head, chunk, norm_stats=stats)
    assert torch.allclose(un[..., :-1], 0.5 * (a0[..., :-1] + 1) * 4.0 - 2.0, atol=1e-5)
    assert torch.allclose(un[..., -1], a0[..., -1])                              # masked dimension stays as predicted
    assert torch.allclose(unnormalize_actions(torch.zeros(adim), stats), torch.zeros(adim), atol=1e-6)
    # a few L1 steps on a fixed target
    target = torch.rand(N, chunk, adim, generator=g) * 2 - 1
    params = list(head.parameters()) + list(proj.parameters()) + [p for p in model.parameters() if p.requires_grad]
    opt = torch.optim.Adam(params, lr=5e-4)
    losses = []
    for _ in range(20):
        opt.zero_grad()
        for p in model.parameters():
            if getattr(p, "main_grad", None) is not None:
                p.main_grad.zero_()
        h = oft_action_hidden(model, proc, prompts, images, chunk * adim, state, proj)
        loss = head.l1_loss(h, target)
        loss.backward()
        for p in model.parameters():                      # the decoder's custom ops accumulate into ``main_grad``
            if p.grad is None and getattr(p, "main_grad", None) is not None:
                p.grad = p.main_grad.to(p.dtype).clone()
        losses.append(float(loss.detach()))
        opt.step()
    assert proj.fc1_weight.grad is not None and proj.fc1_weight.grad.abs().sum() > 0
    assert min(losses[-3:]) < 0.7 * losses[0], losses


def test_oft_diffusion_head_trains_and_samples():
    """OpenVLA-OFT's diffusion head: the noise-prediction loss falls on a fixed target, sampling walks the DDIM steps
    (one decoder forward each) and is reproducible from the generator."""
    from siirl_b200.models.config import get_config
    from siirl_b200.models.decoder import build_model
    from siirl_b200.models.embodied.action_heads import DDIMSchedule, DiffusionActionHead
    from siirl_b200.models.embodied.vla import VLAProcessor, oft_action_hidden, oft_diffusion_actions

    class Tok:
        def encode(self, s):
            return [5 + (ord(c) % 50) for c in s][:12]

    sch = DDIMSchedule(100)
    assert sch.alphas_cumprod[0] > 0.99 and sch.alphas_cumprod[-1] < 1e-3 and (sch.alphas_cumprod.diff() < 0).all()
    steps = sch.inference_steps(10)
    assert steps[0][0] == 99 and steps[-1] == (0, -1) and len(steps) == 10
    x0 = torch.rand(4, 3, 7) * 2 - 1
    eps = torch.randn(4, 3, 7)
    xt = sch.add_noise(x0, eps, torch.tensor([50, 50, 50, 50]))
    assert torch.allclose(sch.step(eps, 50, -1, xt), x0, atol=1e-4)        # the true noise recovers the clean sample
    cfg = get_config("tiny-openvla")
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=2)
    proc = VLAProcessor(cfg, Tok(), image_size=56)
    N, chunk, adim = 2, 2, 7
    head = DiffusionActionHead(cfg.hidden_size, adim, head_hidden=64, num_inference_steps=4, dtype=torch.float32, seed=1)
    g = torch.Generator().manual_seed(0)
    images = torch.randint(0, 255, (N, proc.image_size, proc.image_size, 3), generator=g, dtype=torch.uint8)
    prompts = [proc.prompt_ids("pick up the block"), proc.prompt_ids("open the drawer")]
    a = oft_diffusion_actions(model, proc, prompts, images, head, chunk, generator=torch.Generator().manual_seed(5))
    b = oft_diffusion_actions(model, proc, prompts, images, head, chunk, generator=torch.Generator().manual_seed(5))
    assert a.shape == (N, chunk, adim) and torch.equal(a, b) and a.abs().max() <= 1.0 + 1e-5
    target = torch.rand(N, chunk, adim, generator=g) * 2 - 1
    opt = torch.optim.Adam(head.parameters(), lr=2e-3)
    losses = []
    for it in range(30):
        opt.zero_grad()
        t = torch.randint(0, 100, (N,), generator=g)
        noise = torch.randn(N, chunk, adim, generator=g)
        noisy = head.schedule.add_noise(target, noise, t)
        h = oft_action_hidden(model, proc, prompts, images, chunk * adim, pseudo_tokens=[head.time_embedding(t)],
                              action_embeds=head.project_noisy_actions(noisy))
        loss = ((head.predict_noise(h) - noise) ** 2).mean()
        loss.backward()
        losses.append(float(loss.detach()))
        opt.step()
    assert head.act_in_weight.grad is not None and head.time_weight.grad.abs().sum() > 0
    assert sum(losses[-5:]) / 5 < 0.85 * sum(losses[:5]) / 5, losses


def test_action_statistics_of_a_checkpoint(tmp_path):
    """``dataset_statistics.json`` (or ``norm_stats`` in config.json) + ``embodied.unnorm_key``, with the
    ``_no_noops`` fallback; no statistics -> ``None``."""
    import json as _json

    from siirl_b200.models.embodied.action_heads import load_action_norm_stats, unnormalize_actions
    assert load_action_norm_stats(None, "libero_goal") is None and load_action_norm_stats(str(tmp_path), "x") is None
    st = {"libero_goal_no_noops": {"action": {"q01": [-0.5] * 7, "q99": [0.5] * 7, "mask": [True] * 6 + [False]}}}
    (tmp_path / "dataset_statistics.json").write_text(_json.dumps(st))
    got = load_action_norm_stats(str(tmp_path), "libero_goal")
    assert got["q99"][0] == 0.5
    a = unnormalize_actions(torch.tensor([[1.0] * 7, [-1.0] * 7]), got)
    assert torch.allclose(a[0, :6], torch.full((6,), 0.5), atol=1e-6) and a[0, 6] == 1.0 and a[1, 6] == -1.0
    with pytest.raises(KeyError):
        load_action_norm_stats(str(tmp_path), "bridge_orig")
    other = tmp_path / "b"
    other.mkdir()
    (other / "config.json").write_text(_json.dumps({"norm_stats": {"bridge_orig": {"action": {"q01": [0.0], "q99": [1.0]}}}}))
    assert load_action_norm_stats(str(other), "bridge_orig")["q99"] == [1.0]


@pytest.mark.parametrize("preset", ["tiny-vl", "tiny-openvla"])
def test_processor_with_two_cameras(preset):
    """Two views per step: stacked along the height in storage, one placeholder run and one rope block per view; the
    second view changes the hidden states of the text that follows."""
    from siirl_b200.models.config import get_config
    from siirl_b200.models.decoder import build_model
    from siirl_b200.models.embodied.vla import VLAProcessor
    from siirl_b200.ops.attention import SeqInfo

    class Tok:
        def encode(self, s):
            return [5 + (ord(c) % 50) for c in s][:12]

    cfg = get_config(preset)
    model = build_model(cfg, dtype=torch.float32, device="cpu", seed=2)
    one, two = VLAProcessor(cfg, Tok(), image_size=56), VLAProcessor(cfg, Tok(), image_size=56, num_images=2)
    assert two.image_tokens == 2 * one.tokens_per_image
    p = two.prompt_ids("pick up the block")
    assert len(p) == len(one.prompt_ids("pick up the block")) + one.tokens_per_image
    g = torch.Generator().manual_seed(0)
    frames = torch.randint(0, 255, (1, 2, 64, 64, 3), generator=g, dtype=torch.uint8)
    imgs = two.resize(frames)
    S = two.image_size
    assert imgs.shape == (1, 2 * S, S, 3) and torch.equal(imgs[:, :S], one.resize(frames[:, 0]))

    def hidden(images):
        pv, grid = two.patchify(images, torch.float32)
        info = SeqInfo([len(p)])
        pos = two.rope_layout(len(p))[0] if two.prismatic is None else info.positions
        first = torch.tensor([0])
        return model.forward_hidden(torch.tensor(p), pos, info, pixel_values=pv, image_grid_thw=grid,
                                    image_mask=two.image_mask(first, len(p)))
    assert two.patchify(imgs, torch.float32)[1].shape[0] == 2
    with torch.no_grad():
        a = hidden(imgs)
        other = imgs.clone()
        other[:, S:] = 255 - other[:, S:]                                  # change the wrist view only
        b = hidden(other)
    assert a.shape[0] == len(p) and (a[-1] - b[-1]).abs().max() > 1e-6
    mm = two.mm_inputs(imgs, [len(p)], torch.float32)[0]
    assert mm["image_grid_thw"].shape[0] == 2 and mm["rope_positions"].shape[1] == len(p)
