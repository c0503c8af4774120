"""Embodied rollout: closed-loop episodes of a VLA policy in a batched environment.

Contract of the reference's ``EmbodiedHFRollout`` (siirl/engine/rollout/embodied_rollout.py:135-673): reset the
environments to the (task, trial) of each row, then until every episode ends: camera frame -> crop/resize -> policy
generates one chunk of ``action_chunks_len`` actions as ``action_chunks_len * action_token_len`` tokens ->
environment executes the chunk; finally the episode video is embedded for the reward.  Native design:

* frames stay on the device: the synthetic environment rasterises into a device buffer, the crop+resize kernel
  writes the policy input, patches go straight into the prefill of the paged engine;
* a chunk is one ``RolloutEngine.generate`` call (prefill of image+text, then CUDA-graph decode steps), only for
  environments that are still running;
* the output keeps trajectories un-flattened (``responses [B, L, A]``) with ``finish_step`` / ``complete`` and a
  token mask, which is what the embodied reward manager, filter, advantage and actor consume."""
from __future__ import annotations

import asyncio
import time
from typing import List, Optional

import torch

from ...data_coordinator.protocol import Batch
from ...environment.embodied import make_environment
from ...models.embodied.vla import ActionTokenizer, VLAProcessor
from ..actor.embodied_actor import trajectory_response_mask
from .native_engine import RolloutEngine, SamplingParams


class EmbodiedRollout:
    def __init__(self, engine: RolloutEngine, model_config, tokenizer, embodied_cfg, device, seed: int = 0,
                 video_embedder=None, model_path: Optional[str] = None):
        self.engine, self.cfg, self.device = engine, embodied_cfg, torch.device(device)
        self.model_config = model_config
        self.actions = ActionTokenizer(model_config.action_vocab_size or model_config.vocab_size,
                                       n_bins=model_config.n_action_bins)
        self.num_images = max(1, int(getattr(embodied_cfg, "num_images_in_input", 1) or 1))
        self.proc = VLAProcessor(model_config, tokenizer, image_size=getattr(embodied_cfg, "policy_image_size", 224),
                                 center_crop=embodied_cfg.center_crop, num_images=self.num_images)
        self.chunk = embodied_cfg.action_chunks_len
        self.atl = embodied_cfg.action_token_len
        self.seed = seed
        from ...models.embodied.vla import uses_parallel_decode
        self.parallel = uses_parallel_decode(embodied_cfg, model_config)
        self.env = None
        self.video_embedder = video_embedder
        # fine-tuned checkpoints carry the action statistics of their dataset: decoded bin centres in [-1, 1] become
        # robot units before they reach the environment (``embodied.unnorm_key`` names the dataset)
        from ...models.embodied.action_heads import load_action_norm_stats
        self.norm_stats = load_action_norm_stats(model_path, getattr(embodied_cfg, "unnorm_key", "") or "")

    def _make_env(self, n: int):
        e = self.cfg.env
        if self.env is None or self.env.num_envs != n:
            if self.env is not None:
                self.env.close()
            self.env = make_environment(e.env_type, env_name=e.env_name, num_envs=n, max_steps=e.max_steps,
                                        num_steps_wait=e.num_steps_wait, model_family=e.model_family,
                                        device=str(self.device), **dict(getattr(e, "env_kwargs", None) or {}))
        return self.env

    def _frames(self, ob) -> torch.Tensor:
        """Camera frames of one environment: ``[H, W, 3]``, or ``[num_images, H, W, 3]`` (third-person view first,
        then the wrist camera) when the policy takes several images."""
        if self.num_images == 1:
            return torch.as_tensor(ob["image"])
        views = [ob["image"]] + [ob.get(k) for k in ("wrist_image", "wrist_image_2")[: self.num_images - 1]]
        if len(views) != self.num_images or any(v is None for v in views):
            raise ValueError(f"num_images_in_input={self.num_images}: the environment returned {len(views)} camera views")
        return torch.stack([torch.as_tensor(v) for v in views])

    def _full_model(self):
        m = self.engine.model
        if hasattr(m, "full"):
            raise ValueError("parallel action decoding runs on the whole model: set rollout.tensor_model_parallel_size=1")
        return m

    @staticmethod
    def _run(coro):
        loop = asyncio.new_event_loop()
        try:
            return loop.run_until_complete(coro)
        finally:
            loop.close()

    @torch.no_grad()
    def generate_sequences(self, prompts: Batch) -> Batch:
        t0 = time.time()
        meta = prompts.meta
        validate = bool(meta.get("validate", False))
        temperature = 0.0 if validate or not meta.get("do_sample", True) else float(self.cfg.temperature)
        task_ids = [int(x) for x in prompts["task_id"].reshape(-1).tolist()]
        trial_ids = [int(x) for x in prompts["trial_id"].reshape(-1).tolist()]
        B = len(task_ids)
        e = self.cfg.env
        A = self.chunk * self.atl
        L = (e.max_steps + self.chunk - 1) // self.chunk
        S = self.proc.image_size
        dev = self.device
        out_resp = torch.zeros(B, L, A, dtype=torch.int64, device=dev)
        out_logp = torch.zeros(B, L, A, dtype=torch.float32, device=dev)
        out_img = torch.zeros(B, L, self.num_images * S, S, 3, dtype=torch.uint8, device=dev)   # cameras stacked by height
        finish = torch.zeros(B, dtype=torch.int64)
        complete = torch.zeros(B, dtype=torch.bool)
        prompt_ids: List[Optional[List[int]]] = [None] * B
        n_env = min(e.num_envs, B)
        self.engine.wake_up()
        gen_tokens = 0
        for g0 in range(0, B, n_env):
            rows = list(range(g0, min(g0 + n_env, B)))
            env = self._make_env(len(rows))
            obs = self._run(env.reset([task_ids[i] for i in rows], [trial_ids[i] for i in rows]))
            for k, i in enumerate(rows):
                prompt_ids[i] = self.proc.prompt_ids(obs[k]["task_description"])
            live = [True] * len(rows)
            for l in range(L):
                act_rows = [k for k in range(len(rows)) if live[k]]
                if not act_rows:
                    break
                frames = torch.stack([self._frames(obs[k]) for k in act_rows]).to(dev)
                imgs = self.proc.resize(frames.contiguous())
                p_list = [prompt_ids[rows[k]] for k in act_rows]
                step_seed = (self.seed + 7919 * int(meta.get("global_steps", 0)) + 31 * l + g0) & 0x7FFFFFFF
                if self.parallel:
                    # OpenVLA-OFT: the whole chunk from one forward pass over [prompt][A zero vectors]
                    from ...models.embodied.vla import oft_parallel_decode
                    gen = torch.Generator(device=dev).manual_seed(step_seed)
                    tok, lp = oft_parallel_decode(self._full_model(), self.proc, p_list, imgs, A, temperature, gen)
                else:
                    mm = self.proc.mm_inputs(imgs, [len(p) for p in p_list], self.engine.model.embed_tokens.dtype)
                    sp = SamplingParams(n=1, temperature=temperature, max_new_tokens=A, ignore_eos=True, seed=step_seed)
                    outs = self.engine.generate(p_list, sp, mm_inputs=mm)
                    tok = torch.tensor([o.token_ids for o in outs], dtype=torch.int64, device=dev)
                    lp = torch.tensor([o.logprobs for o in outs], dtype=torch.float32, device=dev)
                gen_tokens += tok.numel()
                gi = torch.tensor([rows[k] for k in act_rows], device=dev)
                out_resp[gi, l], out_logp[gi, l], out_img[gi, l] = tok, lp, imgs
                acts = self.actions.decode(tok).reshape(len(act_rows), self.chunk, self.atl).cpu()
                if self.norm_stats is not None:
                    from ...models.embodied.action_heads import unnormalize_actions
                    acts = unnormalize_actions(acts, self.norm_stats)
                acts = acts.numpy()
                full = torch.zeros(len(rows), self.chunk, self.atl).numpy()
                full[act_rows] = acts
                obs = self._run(env.step(full))
                for k in act_rows:
                    i = rows[k]
                    finish[i] = int(obs[k]["step"])
                    if obs[k]["done"]:
                        live[k] = False
                        complete[i] = bool(obs[k]["success"])
        P = max(len(p) for p in prompt_ids)
        pad = self.model_config.pad_token_id or 0
        step_ids = torch.full((B, P), pad, dtype=torch.int64)
        step_am = torch.zeros(B, P, dtype=torch.int64)
        for i, p in enumerate(prompt_ids):
            step_ids[i, P - len(p):] = torch.tensor(p)
            step_am[i, P - len(p):] = 1
        out = Batch(dict(prompts.tensors), dict(prompts.non_tensors), dict(prompts.meta))
        out["responses"] = out_resp
        out["rollout_log_probs"] = out_logp.reshape(B, L * A)
        out["images"] = out_img
        out["step_input_ids"] = step_ids.to(dev)[:, None, :].expand(B, L, P).contiguous()
        out["step_attention_mask"] = step_am.to(dev)[:, None, :].expand(B, L, P).contiguous()
        out["finish_step"] = finish.to(dev)
        out["complete"] = complete.to(dev)
        mask = trajectory_response_mask(finish.to(dev), L, self.chunk, self.atl)
        out["response_mask"] = mask
        out["attention_mask"] = mask
        if self.video_embedder is not None:
            calls = (finish + self.chunk - 1) // self.chunk
            out["vjepa_embedding"] = self.video_embedder(out_img[:, :, :S], calls).to(dev)     # third-person camera
        out.non_tensors["task_file_name"] = [f"task_{t}" for t in task_ids]
        out.meta["timing_generate_s"] = time.time() - t0
        out.meta["total_output_tokens"] = int(mask.sum())
        out.meta["total_input_tokens"] = int(sum(len(p) for p in prompt_ids))
        out.meta["embodied"] = True
        out.meta["actions_per_call"] = self.chunk
        _ = gen_tokens
        return out
