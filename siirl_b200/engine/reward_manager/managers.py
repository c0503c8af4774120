"""Reward managers: turn a rolled-out batch into ``token_level_scores``.

Placement rule of the reference (siirl/engine/reward_manager/naive.py:25-115, dapo.py:25-141): the scalar score of
a response is written at its LAST valid response token, every other position is 0.  ``DAPORewardManager`` adds the
soft over-length penalty ``min(-(len - (max_resp_len - L_buf)) / L_buf * factor, 0)``; ``ParallelRewardManager``
scores in a process pool; ``EmbodiedRewardManager`` scores trajectories from environment outcomes.  If the batch
already carries ``rm_scores`` (model-based reward) it is returned unchanged.
"""
from __future__ import annotations

import concurrent.futures as cf
from collections import defaultdict
from typing import Any, Callable, Dict, Optional

import torch

from ...utils.reward_score import default_compute_score


def _valid_lengths(batch):
    prompts, responses, am = batch["prompts"], batch["responses"], batch["attention_mask"]
    P = prompts.shape[-1]
    return am[:, :P].sum(-1), am[:, P:].sum(-1)


class NaiveRewardManager:
    def __init__(self, tokenizer, num_examine: int = 0, compute_score: Optional[Callable] = None,
                 reward_fn_key: str = "data_source", **reward_kwargs):
        self.tokenizer = tokenizer
        self.num_examine = num_examine
        self.compute_score = compute_score or default_compute_score
        self.reward_fn_key = reward_fn_key
        self.reward_kwargs = reward_kwargs

    def _score_one(self, batch, i: int, plen: int, rlen: int):
        resp_ids = batch["responses"][i, :rlen].tolist()
        response_str = self.tokenizer.decode(resp_ids, skip_special_tokens=True)
        rm = batch["reward_model"][i] if "reward_model" in batch else {}
        gt = rm.get("ground_truth") if isinstance(rm, dict) else None
        ds = batch[self.reward_fn_key][i] if self.reward_fn_key in batch else "unknown"
        extra = dict(batch["extra_info"][i] or {}) if "extra_info" in batch else {}
        if ds == "synthetic/parity":
            extra["last_token_even"] = 1.0 if (resp_ids and resp_ids[-1] % 2 == 0) else 0.0
        return self.compute_score(data_source=ds, solution_str=response_str, ground_truth=gt, extra_info=extra,
                                  **self.reward_kwargs)

    def _post(self, score, rlen: int) -> float:
        return float(score)

    def __call__(self, batch, return_dict: bool = False):
        if "rm_scores" in batch:
            return {"reward_tensor": batch["rm_scores"]} if return_dict else batch["rm_scores"]
        responses = batch["responses"]
        reward = torch.zeros(responses.shape, dtype=torch.float32)
        extra_info = defaultdict(list)
        plens, rlens = _valid_lengths(batch)
        plens, rlens = plens.tolist(), rlens.tolist()
        scores = self._score_all(batch, plens, rlens)
        for i, score in enumerate(scores):
            if isinstance(score, dict):
                val = score["score"]
                for k, v in score.items():
                    extra_info[k].append(v)
            else:
                val = score
            val = self._post(val, int(rlens[i]))
            if rlens[i] > 0:
                reward[i, int(rlens[i]) - 1] = val
        reward = reward.to(responses.device)
        if return_dict:
            return {"reward_tensor": reward, "reward_extra_info": dict(extra_info)}
        return reward

    def _score_all(self, batch, plens, rlens):
        cpu = batch.to("cpu") if batch["responses"].is_cuda else batch
        return [self._score_one(cpu, i, int(plens[i]), int(rlens[i])) for i in range(cpu.batch_size)]


class DAPORewardManager(NaiveRewardManager):
    def __init__(self, tokenizer, num_examine: int = 0, compute_score=None, reward_fn_key: str = "data_source",
                 max_resp_len: Optional[int] = None, overlong_buffer_cfg=None, **reward_kwargs):
        super().__init__(tokenizer, num_examine, compute_score, reward_fn_key, **reward_kwargs)
        self.max_resp_len = max_resp_len
        self.overlong = overlong_buffer_cfg
        if self.overlong is not None and self.overlong.enable:
            assert max_resp_len is not None, "max_resp_len is required when the overlong buffer is enabled"

    def _post(self, score, rlen: int) -> float:
        score = float(score)
        ob = self.overlong
        if ob is not None and ob.enable:
            expected = self.max_resp_len - ob.len
            exceed = rlen - expected
            score += min(-exceed / ob.len * ob.penalty_factor, 0.0)
        return score


def _pool_score(args):
    fn, kwargs = args
    try:
        return fn(**kwargs)
    except Exception:  # noqa: BLE001  (a failing scorer gives zero reward, like the reference)
        return 0.0


class ParallelRewardManager(NaiveRewardManager):
    """Scores responses in a pool of worker processes (CPU-heavy scorers such as code/math verification)."""

    def __init__(self, tokenizer, num_examine: int = 0, compute_score=None, reward_fn_key: str = "data_source",
                 num_processes: int = 8, timeout_s: float = 300.0, **reward_kwargs):
        super().__init__(tokenizer, num_examine, compute_score, reward_fn_key, **reward_kwargs)
        self.num_processes = num_processes
        self.timeout_s = timeout_s

    def _score_all(self, batch, plens, rlens):
        cpu = batch.to("cpu") if batch["responses"].is_cuda else batch
        jobs = []
        for i in range(cpu.batch_size):
            resp_ids = cpu["responses"][i, : int(rlens[i])].tolist()
            rm = cpu["reward_model"][i] if "reward_model" in cpu else {}
            jobs.append((self.compute_score, dict(
                data_source=cpu[self.reward_fn_key][i] if self.reward_fn_key in cpu else "unknown",
                solution_str=self.tokenizer.decode(resp_ids, skip_special_tokens=True),
                ground_truth=rm.get("ground_truth") if isinstance(rm, dict) else None,
                extra_info=cpu["extra_info"][i] if "extra_info" in cpu else None, **self.reward_kwargs)))
        try:
            with cf.ProcessPoolExecutor(max_workers=self.num_processes) as ex:
                return list(ex.map(_pool_score, jobs, timeout=self.timeout_s))
        except Exception:  # noqa: BLE001
            return [_pool_score(j) for j in jobs]


class EmbodiedRewardManager:
    """Trajectory-level reward for embodied rollouts (reference: siirl/engine/reward_manager/embodied.py:25-207):
    successful episodes score 1, failed ones get a shaped score in [0, 0.6] from ``compute_score`` (distance of
    the episode embedding to clustered successful embeddings) when embeddings are present, else 0.  The score is
    written at the last executed action token of the flattened ``[traj_len * action_token_len]`` response."""

    def __init__(self, tokenizer=None, num_examine: int = 0, compute_score: Optional[Callable] = None,
                 reward_fn_key: str = "data_source", action_token_len: int = 7, **reward_kwargs):
        self.compute_score = compute_score
        self.action_token_len = action_token_len
        self.reward_kwargs = reward_kwargs

    def __call__(self, batch, return_dict: bool = False):
        responses = batch["responses"]
        B = responses.shape[0]
        R = responses.shape[1] * (responses.shape[2] if responses.dim() == 3 else 1)
        complete = batch["complete"].float().reshape(B)
        finish = batch["finish_step"].long().reshape(B)
        scores = complete.clone()
        if self.compute_score is not None and "vjepa_embedding" in batch:
            shaped = self.compute_score(batch_embeddings=batch["vjepa_embedding"], complete=complete,
                                        task_file_name=batch.get("task_file_name"), **self.reward_kwargs)
            scores = torch.as_tensor(shaped, dtype=torch.float32).reshape(B)
        reward = torch.zeros(B, R, dtype=torch.float32)
        last = (finish * self.action_token_len - 1).clamp(min=0, max=R - 1)
        reward[torch.arange(B), last.cpu()] = scores.cpu()
        reward = reward.to(responses.device)
        extra = {"acc": complete.cpu().tolist()}
        return {"reward_tensor": reward, "reward_extra_info": extra} if return_dict else reward


class BatchRewardManager(NaiveRewardManager):
    """``reward_model.reward_manager=batch``: the scoring function is called ONCE per batch with lists,
    ``compute_score(data_sources, solution_strs, ground_truths, extra_infos, **kwargs) -> list of float | dict``
    (the signature of the reference's custom-reward example, examples/custom_reward/rewardfunc_gsm8k.py:34-60).
    For functions that batch their own work: a judge model, a remote verifier, vectorised checks."""

    def _score_all(self, batch, plens, rlens):
        cpu = batch.to("cpu") if batch["responses"].is_cuda else batch
        n = cpu.batch_size
        texts, gts, sources, extras = [], [], [], []
        for i in range(n):
            texts.append(self.tokenizer.decode(cpu["responses"][i, :int(rlens[i])].tolist(), skip_special_tokens=True))
            rm = cpu["reward_model"][i] if "reward_model" in cpu else {}
            gts.append(rm.get("ground_truth") if isinstance(rm, dict) else None)
            sources.append(cpu[self.reward_fn_key][i] if self.reward_fn_key in cpu else "unknown")
            extras.append(dict(cpu["extra_info"][i] or {}) if "extra_info" in cpu else {})
        scores = self.compute_score(data_sources=sources, solution_strs=texts, ground_truths=gts, extra_infos=extras,
                                    **self.reward_kwargs)
        scores = list(scores)
        if len(scores) != n:
            raise ValueError(f"batch reward function returned {len(scores)} scores for {n} samples")
        return scores


REWARD_MANAGERS: Dict[str, Any] = {"naive": NaiveRewardManager, "dapo": DAPORewardManager,
                                   "parallel": ParallelRewardManager, "embodied": EmbodiedRewardManager,
                                   "batch": BatchRewardManager}
