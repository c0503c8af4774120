"""Multi-agent rollout: several agent groups (each with its own policy worker) take turns on every sample.

Semantics of the reference (siirl/execution/rollout_flow/multi_agent/multiagent_generate.py:39-730): inside one turn
the agents run in ``agent_group`` order; agent k's prompt is built by its ``pre_process`` hook from the running
conversation and the environment's last observation for that agent, its response is joined to the conversation by
``post_process``; after the last agent an environment (one per sample) judges the turn's actions and says whether the
sample is finished.  With ``colocate`` the agents share the GPU, so each agent's engine is woken up before and put to
sleep after its part of the turn.  The loop ends when every sample is finished or ``max_turns`` is reached, which
ranks agree on with one all-reduce.

The reference drives this with per-request asyncio tasks against a serving engine; here every agent step is ONE batched
engine call over the samples that are still running, which is what the native engine is fast at.

Result layout (the one MARFT's GAE reads, core_algos.compute_marft_gae_advantage_return): every agent's tensors under
``agent_group_{k}_{key}``, the last agent's under the plain keys; rows of one sample are consecutive, LATEST turn
first, and share ``request_id``; ``traj_len`` is the number of rows of the sample, ``traj_step`` the chronological
turn of a row.  ``env_score`` holds the environment's score of the row's turn."""
from __future__ import annotations

import asyncio
import inspect
import uuid
from typing import Any, Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ....data_coordinator import Batch
from ....data_coordinator.dataloader.partitioned_dataset import left_pad

_KEYS = ("prompts", "responses", "input_ids", "attention_mask", "position_ids", "response_mask")


def _resolve(value):
    """Environments may be written with ``async def step`` (the reference's are); run those to completion."""
    if inspect.iscoroutine(value):
        loop = asyncio.new_event_loop()
        try:
            return loop.run_until_complete(value)
        finally:
            loop.close()
    return value


class MultiAgentLoop:
    """``workers``: agent_group -> policy worker (``generate_sequences(Batch) -> Batch``).

    ``pre_process[k](prompt_ids, obs, agent=k, turn=t) -> prompt_ids`` and
    ``post_process[k](prompt_ids, response_ids, agent=k, turn=t) -> conversation_ids`` are optional; the defaults
    append the observation (tokenised) to the prompt and the response to the prompt.

    ``env_factory() -> env`` makes one environment per sample with
    ``step(actions: List[str], ground_truth) -> (next_obs: List[str] per agent, score, should_stop)``; ``env`` is the
    batched alternative ``step(conversations) -> (obs_ids per sample | None, done per sample)``.
    ``obs_with_env``: the next turn restarts from the sample's original prompt plus the observation instead of from the
    whole conversation so far."""

    def __init__(self, workers: Dict[int, Any], tokenizer, prompt_length: int, max_turns: int = 1,
                 pre_process: Optional[Dict[int, Callable]] = None, post_process: Optional[Dict[int, Callable]] = None,
                 env: Optional[Any] = None, env_factory: Optional[Callable[[], Any]] = None, colocate: bool = True,
                 group=None, use_all_traj: bool = True, obs_with_env: bool = False):
        self.workers = dict(sorted(workers.items()))
        self.tokenizer = tokenizer
        self.prompt_length = prompt_length
        self.max_turns = max(1, int(max_turns or 1))
        self.pre = pre_process or {}
        self.post = post_process or {}
        self.env = env
        self.env_factory = env_factory
        self.colocate = colocate
        self.group = group
        self.use_all_traj = use_all_traj
        self.obs_with_env = obs_with_env

    # ---- helpers -------------------------------------------------------------------------------
    def _build_prompts(self, texts: Sequence[Sequence[int]], template: Batch, non: Dict[str, List[Any]]) -> Batch:
        ids, masks, pos = [], [], []
        pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
        for t in texts:
            a, b, c = left_pad(list(t)[-self.prompt_length:], self.prompt_length, pad, "left")
            ids.append(a), masks.append(b), pos.append(c)
        non = dict(non)
        non["raw_prompt_ids"] = [list(t)[-self.prompt_length:] for t in texts]
        return Batch({"input_ids": torch.stack(ids), "attention_mask": torch.stack(masks),
                      "position_ids": torch.stack(pos)}, non, dict(template.meta))

    def _all_done(self, done: List[bool]) -> bool:
        flag = torch.tensor([0 if all(done) else 1])
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            if dist.get_backend(self.group) == "nccl":
                flag = flag.cuda()
            dist.all_reduce(flag, group=self.group)
        return int(flag.item()) == 0

    def _encode(self, text: str) -> List[int]:
        if not text:
            return []
        try:
            return list(self.tokenizer.encode(text, add_special_tokens=False))
        except TypeError:
            return list(self.tokenizer.encode(text))

    @staticmethod
    def _ground_truth(batch: Batch, i: int):
        rm = batch.non_tensors.get("reward_model")
        if rm is None:
            return None
        item = rm[i]
        return item.get("ground_truth") if isinstance(item, dict) else item

    # ---- the loop ------------------------------------------------------------------------------
    def generate_sequence(self, batch: Batch) -> Batch:
        B = batch.batch_size
        agents = list(self.workers)
        base: List[List[int]] = [list(x) for x in batch["raw_prompt_ids"]]
        convo: List[List[int]] = [list(x) for x in base]
        obs: List[List[Optional[str]]] = [[None] * len(agents) for _ in range(B)]
        done = [False] * B
        envs = [self.env_factory() for _ in range(B)] if self.env_factory is not None else None
        for e in envs or []:
            if hasattr(e, "reset"):
                _resolve(e.reset())
        request_ids = [uuid.uuid4().hex for _ in range(B)]
        # per sample: list over turns of {agent: row tensors}, and the env score of each turn
        turns_of: List[List[Dict[int, Dict[str, torch.Tensor]]]] = [[] for _ in range(B)]
        scores_of: List[List[float]] = [[] for _ in range(B)]
        total_tokens = 0
        for turn in range(self.max_turns):
            active = [i for i in range(B) if not done[i]]
            # every rank makes the same number of engine calls per turn, also with nothing left to do locally
            work = active or [0]
            actions: Dict[int, List[str]] = {i: [] for i in work}
            row_out: Dict[int, Dict[int, Dict[str, torch.Tensor]]] = {i: {} for i in work}
            if self.obs_with_env and turn > 0:
                for i in work:
                    convo[i] = list(base[i])
            for a_idx, k in enumerate(agents):
                w = self.workers[k]
                prompts = []
                for i in work:
                    o = obs[i][a_idx]
                    if k in self.pre:
                        p = self.pre[k](convo[i], o, agent=k, turn=turn)
                    else:
                        p = convo[i] + self._encode(o) if o else convo[i]
                    prompts.append(list(p))
                non = {key: [v[i] for i in work] for key, v in batch.non_tensors.items() if key != "raw_prompt_ids"}
                pb = self._build_prompts(prompts, batch, non)
                eng = getattr(w, "engine", None)
                if self.colocate and eng is not None:
                    eng.wake_up()
                out = w.generate_sequences(pb)
                if self.colocate and eng is not None:
                    eng.sleep()
                total_tokens += int(out.meta.get("total_output_tokens", 0))
                for j, i in enumerate(work):
                    L = int(out["response_mask"][j].sum())
                    resp = out["responses"][j, :L].tolist()
                    if k in self.post:
                        convo[i] = list(self.post[k](prompts[j], resp, agent=k, turn=turn))
                    else:
                        convo[i] = prompts[j] + resp
                    actions[i].append(self.tokenizer.decode(resp) if hasattr(self.tokenizer, "decode") else "")
                    row_out[i][k] = {key: out[key][j].cpu() for key in _KEYS}
            for i in active:
                score, stop = 0.0, False
                if envs is not None:
                    nxt, score, stop = _resolve(envs[i].step(actions[i], self._ground_truth(batch, i)))
                    if nxt is not None:
                        nxt = list(nxt) + [nxt[-1]] * (len(agents) - len(nxt)) if len(nxt) else [None] * len(agents)
                        obs[i] = [None if x is None else str(x) for x in nxt[:len(agents)]]
                turns_of[i].append(row_out[i])
                scores_of[i].append(float(score or 0.0))
                done[i] = done[i] or bool(stop)
            if self.env is not None:
                o_ids, env_done = self.env.step(convo)
                for i in active:
                    done[i] = done[i] or bool(env_done[i])
                    if o_ids is not None and o_ids[i]:
                        convo[i] = convo[i] + list(o_ids[i])
            if self._all_done(done) or turn == self.max_turns - 1:
                break
        out = self._postprocess(batch, turns_of, scores_of, request_ids)
        out.meta["total_output_tokens"] = total_tokens
        return out

    def _postprocess(self, batch: Batch, turns_of, scores_of, request_ids: List[str]) -> Batch:
        agents = list(self.workers)
        last = agents[-1]
        cols: Dict[str, List[torch.Tensor]] = {}
        src: List[int] = []
        traj_len: List[int] = []
        traj_step: List[int] = []
        env_score: List[float] = []
        for i, turns in enumerate(turns_of):
            order = list(range(len(turns) - 1, -1, -1))          # latest turn first
            if not self.use_all_traj:
                order = order[:1]
            for t in order:
                for k in agents:
                    prefix = "" if k == last else f"agent_group_{k}_"
                    for key in _KEYS:
                        cols.setdefault(prefix + key, []).append(turns[t][k][key])
                src.append(i)
                traj_len.append(len(order))
                traj_step.append(t)
                env_score.append(scores_of[i][t])
        tensors = {k: torch.stack(v) for k, v in cols.items()}
        non = {k: [v[i] for i in src] for k, v in batch.non_tensors.items()}
        non["request_id"] = [request_ids[i] for i in src]
        non["traj_len"] = traj_len
        non["traj_step"] = traj_step
        non["env_score"] = env_score
        out = Batch(tensors, non, dict(batch.meta))
        out.meta["agent_group_ids"] = agents[:-1]
        out.meta["multi_agent"] = True
        return out
