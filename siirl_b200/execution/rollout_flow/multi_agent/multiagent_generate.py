"""Multi-agent rollout: several agent groups (each with its own policy worker) take turns on every sample.

Semantics of the reference (siirl/execution/rollout_flow/multi_agent/multiagent_generate.py:39-730): for each turn
the agents run in ``agent_group`` order; agent k's prompt is built by its ``pre_process`` hook from the running
conversation (default: previous agent's output appended to the prompt), its response goes through
``post_process`` and optionally an environment; with ``colocate`` the agents share the GPU, so each agent's engine is
woken up before and put to sleep after its turn; the loop ends when every sample is finished (environment done or
``max_turns``), which ranks agree on with one all-reduce.  The result carries every agent's tensors under
``agent_group_{k}_{key}`` and the last agent's under the plain keys, the layout MARFT's GAE reads
(core_algos.compute_marft_gae_advantage_return)."""
from __future__ import annotations

import uuid
from typing import Any, Callable, Dict, List, Optional

import torch
import torch.distributed as dist

from ....data_coordinator import Batch
from ....data_coordinator.dataloader.partitioned_dataset import left_pad


class MultiAgentLoop:
    def __init__(self, workers: Dict[int, Any], tokenizer, prompt_length: int, max_turns: int = 1,
                 pre_process: Optional[Dict[int, Callable]] = None, post_process: Optional[Dict[int, Callable]] = None,
                 env: Optional[Any] = None, colocate: bool = True, group=None):
        self.workers = dict(sorted(workers.items()))
        self.tokenizer = tokenizer
        self.prompt_length = prompt_length
        self.max_turns = max_turns
        self.pre = pre_process or {}
        self.post = post_process or {}
        self.env = env
        self.colocate = colocate
        self.group = group

    def _build_prompts(self, texts: List[List[int]], template: Batch) -> Batch:
        ids, masks, pos = [], [], []
        pad = getattr(self.tokenizer, "pad_token_id", 0) or 0
        for t in texts:
            a, b, c = left_pad(list(t)[-self.prompt_length:], self.prompt_length, pad, "left")
            ids.append(a), masks.append(b), pos.append(c)
        b = Batch({"input_ids": torch.stack(ids), "attention_mask": torch.stack(masks), "position_ids": torch.stack(pos)},
                  {"raw_prompt_ids": [list(t)[-self.prompt_length:] for t in texts]}, dict(template.meta))
        return b

    def _all_done(self, done: List[bool]) -> bool:
        flag = torch.tensor([0 if all(done) else 1])
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1:
            if dist.get_backend(self.group) == "nccl":
                flag = flag.cuda()
            dist.all_reduce(flag, group=self.group)
        return int(flag.item()) == 0

    def generate_sequence(self, batch: Batch) -> Batch:
        B = batch.batch_size
        convo: List[List[int]] = [list(x) for x in batch["raw_prompt_ids"]]
        done = [False] * B
        request_ids = [uuid.uuid4().hex for _ in range(B)]
        rows: List[Dict[str, Any]] = []          # one entry per (sample, turn): the per-agent outputs of that turn
        agents = list(self.workers)
        for turn in range(self.max_turns):
            turn_out: Dict[int, Batch] = {}
            for k in agents:
                w = self.workers[k]
                prompts = [self.pre[k](c, agent=k, turn=turn) if k in self.pre else c for c in convo]
                pb = self._build_prompts(prompts, batch)
                if self.colocate and getattr(w, "engine", None) is not None:
                    w.engine.wake_up()
                out = w.generate_sequences(pb)
                if self.colocate and getattr(w, "engine", None) is not None:
                    w.engine.sleep()
                turn_out[k] = out
                for i in range(B):
                    L = int(out["response_mask"][i].sum())
                    resp = out["responses"][i, :L].tolist()
                    if k in self.post:
                        resp = self.post[k](resp, agent=k, turn=turn)
                    convo[i] = prompts[i] + resp
            if self.env is not None:
                obs, env_done = self.env.step(convo)
                for i in range(B):
                    done[i] = done[i] or bool(env_done[i])
                    if obs is not None and obs[i]:
                        convo[i] = convo[i] + list(obs[i])
            rows.append(turn_out)
            if self._all_done(done) or turn == self.max_turns - 1:
                break
        return self._postprocess(batch, rows, request_ids)

    def _postprocess(self, batch: Batch, rows: List[Dict[int, Batch]], request_ids: List[str]) -> Batch:
        """Stack the turns of each sample as consecutive rows (row = sample * traj_len + turn)."""
        agents = list(self.workers)
        last = agents[-1]
        T = len(rows)
        B = batch.batch_size
        out_t: Dict[str, torch.Tensor] = {}
        for k in agents:
            prefix = "" if k == last else f"agent_group_{k}_"
            for key in ("prompts", "responses", "input_ids", "attention_mask", "position_ids", "response_mask"):
                stacked = torch.stack([rows[t][k][key] for t in range(T)], dim=1)      # [B, T, ...]
                out_t[prefix + key] = stacked.reshape(B * T, *stacked.shape[2:])
        non = {k: [v[i] for i in range(B) for _ in range(T)] for k, v in batch.non_tensors.items()}
        non["request_id"] = [request_ids[i] for i in range(B) for _ in range(T)]
        non["traj_len"] = [T] * (B * T)
        non["traj_step"] = [t for _ in range(B) for t in range(T)]
        out = Batch(out_t, non, dict(batch.meta))
        out.meta["agent_group_ids"] = agents[:-1]
        return out
