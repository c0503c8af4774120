"""Periodic validation: generate with the validation sampling parameters, score with the validation reward
manager, aggregate per data source (reference: siirl/dag_worker/validator.py:38-433).  Rows flagged
``padded_duplicate`` by the dataset are generated (so all ranks run the same number of batches) but excluded from
the scores."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..data_coordinator import Batch
from ..execution.scheduler.reward import compute_reward
from ..utils.logger.tracking import ValidationGenerationsLogger
from ..utils.metrics.metric_utils import process_validation_metrics


class Validator:
    def __init__(self, worker):
        self.w = worker
        self.enabled = worker.dataloader.val_dataset is not None and len(worker.dataloader.val_dataset) > 0 and \
            (worker.config.trainer.test_freq > 0 or worker.config.trainer.val_before_train)

    def validate(self) -> Optional[Dict[str, float]]:
        w = self.w
        if not self.enabled:
            return None
        dl = w.dataloader
        sources: List[str] = []
        inputs: List[str] = []
        scores: List[float] = []
        outputs: List[str] = []
        n_val = w.config.actor_rollout_ref.rollout.val_kwargs.n
        for _ in range(dl.num_val_batches):
            batch: Batch = dl.run(is_validation_step=True)
            if n_val > 1:
                batch = batch.repeat(n_val, interleave=True)
            batch.meta.update({"validate": True, "eos_token_id": getattr(w.tokenizer, "eos_token_id", None),
                               "pad_token_id": getattr(w.tokenizer, "pad_token_id", 0) or 0,
                               "global_steps": w.global_steps})
            if getattr(w, "_multi_agent", False):
                # joint loop of all agents; each sample is judged on its final turn (rows are latest turn first)
                out = w.multi_agent_loop.generate_sequence(batch.to("cpu"))
                first, seen = [], set()
                for i, rid in enumerate(out.non_tensors["request_id"]):
                    if rid not in seen:
                        seen.add(rid)
                        first.append(i)
                out = out.select_idxs(first).to(w.device)
            else:
                out = w._arr(None).generate_sequences(batch.to(w.device))
            reward, _extra = compute_reward(out, w.val_reward_fn)
            seq = reward.sum(-1).cpu().tolist()
            dup = out["padded_duplicate"] if "padded_duplicate" in out else [False] * out.batch_size
            if out["responses"].dim() == 3:
                # embodied episodes (reference validator.py, embodied variant): score = task success / shaped
                # reward, the logged "text" is the task and the episode summary
                for i in range(out.batch_size):
                    if dup[i]:
                        continue
                    sources.append(str(out["data_source"][i]) if "data_source" in out else "embodied")
                    inputs.append(str(out.non_tensors.get("task_file_name", ["task"] * out.batch_size)[i]))
                    outputs.append(f"finish_step={int(out['finish_step'][i])} complete={bool(out['complete'][i])}")
                    scores.append(float(out["complete"][i]))
                continue
            P = out["prompts"].shape[1]
            for i in range(out.batch_size):
                if dup[i]:
                    continue
                sources.append(str(out["data_source"][i]) if "data_source" in out else "unknown")
                pm = out["attention_mask"][i, :P].bool()
                inputs.append(w.tokenizer.decode(out["prompts"][i][pm].tolist()))
                rl = int(out["response_mask"][i].sum())
                outputs.append(w.tokenizer.decode(out["responses"][i, :rl].tolist()))
                scores.append(float(seq[i]))
        self._dump_rank_generations(sources, inputs, outputs, scores)
        if w._dist and w.world_size > 1:
            gathered = [None] * w.world_size
            dist.all_gather_object(gathered, (sources, inputs, scores, outputs))
            sources = [x for g in gathered for x in g[0]]
            inputs = [x for g in gathered for x in g[1]]
            scores = [x for g in gathered for x in g[2]]
            outputs = [x for g in gathered for x in g[3]]
        if not scores:
            return {}
        per = process_validation_metrics(sources, inputs, {"reward": scores})
        metrics: Dict[str, float] = {}
        for ds, var2 in per.items():
            for var, d in var2.items():
                for k, v in d.items():
                    core = k.startswith("mean@") or k.startswith("best@")
                    metrics[f"{'val-core' if core else 'val-aux'}/{ds}/{var}/{k}"] = v
        metrics["val-core/all/reward/mean"] = float(torch.tensor(scores).mean())
        t = w.config.trainer
        if w._rank == 0 and t.log_val_generations > 0 and t.validation_data_dir:
            ValidationGenerationsLogger(t.validation_data_dir).log(
                list(zip(inputs, outputs, scores))[: t.log_val_generations], w.global_steps)
        return metrics

    def _dump_rank_generations(self, sources, inputs, outputs, scores) -> None:
        """``trainer.rollout_data_dir``: every rank writes the validation generations it produced to
        ``step_<N>_rank_<r>.json`` (reference: siirl/dag_worker/dag_utils.py:637-683)."""
        import json
        import os
        w = self.w
        out_dir = getattr(w.config.trainer, "rollout_data_dir", None)
        if not out_dir:
            return
        try:
            os.makedirs(out_dir, exist_ok=True)
            rows = [{"rank": w._rank, "global_step": w.global_steps, "data_source": s, "input": i, "output": o,
                     "score": float(c)} for s, i, o, c in zip(sources, inputs, outputs, scores)]
            with open(os.path.join(out_dir, f"step_{w.global_steps}_rank_{w._rank}.json"), "w", encoding="utf-8") as f:
                json.dump(rows, f, ensure_ascii=False, indent=4)
        except OSError as e:
            print(f"[siirl_b200] rank {w._rank}: could not write validation generations to {out_dir}: {e}")
