"""Cache-free rollout: every decoding step runs the model's packed training forward over all live sequences.

The reference keeps a plain ``model.generate`` rollout beside the vLLM / SGLang engines
(siirl/engine/rollout/hf_rollout.py:36-170, ``rollout.name=hf``).  This is its counterpart here, with the interface of
:class:`RolloutEngine` (``generate / wake_up / sleep``): no paged cache, no CUDA graphs, cost quadratic in the response
length.  It serves (i) ``rollout.name=hf`` and (ii) model families whose attention has no paged-cache kernel yet
(multi-head latent attention), and it is the independent statement the paged engine is tested against.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ...ops.attention import SeqInfo
from ...ops.sampling import sample
from .native_engine import RolloutOutput, SamplingParams


class RecomputeEngine:
    def __init__(self, model, max_num_seqs: int = 64, max_model_len: int = 8192, **_unused):
        self.model = model
        self.max_num_seqs = max_num_seqs
        self.max_model_len = max_model_len
        self.device = model.embed_tokens.device
        self.cache = True                      # "awake" marker: there is no cache to allocate or free
        self.stats = {"prefill_tokens": 0, "decode_steps": 0, "generated_tokens": 0}

    def wake_up(self) -> None:
        self.cache = True

    def sleep(self) -> None:
        self.cache = None

    def cache_utilization(self) -> float:
        return 0.0

    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], sp: SamplingParams,
                 mm_inputs: Optional[Sequence[Optional[dict]]] = None) -> List[RolloutOutput]:
        dev = self.device
        seqs = []                                # one entry per (prompt, sample)
        for i, p in enumerate(prompts):
            for s in range(sp.n):
                seqs.append({"pi": i, "si": s, "ids": list(p), "new": [], "lp": [], "done": None})
        gen = torch.Generator(device="cpu").manual_seed(sp.seed) if dev.type == "cpu" else None
        out: List[RolloutOutput] = []
        for step in range(sp.max_new_tokens):
            live = [q for q in seqs if q["done"] is None]
            if not live:
                break
            for g0 in range(0, len(live), self.max_num_seqs):
                grp = live[g0:g0 + self.max_num_seqs]
                lens = [len(q["ids"]) + len(q["new"]) for q in grp]
                ids = torch.tensor([t for q in grp for t in q["ids"] + q["new"]], dtype=torch.int64, device=dev)
                info = SeqInfo(lens, device=dev)
                kw = {}
                positions = info.positions
                if mm_inputs is not None and any(mm_inputs[q["pi"]] for q in grp):
                    mms = [mm_inputs[q["pi"]] or {} for q in grp]
                    pv = [m["pixel_values"].to(dev) for m in mms if m.get("pixel_values") is not None]
                    if pv:
                        kw["pixel_values"] = torch.cat(pv)
                        kw["image_grid_thw"] = torch.cat([torch.as_tensor(m["image_grid_thw"]).reshape(-1, 3)
                                                          for m in mms if m.get("pixel_values") is not None])
                        # placeholders of the prompt only: a sampled token may collide with the placeholder id
                        mask = torch.zeros(ids.shape[0], dtype=torch.bool, device=dev)
                        at = 0
                        for q, n in zip(grp, lens):
                            pl = len(q["ids"])
                            mask[at:at + pl] = ids[at:at + pl] == self.model.cfg.image_token_id
                            at += n
                        kw["image_mask"] = mask
                    if any(m.get("rope_positions") is not None for m in mms):
                        rows = []
                        for q, m, n in zip(grp, mms, lens):
                            pl = len(q["ids"])
                            if m.get("rope_positions") is not None:
                                rp = torch.as_tensor(m["rope_positions"])
                                nxt = pl - int(m.get("rope_delta", 0))
                                tail = (torch.arange(n - pl) + nxt).expand(3, n - pl)
                                rows.append(torch.cat([rp, tail], 1))
                            else:
                                rows.append(torch.arange(n).expand(3, n))
                        positions = torch.cat(rows, 1).to(dev)
                hidden = self.model.forward_hidden(ids, positions, info, **kw)
                last = torch.tensor(info.cu_seqlens_cpu[1:], device=dev) - 1
                logits = hidden.index_select(0, last).float() @ self.model.head_weight.float().t()
                tok, lp = sample(logits, sp.temperature, sp.top_k, sp.top_p, seed=sp.seed, step=step * 4099 + g0,
                                 generator=gen)
                self.stats["decode_steps"] += 1
                self.stats["generated_tokens"] += len(grp)
                self.stats["d2h_bytes"] = self.stats.get("d2h_bytes", 0) + 12 * len(grp)
                for q, t, l in zip(grp, tok.tolist(), lp.tolist()):
                    q["new"].append(int(t))
                    q["lp"].append(float(l))
                    if not sp.ignore_eos and sp.eos_token_id is not None and int(t) == sp.eos_token_id:
                        q["done"] = "stop"
                    elif len(q["new"]) >= sp.max_new_tokens or len(q["ids"]) + len(q["new"]) >= self.max_model_len:
                        q["done"] = "length"
        for q in seqs:
            out.append(RolloutOutput(q["pi"], q["si"], q["new"], q["lp"], q["done"] or "length"))
        out.sort(key=lambda o: (o.prompt_index, o.sample_index))
        return out
