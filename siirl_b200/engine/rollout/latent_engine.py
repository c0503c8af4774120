"""Rollout engine for multi-head latent attention (DeepSeek-V3 / Moonlight / Kimi-VL): a cache of the compressed
latents and decoding with the key / value expansion folded into the query and the output.

The reference serves these families through vLLM's MLA backend (siirl/engine/rollout/vllm_rollout/
vllm_rollout_spmd.py:261-416 with a DeepSeek-style ``hf_config``).  Per token and layer the cache keeps the normalised
latent (``kv_lora_rank`` values) and the rotated shared rotary key (``qk_rope_head_dim`` values): 576 values for
DeepSeek-V3 against ``num_heads * (192 + 128) = 40960`` for expanded keys and values.  A decoding step never expands
them.  With ``W_uk [nh, nope, R]`` and ``W_uv [nh, v, R]`` the two halves of ``kv_b_proj``:

    score[h, l] = (q_nope[h] W_uk[h]) . latent[l] + q_rope[h] . k_rope[l]
    out[h]      = (sum_l p[h, l] latent[l]) W_uv[h]^T

so attention runs as multi-query attention over one 576-wide "key" and one ``R``-wide "value" shared by all heads.
Prefill runs the packed training attention over the prompt (each distinct prompt once; its ``n`` samples copy the
latent rows).  The contractions here are batched matrix products of the tensor library, not hand-written kernels:
this engine replaces the cache-free recompute rollout (cost quadratic in the response length) for these families.

Slots are static: ``max_num_seqs`` sequences of up to ``max_model_len`` tokens, allocated on ``wake_up`` and freed on
``sleep``; longer batches run in waves.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ... import ops
from ...ops.attention import SeqInfo
from ...ops.sampling import sample
from .native_engine import RolloutOutput, SamplingParams


class LatentCacheEngine:
    def __init__(self, model, max_num_seqs: int = 64, max_model_len: int = 8192, max_num_batched_tokens: int = 16384,
                 lockstep_group=None, **_unused):
        """``lockstep_group``: ranks whose forward passes contain collectives over DIFFERENT requests (expert
        parallelism: every mixture-of-experts layer exchanges tokens with the group).  Those ranks must run the same
        number of forward passes, so generation proceeds in rounds: a rank that has a prefill pass or a decoding
        step left runs it, a rank that has finished runs a one-token pass, until no rank has work."""
        cfg = model.cfg
        assert cfg.is_mla, "the latent-cache engine serves multi-head latent attention models"
        self.model = model
        self.max_num_seqs = int(max_num_seqs)
        self.max_model_len = int(max_model_len)
        self.max_num_batched_tokens = max(1, int(max_num_batched_tokens or 16384))   # prompt tokens per prefill pass
        self.lockstep_group = lockstep_group
        bound = int(getattr(model.layers[-1], "ep_pad_tokens", 0) or 0) if len(model.layers) else 0
        if lockstep_group is not None and bound:
            self.max_num_batched_tokens = min(self.max_num_batched_tokens, bound)    # the exchange buffers' row bound
        self.device = model.embed_tokens.device
        self.width = cfg.kv_lora_rank + cfg.qk_rope_head_dim
        self.cache: Optional[torch.Tensor] = None
        self.stats = {"prefill_tokens": 0, "decode_steps": 0, "generated_tokens": 0, "d2h_bytes": 0}

    # ---- memory ------------------------------------------------------------------------------------------------------
    def cache_bytes(self) -> int:
        return self.model.cfg.num_layers * self.max_num_seqs * self.max_model_len * self.width * 2

    def wake_up(self) -> None:
        if self.cache is None:
            self.cache = torch.zeros(self.model.cfg.num_layers, self.max_num_seqs, self.max_model_len, self.width,
                                     dtype=self.model.embed_tokens.dtype, device=self.device)

    def sleep(self) -> None:
        self.cache = None
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    def cache_utilization(self) -> float:
        return float(getattr(self, "_last_util", 0.0))

    # ---- model pieces --------------------------------------------------------------------------------------------------
    def _rope(self, positions: torch.Tensor):
        # tables for the engine's whole context length: no device read-back of the largest position per pass
        return self.model.rope_tables(self.device, self.max_model_len)

    def _absorbed(self, layer):
        """``kv_b_proj`` as ``W_uk [nh, nope, R]`` and ``W_uv [nh, v, R]`` (views of the parameter)."""
        cfg = self.model.cfg
        w = layer.kv_b_proj_weight.detach().view(cfg.num_heads, cfg.qk_nope_head_dim + cfg.v_head_dim, cfg.kv_lora_rank)
        return w[:, : cfg.qk_nope_head_dim], w[:, cfg.qk_nope_head_dim:]

    @torch.no_grad()
    def _prefill(self, prompts: Sequence[Sequence[int]], slots: List[int], mms) -> torch.Tensor:
        """Packed forward of whole prompts; latents go to ``cache[:, slot, :len]``.  Returns the final-norm hidden
        state of every prompt's last token ``[len(prompts), H]``."""
        m, cfg, dev = self.model, self.model.cfg, self.device
        lens = [len(p) for p in prompts]
        ids = torch.tensor([t for p in prompts for t in p], dtype=torch.int64, device=dev)
        info = SeqInfo(lens, device=dev)
        positions = info.positions
        kw = {}
        if mms is not None and any(mm and mm.get("pixel_values") is not None for mm in mms):
            have = [mm for mm in mms if mm and mm.get("pixel_values") is not None]
            kw["pixel_values"] = torch.cat([mm["pixel_values"].to(dev) for mm in have])
            kw["image_grid_thw"] = torch.cat([torch.as_tensor(mm["image_grid_thw"]).reshape(-1, 3) for mm in have])
            kw["image_mask"] = ids == cfg.image_token_id
        rope = self._rope(positions)
        h = m.embed(ids, kw.get("pixel_values"), kw.get("image_grid_thw"), kw.get("image_mask"))
        delta = None
        rows = torch.cat([torch.arange(n) for n in lens]).to(dev)
        slot_of_row = torch.cat([torch.full((n,), s, dtype=torch.int64) for n, s in zip(lens, slots)]).to(dev)
        from ...ops.attention import attention_wide_heads
        nh, dn, dr, dv = cfg.num_heads, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        T = ids.shape[0]
        for li, layer in enumerate(m.layers):
            x, h = ops.rmsnorm(delta if delta is not None else h, layer.input_layernorm, cfg.rms_norm_eps,
                               residual=h if delta is not None else None)
            q, cn, k_pe = layer.mla_latent(x, positions, rope)
            self.cache[li, slot_of_row, rows] = torch.cat([cn, k_pe], -1)
            kv = ops.linear(cn, layer.kv_b_proj_weight).reshape(T, nh, dn + dv)
            k = torch.cat([kv[:, :, :dn], k_pe[:, None, :].expand(T, nh, dr)], -1)
            a = attention_wide_heads(q, k, kv[:, :, dn:], info, causal=True, scale=layer.mla_scale()).reshape(T, -1)
            x, h = ops.rmsnorm(layer._linear(a, "o_proj"), layer.post_attention_layernorm, cfg.rms_norm_eps, residual=h)
            delta = layer.mlp(x)
        out, _ = ops.rmsnorm(delta, m.norm, cfg.rms_norm_eps, residual=h)
        self.stats["prefill_tokens"] = self.stats.get("prefill_tokens", 0) + T
        last = torch.tensor(info.cu_seqlens_cpu[1:], device=dev) - 1
        return out.index_select(0, last)

    @torch.no_grad()
    def _decode(self, tokens: torch.Tensor, slots: torch.Tensor, lens: torch.Tensor, lmax: Optional[int] = None,
                dense_slots: bool = False) -> torch.Tensor:
        """One token per running sequence: ``tokens [B]`` sit at cache positions ``lens - 1``.  Returns hidden
        ``[B, H]``.  ``lmax``: the largest entry of ``lens`` when the caller knows it on the host; ``dense_slots``:
        ``slots`` is ``0 .. B-1`` (every sequence of the wave still runs), so the cache is read in place."""
        m, cfg = self.model, self.model.cfg
        B = tokens.shape[0]
        nh, dn, dr, dv, R = cfg.num_heads, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        positions = lens - 1
        rope = self._rope(positions)
        Lmax = int(lmax) if lmax is not None else int(lens.max().item())
        dead = torch.arange(Lmax, device=self.device)[None, :] >= lens[:, None]          # [B, Lmax]
        h = m.embed(tokens)
        delta = None
        for li, layer in enumerate(m.layers):
            x, h = ops.rmsnorm(delta if delta is not None else h, layer.input_layernorm, cfg.rms_norm_eps,
                               residual=h if delta is not None else None)
            q, cn, k_pe = layer.mla_latent(x, positions, rope)
            self.cache[li, slots, positions] = torch.cat([cn, k_pe], -1)
            lat = self.cache[li, :B, :Lmax] if dense_slots else \
                self.cache[li, :, :Lmax].index_select(0, slots)                           # [B, Lmax, R + dr]
            w_uk, w_uv = self._absorbed(layer)
            q_abs = torch.einsum("bhd,hdr->bhr", q[:, :, :dn], w_uk)                     # [B, nh, R]
            qq = torch.cat([q_abs, q[:, :, dn:]], -1)                                    # one 576-wide query per head
            sc = torch.bmm(qq, lat.transpose(1, 2)).float() * layer.mla_scale()          # [B, nh, Lmax]
            sc = sc.masked_fill(dead[:, None, :], float("-inf"))
            p = torch.softmax(sc, -1).to(lat.dtype)
            o_lat = torch.bmm(p, lat[:, :, :R])                                          # [B, nh, R]
            a = torch.einsum("bhr,hvr->bhv", o_lat, w_uv).reshape(B, nh * dv)
            x, h = ops.rmsnorm(layer._linear(a, "o_proj"), layer.post_attention_layernorm, cfg.rms_norm_eps, residual=h)
            delta = layer.mlp(x)
        out, _ = ops.rmsnorm(delta, m.norm, cfg.rms_norm_eps, residual=h)
        return out

    def _logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return ops.linear(hidden, self.model.head_weight).float()

    # ---- generation ----------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], sp: SamplingParams,
                 mm_inputs: Optional[Sequence[Optional[dict]]] = None) -> List[RolloutOutput]:
        asleep = self.cache is None
        if asleep:
            self.wake_up()
        out: List[RolloutOutput] = []
        self._drive(self._work(prompts, sp, mm_inputs, out))
        if asleep:
            self.sleep()
        out.sort(key=lambda o: (o.prompt_index, o.sample_index))
        return out

    def _drive(self, work) -> None:
        """Run the forward passes ``work`` asks for (it yields callables and receives their results).  With a
        lock-step group every rank runs one pass per round, an idle one-token pass once its own work is done."""
        result, finished = None, False
        while True:
            job = None
            if not finished:
                try:
                    job = work.send(result)
                except StopIteration:
                    finished = True
            if self.lockstep_group is not None:
                import torch.distributed as dist
                flag = torch.tensor([0.0 if finished else 1.0], device=self.device)
                dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=self.lockstep_group)
                if float(flag.item()) == 0.0:
                    return
            elif finished:
                return
            if job is not None:
                result = job()
            else:
                pad = self.model.cfg.pad_token_id or 0
                self._prefill([[pad]], [0], None)

    def _work(self, prompts, sp: SamplingParams, mm_inputs, out: List[RolloutOutput]):
        dev = self.device
        gen = torch.Generator(device="cpu").manual_seed(sp.seed) if dev.type == "cpu" else None
        n = max(1, sp.n)
        per_wave = max(1, self.max_num_seqs // n)                 # prompts per wave: all samples of a prompt together
        for w0 in range(0, len(prompts), per_wave):
            wave = [list(p)[: self.max_model_len - 1] for p in prompts[w0:w0 + per_wave]]
            P = len(wave)
            first_slots = [i * n for i in range(P)]
            mms = mm_inputs[w0:w0 + per_wave] if mm_inputs is not None else None
            parts, g0 = [], 0
            while g0 < P:                                          # prompts of one prefill pass: bounded token count
                g1, toks = g0, 0
                while g1 < P and (g1 == g0 or toks + len(wave[g1]) <= self.max_num_batched_tokens):
                    toks += len(wave[g1])
                    g1 += 1
                a, b = g0, g1
                parts.append((yield lambda: self._prefill(wave[a:b], first_slots[a:b],
                                                          mms[a:b] if mms is not None else None)))
                g0 = g1
            hidden = torch.cat(parts)
            plen = [len(p) for p in wave]
            if n > 1:                                              # the samples of a prompt share its latent rows
                src = torch.tensor(first_slots, device=dev)
                for s in range(1, n):
                    self.cache[:, src + s, :max(plen)] = self.cache[:, src, :max(plen)]
            B = P * n
            lens = [plen[b // n] for b in range(B)]                # tokens in the cache per sequence (slot = index)
            hidden = hidden.repeat_interleave(n, 0)
            new: List[List[int]] = [[] for _ in range(B)]
            lps: List[List[float]] = [[] for _ in range(B)]
            done: List[Optional[str]] = [None] * B
            live = list(range(B))
            self._last_util = float(sum(lens)) / (self.max_num_seqs * self.max_model_len)
            for step in range(sp.max_new_tokens):
                tok, lp = sample(self._logits(hidden), sp.temperature, sp.top_k, sp.top_p, seed=sp.seed,
                                 step=step * 4099 + w0, generator=gen)
                for key, inc in (("generated_tokens", len(live)), ("d2h_bytes", 12 * len(live))):
                    self.stats[key] = self.stats.get(key, 0) + inc
                keep = []
                for j, (b, t, l) in enumerate(zip(live, tok.tolist(), lp.tolist())):
                    new[b].append(int(t))
                    lps[b].append(float(l))
                    if not sp.ignore_eos and sp.eos_token_id is not None and int(t) == sp.eos_token_id:
                        done[b] = "stop"
                    elif len(new[b]) >= sp.max_new_tokens or lens[b] + 1 >= self.max_model_len:
                        done[b] = "length"
                    else:
                        keep.append(j)
                if not keep:
                    break
                live = [live[j] for j in keep]
                for b in live:
                    lens[b] += 1
                kidx = torch.tensor(keep, device=dev)
                step_tok, step_slots = tok.to(dev).index_select(0, kidx), torch.tensor(live, device=dev)
                host_lens = [lens[b] for b in live]
                step_lens, step_max, dense = torch.tensor(host_lens, device=dev), max(host_lens), len(live) == B
                hidden = yield lambda: self._decode(step_tok, step_slots, step_lens, step_max, dense)
                self.stats["decode_steps"] = self.stats.get("decode_steps", 0) + 1
            for b in range(B):
                out.append(RolloutOutput(w0 + b // n, b % n, new[b], lps[b], done[b] or "length"))
