"""Native rollout engine: paged KV cache, continuous batching, prefix sharing, CUDA-graph decode.

This replaces the vLLM / SGLang engines of the reference (siirl/engine/rollout/vllm_rollout/vllm_rollout_spmd.py,
siirl/engine/rollout/sglang_rollout/*).  It runs in the same process and on the same weights as the trainer
(hybrid engine): ``sleep()`` frees the cache arena, ``wake_up()`` re-allocates it.

Scheduling model
* A request is one prompt with ``n`` samples.  The prompt is prefilled once; its full cache blocks are shared by
  the ``n`` sequences (reference counts) and only the last, partially filled block is copied per sample.
* Running sequences decode in lock-step.  Everything a decode step needs (context lengths, block tables, last
  tokens, finished flags, the sampler's counter) lives in device tensors, so a step is replayed from a CUDA
  graph; the host looks at the finished flags only every ``sync_interval`` steps, and at that point retires
  finished sequences, admits waiting requests into the freed slots and grows block tables.
* Slots of the running batch are fixed-size (``max_num_seqs`` rounded to the captured batch sizes); empty slots
  have context length 0 and are skipped by the kernels.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ...models.decoder import DecoderLM
from ...ops import kv_cache as kvc
from ...ops.attention import SeqInfo
from ...ops.lm_head import lm_head_logits
from ...ops.sampling import sample

BLOCK = kvc.BLOCK


_STREAM_KEY = 0x9E3779B97F4A7C15 & 0x7FFFFFFFFFFFFFFF      # Philox key of the CUDA-graph decode path


@dataclass
class SamplingParams:
    n: int = 1
    temperature: float = 1.0
    top_k: int = -1
    top_p: float = 1.0
    max_new_tokens: int = 16
    eos_token_id: Optional[int] = None
    ignore_eos: bool = False
    seed: int = 0


@dataclass
class RolloutOutput:
    prompt_index: int
    sample_index: int
    token_ids: List[int]
    logprobs: List[float]
    finish_reason: str  # "stop" (EOS) or "length"


@dataclass
class _Seq:
    prompt_index: int
    sample_index: int
    prompt_len: int
    max_new: int
    blocks: List[int] = field(default_factory=list)
    slot: int = -1
    generated: int = 0
    prefilled: int = 0          # prompt tokens whose K/V are in the cache (first sample of a group)


class BlockAllocator:
    """Reference-counted free list of cache blocks (host side) with a prefix cache on top.

    A full block of prompt tokens can be *registered* under the hash of the whole token prefix it ends.  When its last
    user releases it, a registered block is not freed but parked in an LRU list: a later prompt that starts with the
    same tokens takes it back (``lookup``) instead of prefilling them again; ``alloc`` evicts the least recently used
    parked block when the free list is empty.  Cached blocks are valid for one set of weights: the engine drops the
    allocator (and with it the cache) every time it goes to sleep."""

    def __init__(self, num_blocks: int):
        from collections import OrderedDict
        self.num_blocks = num_blocks
        self.free: List[int] = list(range(num_blocks - 1, -1, -1))
        self.ref = [0] * num_blocks
        self.by_hash: Dict[int, int] = {}          # prefix hash -> block
        self.hash_of: Dict[int, int] = {}          # block -> prefix hash
        self.parked = OrderedDict()                # zero-reference registered blocks, oldest first
        self.hits = self.misses = 0

    def alloc(self) -> int:
        if self.free:
            b = self.free.pop()
        elif self.parked:
            b, _ = self.parked.popitem(last=False)
            del self.by_hash[self.hash_of.pop(b)]
        else:
            raise MemoryError("KV cache exhausted")
        self.ref[b] = 1
        return b

    def share(self, b: int) -> int:
        self.ref[b] += 1
        return b

    def release(self, b: int) -> None:
        self.ref[b] -= 1
        if self.ref[b] == 0:
            if b in self.hash_of:
                self.parked[b] = None
            else:
                self.free.append(b)

    def register(self, key: int, b: int) -> None:
        if key not in self.by_hash and b not in self.hash_of:
            self.by_hash[key] = b
            self.hash_of[b] = key

    def lookup(self, key: int) -> Optional[int]:
        """Block cached under ``key`` with one more reference, or ``None``."""
        b = self.by_hash.get(key)
        if b is None:
            self.misses += 1
            return None
        self.hits += 1
        if self.ref[b] == 0:
            self.parked.pop(b, None)
        self.ref[b] += 1
        return b

    @property
    def num_free(self) -> int:
        return len(self.free) + len(self.parked)


def _prefix_hashes(tokens: Sequence[int], n_blocks: int) -> List[int]:
    """Hash of tokens[0 : (j + 1) * BLOCK] for j < n_blocks, chained so that each costs one block of hashing."""
    out, h = [], 0
    for j in range(n_blocks):
        h = hash((h, tuple(tokens[j * BLOCK:(j + 1) * BLOCK])))
        out.append(h)
    return out


class RolloutEngine:
    def __init__(self, model: DecoderLM, max_num_seqs: int = 256, max_model_len: int = 8192,
                 num_blocks: Optional[int] = None, gpu_memory_utilization: float = 0.5, sync_interval: int = 16,
                 use_cuda_graph: bool = True, max_num_batched_tokens: int = 8192, lockstep_group=None,
                 enable_chunked_prefill: bool = False, enable_prefix_caching: bool = True):
        """``lockstep_group``: ranks whose forward passes contain collectives over DIFFERENT requests (expert
        parallelism).  They then run the same sequence of prefill / decode calls: a rank without work joins with
        an empty prefill or an all-inactive decode step, and decode runs eagerly (the barriers of the expert
        exchange carry a host-side epoch)."""
        self.lockstep_group = lockstep_group
        if lockstep_group is not None:
            use_cuda_graph = False
            enable_chunked_prefill = enable_prefix_caching = False      # every rank must prefill the same shapes
        # Chunked prefill: a prompt longer than ``max_num_batched_tokens`` enters the cache in several engine
        # iterations (decode steps of the running sequences in between) instead of one oversized batch.  Prefix
        # caching: full prompt blocks are kept under the hash of their token prefix and reused by later prompts of
        # the same wake period (multi-turn conversations re-send their history; n-sample groups already share blocks).
        self.enable_chunked_prefill = bool(enable_chunked_prefill)
        self.enable_prefix_caching = bool(enable_prefix_caching)
        # Device memory the engine may use for KV blocks while it is awake (the trainer's fp32 gradient buffer, idle
        # and about to be zeroed between an optimizer step and the next backward): on a 180 GB part with the Adam
        # state resident this is what lets all sequences of a step decode in one wave.  Its contents are clobbered.
        self.borrowed: Optional[torch.Tensor] = None
        self.model = model
        self.cfg = model.cfg
        self.device = model.embed_tokens.device
        self.dtype = model.embed_tokens.dtype
        self.max_num_seqs = max_num_seqs
        self.max_model_len = max_model_len
        self.max_blocks_per_seq = (max_model_len + BLOCK - 1) // BLOCK
        self.sync_interval = max(1, sync_interval)
        self.use_cuda_graph = use_cuda_graph and self.device.type == "cuda"
        self.max_num_batched_tokens = max_num_batched_tokens
        self._requested_blocks = num_blocks
        self._mem_util = gpu_memory_utilization
        self.cache: Optional[List[torch.Tensor]] = None      # per layer [blocks, 2, Hkv, 64, D]
        self.alloc: Optional[BlockAllocator] = None
        self._graphs: Dict[int, object] = {}
        self._graph_launches: Dict[int, int] = {}
        self._out_buf = None
        self.stats = {"prefill_tokens": 0, "decode_steps": 0, "generated_tokens": 0}
        # SIIRL_ENGINE_TIMING=1: synchronise around every decode round and accumulate decode_s / capture_s in stats
        self._timing = os.environ.get("SIIRL_ENGINE_TIMING", "0") not in ("", "0") and self.device.type == "cuda"
        self.wake_up()

    # ---- memory hand-off with the trainer -------------------------------------------------------
    def _block_bytes(self) -> int:
        c = self.cfg
        return c.num_layers * 2 * c.num_kv_heads * BLOCK * c.head_dim * torch.finfo(self.dtype).bits // 8

    def wake_up(self) -> None:
        if self.cache is not None:
            return
        c = self.cfg
        nb = self._requested_blocks
        esize = torch.finfo(self.dtype).bits // 8
        lent = 0
        if self.borrowed is not None and self.borrowed.device == self.device:
            lent = self.borrowed.numel() * self.borrowed.element_size()
        if nb is None:
            if self.device.type == "cuda":
                torch.cuda.empty_cache()        # cached training blocks would hide free memory from the query
                free, _total = torch.cuda.mem_get_info(self.device)
                nb = max(16, (int(free * self._mem_util) + lent) // self._block_bytes())
            else:
                nb = max(16, self.max_num_seqs * self.max_blocks_per_seq)
            nb = min(nb, self.max_num_seqs * self.max_blocks_per_seq + 8)
        # one tensor per layer [nb, 2, Hkv, 64, D]: the first layers live in the borrowed buffer, the rest is new
        per_layer = nb * 2 * c.num_kv_heads * BLOCK * c.head_dim
        n_lent = min(c.num_layers, lent // (per_layer * esize)) if lent else 0
        shape = (nb, 2, c.num_kv_heads, BLOCK, c.head_dim)
        layers = []
        if n_lent:
            flat = self.borrowed.reshape(-1).view(torch.uint8)[: n_lent * per_layer * esize].view(self.dtype)
            flat.zero_()    # rows past a sequence's length are multiplied by zero weights: they must be finite
            layers += [flat[i * per_layer:(i + 1) * per_layer].view(shape) for i in range(n_lent)]
        if n_lent < c.num_layers:
            own = torch.zeros(c.num_layers - n_lent, *shape, dtype=self.dtype, device=self.device)
            layers += [own[i] for i in range(c.num_layers - n_lent)]
        self.cache = layers
        self.kv_layout = {"blocks": nb, "layers_in_borrowed_memory": n_lent}
        self.alloc = BlockAllocator(nb)
        self.num_slots = 0
        self._graphs.clear()
        self._out_buf = None

    def _ensure_slots(self, S: int) -> None:
        """(Re)allocate the per-slot device state for ``S`` concurrent sequences."""
        if self.num_slots == S:
            return
        dev = self.device
        self.num_slots = S
        self.block_table = torch.full((S, self.max_blocks_per_seq), -1, dtype=torch.int32, device=dev)
        self.ctx_len = torch.zeros(S, dtype=torch.int32, device=dev)       # tokens in the cache
        self.last_token = torch.zeros(S, dtype=torch.int64, device=dev)
        self.finished = torch.ones(S, dtype=torch.bool, device=dev)
        self.remaining = torch.zeros(S, dtype=torch.int32, device=dev)     # new tokens still allowed
        self.step_counter = torch.zeros(1, dtype=torch.int64, device=dev)
        self.slot_ids = torch.arange(S, dtype=torch.int32, device=dev)
        self.gen_index = torch.zeros(S, dtype=torch.int32, device=dev)
        self.hit_eos = torch.zeros(S, dtype=torch.bool, device=dev)
        self.rope_delta = torch.zeros(S, dtype=torch.int32, device=dev)    # cache position - rope position
        # inputs of one decode forward, rewritten by the prepare kernel every step
        self._step_bufs = {k: torch.zeros(S, dtype=torch.int32, device=dev)
                           for k in ("pos", "seq_ids", "seq_lens", "rope_pos")}
        self._graphs.clear()
        self._out_buf = None

    def sleep(self) -> None:
        """Free the cache arena (the trainer gets the memory back)."""
        self.cache = None
        self.alloc = None
        self._graphs.clear()
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    # ---- prefill --------------------------------------------------------------------------------
    @torch.no_grad()
    def _prefill(self, seqs: List[_Seq], chunks: List[List[int]], starts: Optional[List[int]] = None,
                 mm_inputs=None) -> torch.Tensor:
        """Prefill one packed batch: ``chunks[i]`` are the next tokens of the prompt of ``seqs[i]`` (sample 0 of its
        group), ``starts[i]`` how many of its tokens the cache holds already (a prefix-cache hit or earlier chunks;
        default 0 = whole prompts).  Returns the final hidden state of the last token of each chunk
        ``[len(seqs), H]``.  ``mm_inputs[i]`` (optional, whole prompts only) holds prompt i's ``pixel_values
        [patches, D]``, ``image_grid_thw [images, 3]`` and ``rope_positions [3, len]``."""
        lens = [len(p) for p in chunks]
        starts = list(starts) if starts is not None else [0] * len(chunks)
        mm = {}
        if mm_inputs is not None and any(m for m in mm_inputs):
            pv = [m["pixel_values"] for m in mm_inputs if m and m.get("pixel_values") is not None]
            if pv:
                mm["pixel_values"] = torch.cat([x.to(self.device) for x in pv], 0)
                mm["image_grid_thw"] = torch.cat([torch.as_tensor(m["image_grid_thw"]).reshape(-1, 3)
                                                  for m in mm_inputs if m and m.get("pixel_values") is not None], 0)
            if any(m and m.get("rope_positions") is not None for m in mm_inputs):
                rp = [torch.as_tensor(m["rope_positions"]) if m and m.get("rope_positions") is not None
                      else torch.arange(n).expand(3, n) for m, n in zip(mm_inputs, lens)]
                mm["rope_positions"] = torch.cat(rp, 1).to(self.device)
        info = SeqInfo(lens, device=self.device)
        ids = torch.tensor([t for p in chunks for t in p], dtype=torch.int64, device=self.device)
        seq_ids = torch.repeat_interleave(torch.tensor([s.slot for s in seqs], dtype=torch.int32),
                                          torch.tensor(lens)).to(self.device)
        positions = info.positions
        if any(starts):
            positions = torch.cat([torch.arange(st, st + n, dtype=torch.int32) for st, n in zip(starts, lens)]).to(
                self.device)
            mm["prefix_lens"] = starts
            mm["prefill_slots"] = [s.slot for s in seqs]
        hidden = self.model.forward_cached(ids, positions, self.cache, self.block_table, seq_ids,
                                           prefill_info=info, **mm)
        last = torch.tensor([c - 1 for c in info.cu_seqlens_cpu[1:]], dtype=torch.int64, device=self.device)
        self.stats["prefill_tokens"] += sum(lens)
        return hidden.index_select(0, last)

    # ---- decode ---------------------------------------------------------------------------------
    def _decode_step(self, sp: SamplingParams, tokens_out: torch.Tensor, logp_out: torch.Tensor) -> None:
        """One lock-step decode of all slots.  Pure device work (graph-capturable)."""
        S = self.num_slots
        if self.device.type == "cuda":
            return self._decode_step_native(sp, tokens_out, logp_out)
        active = ~self.finished
        pos = torch.where(active, self.ctx_len, torch.full_like(self.ctx_len, -1))
        seq_ids = torch.where(active, self.slot_ids, torch.full_like(self.slot_ids, -1))
        seq_lens = torch.where(active, self.ctx_len + 1, torch.zeros_like(self.ctx_len))
        hidden = self.model.forward_cached(self.last_token, pos.clamp(min=0), self.cache, self.block_table, seq_ids,
                                           seq_lens=seq_lens, rope_positions=(pos - self.rope_delta).clamp(min=0))
        logits = lm_head_logits(hidden, self.model.head_weight)
        tok, lp = sample(logits, sp.temperature, sp.top_k, sp.top_p, seed=sp.seed, step_dev=self.step_counter
                         if self.device.type == "cuda" else None, step=int(self.step_counter.item())
                         if self.device.type != "cuda" else 0)
        col = self.gen_index.clamp(max=tokens_out.shape[1] - 1).long()
        rows = torch.arange(S, device=self.device)
        pad = self.cfg.pad_token_id
        tokens_out[rows, col] = torch.where(active, tok, tokens_out[rows, col])
        logp_out[rows, col] = torch.where(active, lp, logp_out[rows, col])
        self.gen_index += active.to(torch.int32)
        self.ctx_len += active.to(torch.int32)
        self.remaining -= active.to(torch.int32)
        self.last_token.copy_(torch.where(active, tok, self.last_token))
        done = self.remaining <= 0
        if sp.eos_token_id is not None and not sp.ignore_eos:
            done = done | (tok == sp.eos_token_id)
            self.hit_eos |= active & (tok == sp.eos_token_id)
        self.finished |= done
        self.step_counter += 1
        _ = pad

    def _decode_step_native(self, sp: SamplingParams, tokens_out: torch.Tensor, logp_out: torch.Tensor) -> None:
        """The same step on CUDA: two bookkeeping kernels (``csrc/decode_state.cu``) around forward, LM head and
        sampler; no element-wise torch launches."""
        import ctypes

        from ...ops import lib as _lib
        L = _lib.get_lib()
        S = self.num_slots
        st = self._step_bufs
        _lib.check(L.sb_decode_prepare(_lib.ptr(self.finished), _lib.ptr(self.ctx_len), _lib.ptr(self.rope_delta),
                                       _lib.ptr(st["pos"]), _lib.ptr(st["seq_ids"]), _lib.ptr(st["seq_lens"]),
                                       _lib.ptr(st["rope_pos"]), S, _lib.stream()), "sb_decode_prepare")
        hidden = self.model.forward_cached(self.last_token, st["pos"], self.cache, self.block_table, st["seq_ids"],
                                           seq_lens=st["seq_lens"], rope_positions=st["rope_pos"])
        logits = lm_head_logits(hidden, self.model.head_weight)
        # the request's seed lives in the device-side step counter (see ``generate``), not in a launch argument, so
        # that one captured graph serves every seed
        tok, lp = sample(logits, sp.temperature, sp.top_k, sp.top_p, seed=_STREAM_KEY, step_dev=self.step_counter)
        eos = -1 if (sp.eos_token_id is None or sp.ignore_eos) else int(sp.eos_token_id)
        _lib.check(L.sb_decode_commit(_lib.ptr(tok), _lib.ptr(lp), _lib.ptr(self.finished), _lib.ptr(self.hit_eos),
                                      _lib.ptr(self.ctx_len), _lib.ptr(self.remaining), _lib.ptr(self.gen_index),
                                      _lib.ptr(self.last_token), _lib.ptr(tokens_out), _lib.ptr(logp_out),
                                      _lib.ptr(self.step_counter), S, tokens_out.shape[1], ctypes.c_longlong(eos),
                                      _lib.stream()), "sb_decode_commit")

    def _run_decode_steps(self, k: int, sp: SamplingParams, tokens_out, logp_out) -> None:
        if not self.use_cuda_graph:
            for _ in range(k):
                self._decode_step(sp, tokens_out, logp_out)
            return
        key = (k, sp.temperature, sp.top_k, sp.top_p, sp.eos_token_id, sp.ignore_eos)
        g = self._graphs.get(key)
        if g is None:
            # warm-up on a side stream (allocator and lazy initialisation), then capture k steps as one graph
            from ...ops import lib as _lib
            _lib.status_word(self.device)
            snapshot = [t.clone() for t in (self.ctx_len, self.last_token, self.finished, self.remaining,
                                            self.step_counter, self.gen_index, self.hit_eos, tokens_out, logp_out)]
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self._decode_step(sp, tokens_out, logp_out)
            torch.cuda.current_stream().wait_stream(s)
            for dst, src in zip((self.ctx_len, self.last_token, self.finished, self.remaining, self.step_counter,
                                 self.gen_index, self.hit_eos, tokens_out, logp_out), snapshot):
                dst.copy_(src)
            g = torch.cuda.CUDAGraph()
            before = _lib.launch_count()
            with torch.cuda.graph(g):
                for _ in range(k):
                    self._decode_step(sp, tokens_out, logp_out)
            self._graph_launches[key] = _lib.launch_count() - before
            _lib.add_launches(-self._graph_launches[key])  # capture itself runs nothing
            for dst, src in zip((self.ctx_len, self.last_token, self.finished, self.remaining, self.step_counter,
                                 self.gen_index, self.hit_eos, tokens_out, logp_out), snapshot):
                dst.copy_(src)
            self._graphs[key] = g
        g.replay()
        from ...ops import lib as _l
        _l.add_launches(self._graph_launches.get(key, 0))

    # ---- public API -------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], sp: SamplingParams,
                 mm_inputs: Optional[Sequence[Optional[dict]]] = None) -> List[RolloutOutput]:
        """Generate ``sp.n`` samples for every prompt (token id lists).  Returns outputs ordered by
        (prompt_index, sample_index).  ``mm_inputs[i]``: multimodal inputs of prompt i (``pixel_values``,
        ``image_grid_thw``, ``rope_positions [3, len]``, ``rope_delta`` = prompt length minus the next rope
        position, so that decode continues the multimodal rope numbering)."""
        assert self.cache is not None, "engine is asleep: call wake_up()"
        dev = self.device
        S = min(self.max_num_seqs, max(8, (len(prompts) * sp.n + 7) // 8 * 8))
        if self.lockstep_group is not None:
            S = self.max_num_seqs       # every rank of the group decodes the same number of rows
        self._ensure_slots(S)
        R = sp.max_new_tokens
        waiting: List[int] = list(range(len(prompts)))[::-1]
        results: Dict[tuple, RolloutOutput] = {}
        slots: List[Optional[_Seq]] = [None] * S
        if self._out_buf is None or self._out_buf[0].shape[1] != R:
            self._out_buf = (torch.zeros(S, R, dtype=torch.int64, device=dev),
                             torch.zeros(S, R, dtype=torch.float32, device=dev))
            self._graphs.clear()
        tokens_out, logp_out = self._out_buf
        tokens_out.zero_()
        logp_out.zero_()
        self.gen_index.zero_()
        self.hit_eos.zero_()
        if dev.type == "cuda":
            # random stream of this call: counter range [seed << 24, ...) of the fixed key (16 M steps per seed)
            self.step_counter.fill_((int(sp.seed) & 0x7FFFFFFF) << 24)
        self.finished.fill_(True)
        self.ctx_len.zero_()
        self.remaining.zero_()
        self.rope_delta.zero_()
        self.block_table.fill_(-1)

        def blocks_needed(plen: int) -> int:
            return (plen + R + BLOCK - 1) // BLOCK

        def retire(slot: int, fin_reason: str, n_gen: int) -> None:
            seq = slots[slot]
            toks = tokens_out[slot, :n_gen].tolist()
            lps = logp_out[slot, :n_gen].tolist()
            self.stats["d2h_bytes"] = self.stats.get("d2h_bytes", 0) + 12 * n_gen
            results[(seq.prompt_index, seq.sample_index)] = RolloutOutput(seq.prompt_index, seq.sample_index, toks,
                                                                         lps, fin_reason)
            for b in seq.blocks:
                self.alloc.release(b)
            slots[slot] = None
            self.stats["generated_tokens"] += n_gen

        def group_any(*flags: bool) -> List[bool]:
            if self.lockstep_group is None:
                return list(flags)
            import torch.distributed as dist
            t = torch.tensor([float(f) for f in flags], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.lockstep_group)
            return [bool(v) for v in t.tolist()]

        pending: List[List[_Seq]] = []      # admitted groups whose prompt is not completely in the cache yet
        chunked = self.enable_chunked_prefill and mm_inputs is None
        use_cache = self.enable_prefix_caching and mm_inputs is None
        while group_any(bool(waiting) or any(s is not None for s in slots))[0]:
            # ---- prefill work of this iteration: continue started prompts, then admit new ones (all n samples of a
            # prompt at once) while slots, blocks and the token budget last ----
            free_slots = [i for i, s in enumerate(slots) if s is None]
            budget = self.max_num_batched_tokens
            jobs: List[tuple] = []          # (group, first token, end token) of the prompt range to prefill now
            for group in pending:
                lead = group[0]
                take = min(budget, lead.prompt_len - lead.prefilled)
                if take > 0:
                    jobs.append((group, lead.prefilled, lead.prefilled + take))
                    budget -= take
            new_groups: List[List[_Seq]] = []
            while waiting and budget > 0:
                pi = waiting[-1]
                p = list(prompts[pi])
                if len(p) + R > self.max_model_len:
                    raise ValueError(f"prompt {pi}: {len(p)} + {R} tokens exceed max_model_len {self.max_model_len}")
                full = len(p) // BLOCK
                hit: List[int] = []
                if use_cache and full:
                    # leave at least one token to prefill: its hidden state samples the first response token
                    keys = _prefix_hashes(p, full if len(p) % BLOCK else full - 1)
                    for k in keys:
                        b = self.alloc.lookup(k)
                        if b is None:
                            break
                        hit.append(b)
                need = blocks_needed(len(p)) - len(hit) + (sp.n - 1) * (blocks_needed(len(p)) - full)
                todo = len(p) - len(hit) * BLOCK
                if len(free_slots) < sp.n or self.alloc.num_free < need or (
                        not chunked and jobs and todo > budget):
                    for b in hit:
                        self.alloc.release(b)
                    break
                waiting.pop()
                group = []
                for si in range(sp.n):
                    seq = _Seq(pi, si, len(p), R, slot=free_slots.pop(0))
                    slots[seq.slot] = seq
                    group.append(seq)
                first = group[0]
                first.blocks = hit + [self.alloc.alloc() for _ in range(blocks_needed(len(p)) - len(hit))]
                first.prefilled = len(hit) * BLOCK
                self.stats["prefix_cache_hit_tokens"] = self.stats.get("prefix_cache_hit_tokens", 0) + first.prefilled
                for other in group[1:]:
                    other.blocks = [self.alloc.share(b) for b in first.blocks[:full]]
                    for j in range(full, len(first.blocks)):
                        other.blocks.append(self.alloc.alloc())
                take = min(budget, todo) if chunked else todo
                jobs.append((group, first.prefilled, first.prefilled + take))
                budget -= take
                new_groups.append(group)
            pending += new_groups
            if waiting and not jobs and not any(s is not None for s in slots):
                raise MemoryError("a single request does not fit into the KV cache / slot budget")
            any_prefill, = group_any(bool(jobs))
            if any_prefill and not jobs:
                # another rank of the lock-step group prefills: join its collectives with one unrouted token
                one = SeqInfo([1], device=dev)
                self.model.forward_cached(torch.zeros(1, dtype=torch.int64, device=dev), one.positions, self.cache,
                                          self.block_table, torch.full((1,), -1, dtype=torch.int32, device=dev),
                                          prefill_info=one)
            if jobs:
                if new_groups:
                    bt = self.block_table.cpu()
                    for group in new_groups:
                        for seq in group:
                            bt[seq.slot, : len(seq.blocks)] = torch.tensor(seq.blocks, dtype=torch.int32)
                    self.block_table.copy_(bt)
                batch_mm = [mm_inputs[g[0].prompt_index] for g, _, _ in jobs] if mm_inputs is not None else None
                hidden = self._prefill([g[0] for g, _, _ in jobs],
                                       [list(prompts[g[0].prompt_index])[a:b] for g, a, b in jobs],
                                       [a for _, a, _ in jobs], batch_mm)
                done_rows, batch_seqs, forks = [], [], []
                for row, (group, _a, b) in enumerate(jobs):
                    lead = group[0]
                    lead.prefilled = b
                    if b < lead.prompt_len:
                        continue
                    done_rows.append(row)
                    batch_seqs.append(group)
                    plen = lead.prompt_len
                    full = plen // BLOCK
                    if plen % BLOCK:
                        forks += [(lead.blocks[full], other.blocks[full]) for other in group[1:]]
                    if use_cache:
                        for j, k in enumerate(_prefix_hashes(list(prompts[lead.prompt_index]), full)):
                            self.alloc.register(k, lead.blocks[j])
                pending = [g for g in pending if g[0].prefilled < g[0].prompt_len]
                if forks:
                    src = torch.tensor([a for a, _ in forks], dtype=torch.int32, device=dev)
                    dst = torch.tensor([b for _, b in forks], dtype=torch.int32, device=dev)
                    for li in range(self.cfg.num_layers):
                        kvc.kv_copy_blocks(self.cache[li], src, dst)
            if jobs and batch_seqs:
                # first token of every sample comes from the prompt's last hidden state
                rep_idx = torch.tensor([done_rows[i] for i, g in enumerate(batch_seqs) for _ in g], device=dev)
                logits = lm_head_logits(hidden.index_select(0, rep_idx), self.model.head_weight)
                tok, lp = sample(logits, sp.temperature, sp.top_k, sp.top_p, seed=sp.seed ^ 0x5bd1e995,
                                 step=int(self.step_counter.item()))
                self.step_counter += 1
                flat = [s for g in batch_seqs for s in g]
                sl = torch.tensor([s.slot for s in flat], dtype=torch.int64, device=dev)
                tokens_out[sl, 0] = tok
                logp_out[sl, 0] = lp
                self.gen_index[sl] = 1
                self.ctx_len[sl] = torch.tensor([s.prompt_len for s in flat], dtype=torch.int32, device=dev)
                self.remaining[sl] = R - 1
                if mm_inputs is not None:
                    self.rope_delta[sl] = torch.tensor([int((mm_inputs[s.prompt_index] or {}).get("rope_delta", 0))
                                                        for s in flat], dtype=torch.int32, device=dev)
                self.last_token[sl] = tok
                fin = torch.zeros(len(flat), dtype=torch.bool, device=dev) | (R <= 1)
                if sp.eos_token_id is not None and not sp.ignore_eos:
                    eos = tok == sp.eos_token_id
                    self.hit_eos[sl] = eos
                    fin = fin | eos
                else:
                    self.hit_eos[sl] = False
                self.finished[sl] = fin
            # ---- decode until the next host check ----
            if group_any(bool((~self.finished).any().item()))[0]:
                if self._timing:
                    torch.cuda.synchronize(dev)
                    t_dec = time.perf_counter()
                    n_graphs = len(self._graphs)
                self._run_decode_steps(self.sync_interval, sp, tokens_out, logp_out)
                if self._timing:
                    torch.cuda.synchronize(dev)
                    dt = time.perf_counter() - t_dec
                    key = "capture_s" if len(self._graphs) != n_graphs else "decode_s"
                    self.stats[key] = self.stats.get(key, 0.0) + dt
                self.stats["decode_steps"] += self.sync_interval
            # ---- retire finished sequences ----
            fin_cpu = self.finished.cpu().tolist()
            gen_cpu = self.gen_index.cpu().tolist()
            eos_cpu = self.hit_eos.cpu().tolist()
            self.stats["d2h_bytes"] = self.stats.get("d2h_bytes", 0) + 6 * S
            prefilling = {s.slot for g in pending for s in g}
            for slot, seq in enumerate(slots):
                if seq is not None and fin_cpu[slot] and slot not in prefilling:
                    retire(slot, "stop" if eos_cpu[slot] else "length", gen_cpu[slot])
                    self.ctx_len[slot] = 0
                    self.gen_index[slot] = 0
                    self.block_table[slot].fill_(-1)
        return [results[k] for k in sorted(results)]

    def cache_utilization(self) -> float:
        return 1.0 - self.alloc.num_free / self.alloc.num_blocks if self.alloc else 0.0

