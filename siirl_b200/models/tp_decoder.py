"""Tensor-parallel view of a ``DecoderLM`` for the rollout engine.

Training keeps a full bf16 replica of the parameters on every rank (the optimizer state is what is sharded), so
the tensor-parallel layout of the rollout needs no communication: each rank slices its heads / FFN columns out of
its own replica.  The reference instead gathers FSDP or Megatron shards and pushes them parameter by parameter into
vLLM (siirl/engine/sharding_manager/fsdp_vllm.py:113-159, megatron_vllm.py).  Column-parallel weights (QKV, gate/up)
are gathered into contiguous per-rank copies by ``sync_weights`` (row ranges of the replica); row-parallel weights
(attention output, FFN down) are used in place as column-slice views, and their GEMM is fused with the all-reduce
(``TPContext.row_parallel_linear``).  Embedding, final norm and LM head stay replicated, so sampling needs no
cross-rank exchange and every rank of the group draws the same tokens from the same seed.
"""
from __future__ import annotations

import copy
from typing import List, Optional

import torch

from .. import ops
from ..ops.attention import SeqInfo, attention_packed
from ..parallel.tensor_parallel import TPContext
from .decoder import DecoderLM


class _TPLayer:
    __slots__ = ("qkv_w", "qkv_b", "gate_up_w", "o_w", "down_w")


class TPDecoder:
    def __init__(self, model: DecoderLM, tp: TPContext, presharded: bool = False):
        """``presharded``: ``model`` was cut into tensor-parallel slices for training already
        (``parallel.megatron_tp.shard_decoder`` with the same group); the engine then reads those parameters in place
        and ``sync_weights`` has nothing to copy."""
        cfg = getattr(model, "full_cfg", model.cfg)
        self.presharded = bool(presharded)
        w = tp.world
        if cfg.is_moe:
            raise NotImplementedError("tensor-parallel rollout of MoE layers: use expert parallelism instead")
        if cfg.num_heads % w or cfg.num_kv_heads % w or cfg.intermediate_size % (w * 8):
            raise ValueError(f"tensor_model_parallel_size={w} must divide heads ({cfg.num_heads}/{cfg.num_kv_heads}) "
                             f"and intermediate_size/8 ({cfg.intermediate_size})")
        self.full = model
        self.tp = tp
        self.cfg = copy.copy(cfg)
        self.cfg.num_heads = cfg.num_heads // w
        self.cfg.num_kv_heads = cfg.num_kv_heads // w
        self.full_cfg = cfg
        self.layers: List[_TPLayer] = []
        self.sync_weights()

    # engine-facing attributes of DecoderLM
    @property
    def embed_tokens(self):
        return self.full.embed_tokens

    @property
    def head_weight(self):
        return self.full.head_weight

    def rope_tables(self, device, min_len: int = 0):
        return self.full.rope_tables(device, min_len)

    @torch.no_grad()
    def sync_weights(self) -> None:
        """Refresh the per-rank copies of the column-parallel weights from the replica (after an optimizer step)."""
        if self.presharded:
            self.layers = []
            for layer in self.full.layers:
                t = _TPLayer()
                t.qkv_w = layer.qkv_proj_weight.detach()
                t.qkv_b = layer.qkv_proj_bias.detach() if layer.qkv_proj_bias is not None else None
                t.gate_up_w = layer.gate_up_proj_weight.detach()
                t.o_w = layer.o_proj_weight.detach()
                t.down_w = layer.down_proj_weight.detach()
                self.layers.append(t)
            return
        c, w, r = self.full_cfg, self.tp.world, self.tp.rank
        D = c.head_dim
        hq, hk, I = c.num_heads // w, c.num_kv_heads // w, c.intermediate_size // w
        q0, k0, v0 = 0, c.num_heads * D, (c.num_heads + c.num_kv_heads) * D
        rows = torch.cat([torch.arange(q0 + r * hq * D, q0 + (r + 1) * hq * D),
                          torch.arange(k0 + r * hk * D, k0 + (r + 1) * hk * D),
                          torch.arange(v0 + r * hk * D, v0 + (r + 1) * hk * D)]).to(self.full.embed_tokens.device)
        gu_rows = torch.cat([torch.arange(r * I, (r + 1) * I),
                             torch.arange(c.intermediate_size + r * I, c.intermediate_size + (r + 1) * I)]).to(rows.device)
        first = not self.layers
        if c.lora_rank > 0:
            # low-rank adapters are folded into the engine's slices: W + (alpha / r) B A, cut the same way (rows of
            # B for the column-parallel layers, columns of A for the row-parallel ones).  The trainer keeps base
            # weights and adapters apart; the engine decodes with one GEMM per projection.
            sc = c.lora_alpha / c.lora_rank
            o_cols = torch.arange(r * hq * D, (r + 1) * hq * D, device=rows.device)
            d_cols = torch.arange(r * I, (r + 1) * I, device=rows.device)

            def fold(layer, name, row_idx=None, col_idx=None):
                W = getattr(layer, f"{name}_weight").detach()
                if not hasattr(layer, f"{name}_lora_A") or not getattr(layer, "lora_enabled", True):
                    W = W.index_select(0, row_idx) if row_idx is not None else W
                    return (W.index_select(1, col_idx) if col_idx is not None else W).contiguous()
                A = getattr(layer, f"{name}_lora_A").detach().float()
                B = getattr(layer, f"{name}_lora_B").detach().float()
                if row_idx is not None:
                    W, B = W.index_select(0, row_idx), B.index_select(0, row_idx)
                if col_idx is not None:
                    W, A = W.index_select(1, col_idx), A.index_select(1, col_idx)
                return (W.float() + sc * (B @ A)).to(W.dtype)

            self.layers = []
            for layer in self.full.layers:
                t = _TPLayer()
                t.qkv_w = fold(layer, "qkv_proj", row_idx=rows)
                t.qkv_b = layer.qkv_proj_bias.detach().index_select(0, rows) if layer.qkv_proj_bias is not None else None
                t.gate_up_w = fold(layer, "gate_up_proj", row_idx=gu_rows)
                t.o_w = fold(layer, "o_proj", col_idx=o_cols)
                t.down_w = fold(layer, "down_proj", col_idx=d_cols)
                self.layers.append(t)
            return
        for li, layer in enumerate(self.full.layers):
            if first:
                t = _TPLayer()
                t.qkv_w = layer.qkv_proj_weight.detach().index_select(0, rows)
                t.qkv_b = layer.qkv_proj_bias.detach().index_select(0, rows) if layer.qkv_proj_bias is not None else None
                t.gate_up_w = layer.gate_up_proj_weight.detach().index_select(0, gu_rows)
                self.layers.append(t)
            else:
                t = self.layers[li]
                torch.index_select(layer.qkv_proj_weight.detach(), 0, rows, out=t.qkv_w)
                if t.qkv_b is not None:
                    torch.index_select(layer.qkv_proj_bias.detach(), 0, rows, out=t.qkv_b)
                torch.index_select(layer.gate_up_proj_weight.detach(), 0, gu_rows, out=t.gate_up_w)
            # row-parallel weights: column slices of the replica, always current
            t.o_w = layer.o_proj_weight.detach()[:, r * hq * D:(r + 1) * hq * D]
            t.down_w = layer.down_proj_weight.detach()[:, r * I:(r + 1) * I]

    def _qkv_pre_rope(self, layer, t: _TPLayer, x: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        qkv = ops.linear(x, t.qkv_w, t.qkv_b)
        if cfg.qk_norm:
            T = qkv.shape[0]
            nrot = cfg.num_heads + cfg.num_kv_heads
            qk = qkv[:, : nrot * cfg.head_dim].reshape(T, nrot, cfg.head_dim)
            qn, _ = ops.rmsnorm(qk[:, : cfg.num_heads].reshape(-1, cfg.head_dim), layer.q_norm, cfg.rms_norm_eps)
            kn, _ = ops.rmsnorm(qk[:, cfg.num_heads:].reshape(-1, cfg.head_dim), layer.k_norm, cfg.rms_norm_eps)
            qkv = torch.cat([qn.reshape(T, -1), kn.reshape(T, -1), qkv[:, nrot * cfg.head_dim:]], dim=-1)
        return qkv

    @torch.no_grad()
    def forward_cached(self, input_ids: torch.Tensor, positions: torch.Tensor, cache: torch.Tensor,
                       block_table: torch.Tensor, seq_ids: torch.Tensor, *, prefill_info: Optional[SeqInfo] = None,
                       seq_lens: Optional[torch.Tensor] = None, pixel_values=None, image_grid_thw=None,
                       rope_positions: Optional[torch.Tensor] = None, prefix_lens=None,
                       prefill_slots=None) -> torch.Tensor:
        """Same contract as ``DecoderLM.forward_cached``; ``cache`` holds this rank's KV heads only."""
        from ..ops import kv_cache as kvc
        cfg, tp = self.cfg, self.tp
        rp = positions if rope_positions is None else rope_positions
        pmax = int(cfg.max_position_embeddings if rp.is_cuda else rp.max().item() + 1)
        rope = self.full.rope_tables(input_ids.device, min(pmax, 32768))
        h = self.full.embed(input_ids, pixel_values, image_grid_thw)
        delta = None
        pos32 = positions.to(torch.int32).contiguous()
        if cfg.mrope_section is None and rp.dim() == 2:
            rp = rp[0]
        rp32 = rp.to(torch.int32).contiguous()
        for li, layer in enumerate(self.full.layers):
            t = self.layers[li]
            x, h = ops.rmsnorm(delta if delta is not None else h, layer.input_layernorm, cfg.rms_norm_eps,
                               residual=h if delta is not None else None)
            qkv = kvc.rope_kv_append(self._qkv_pre_rope(layer, t, x), rp32, rope[0], rope[1], cfg.mrope_section,
                                     seq_ids, pos32, block_table, cache[li], cfg.num_heads, cfg.num_kv_heads,
                                     cfg.head_dim)
            if prefill_info is not None and prefix_lens is not None and any(int(p) > 0 for p in prefix_lens):
                # chunked prefill / prefix-cache hit: the chunk attends to the tokens already in the cache as well
                a = kvc.prefill_attention_with_prefix(qkv, prefill_info.seqlens, prefix_lens, prefill_slots, cache[li],
                                                      block_table, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim)
            elif prefill_info is not None:
                a = attention_packed(qkv, prefill_info, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, causal=True)
            else:
                a = kvc.decode_attention(qkv, cache[li], seq_lens, block_table, cfg.num_heads, cfg.num_kv_heads,
                                         cfg.head_dim)
            attn_out = tp.row_parallel_linear(a, t.o_w)
            x, h = ops.rmsnorm(attn_out, layer.post_attention_layernorm, cfg.rms_norm_eps, residual=h)
            delta = tp.row_parallel_linear(ops.swiglu(ops.linear(x, t.gate_up_w)), t.down_w)
        out, _ = ops.rmsnorm(delta, self.full.norm, cfg.rms_norm_eps, residual=h)
        return out
