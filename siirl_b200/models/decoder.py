"""Decoder-only transformer (Llama / Qwen2 / Qwen3 / Qwen3-MoE / Qwen2.5-VL language tower) on packed tokens.

One implementation serves training, log-prob computation and (through ``forward_cached``) the rollout engine.
Inputs are *packed*: ``input_ids [T]`` with sequence boundaries in a :class:`SeqInfo`, no padding anywhere; this
is the native layout of every kernel in ``siirl_b200.ops``.  The reference gets the same effect by un-padding
HF models around flash-attn varlen (siirl/engine/actor/dp_actor.py:87-263, siirl/models/transformers/qwen2.py).

Weights use fused projections (``qkv_proj``, ``gate_up_proj``); ``siirl_b200.models.hf_io`` converts to and from
the HF names (q_proj/k_proj/v_proj, gate_proj/up_proj) for safetensors checkpoints.
"""
from __future__ import annotations

import contextlib
import math

from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.utils.checkpoint as ckpt

from .. import ops
from ..ops.attention import SeqInfo, attention_packed
from ..ops.lm_head import lm_head_logits, lm_head_logprob_entropy
from .config import DecoderConfig


class _Init:
    """Seeded initialiser: CPU tensors draw from a CPU generator (bit-reproducible across machines), CUDA
    tensors from a generator on their own device (fast for multi-billion-parameter random-init models)."""

    def __init__(self, seed: int, device):
        self.device = torch.device(device)
        self.seed = seed
        self.gen = torch.Generator(device=self.device if self.device.type == "cuda" else "cpu").manual_seed(seed)


def _param(shape, dtype, device, std: float, gen: "_Init") -> nn.Parameter:
    dev = gen.device if gen.device.type == "cuda" else torch.device("cpu")
    t = torch.empty(*shape, dtype=torch.float32 if dev.type == "cpu" else dtype, device=dev)
    if std > 0:
        t.normal_(0.0, std, generator=gen.gen)
    elif std == 0:
        t.zero_()
    else:
        t.fill_(1.0)
    return nn.Parameter(t.to(device=device, dtype=dtype))


class DecoderLayer(nn.Module):
    def __init__(self, cfg: DecoderConfig, dtype, device, gen, layer_idx: int = 0):
        super().__init__()
        H, std = cfg.hidden_size, cfg.initializer_range
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.is_moe = cfg.layer_is_moe(layer_idx)
        self.input_layernorm = _param((H,), dtype, device, -1, gen)
        if cfg.is_mla:
            # multi-head latent attention: queries (optionally through a low-rank bottleneck), one projection to the
            # KV latent plus the shared rotary key, and the expansion of the latent to per-head keys and values
            nh, dq = cfg.num_heads, cfg.qk_nope_head_dim + cfg.qk_rope_head_dim
            if cfg.q_lora_rank > 0:
                self.q_a_proj_weight = _param((cfg.q_lora_rank, H), dtype, device, std, gen)
                self.q_a_layernorm = _param((cfg.q_lora_rank,), dtype, device, -1, gen)
                self.q_b_proj_weight = _param((nh * dq, cfg.q_lora_rank), dtype, device, std, gen)
            else:
                self.q_proj_weight = _param((nh * dq, H), dtype, device, std, gen)
            self.kv_a_proj_weight = _param((cfg.kv_lora_rank + cfg.qk_rope_head_dim, H), dtype, device, std, gen)
            self.kv_a_layernorm = _param((cfg.kv_lora_rank,), dtype, device, -1, gen)
            self.kv_b_proj_weight = _param((nh * (cfg.qk_nope_head_dim + cfg.v_head_dim), cfg.kv_lora_rank), dtype,
                                           device, std, gen)
            self.o_proj_weight = _param((H, nh * cfg.v_head_dim), dtype, device, std, gen)
            self.qkv_proj_bias = None
        else:
            self.qkv_proj_weight = _param((cfg.qkv_width, H), dtype, device, std, gen)
            self.qkv_proj_bias = _param((cfg.qkv_width,), dtype, device, 0, gen) if cfg.qkv_bias else None
            if cfg.qk_norm:
                self.q_norm = _param((cfg.head_dim,), dtype, device, -1, gen)
                self.k_norm = _param((cfg.head_dim,), dtype, device, -1, gen)
            self.o_proj_weight = _param((H, cfg.q_width), dtype, device, std, gen)
        self.post_attention_layernorm = _param((H,), dtype, device, -1, gen)
        if self.is_moe:
            E, I = cfg.num_experts, cfg.moe_intermediate_size
            El = E // max(cfg.ep_size, 1)
            self.router_weight = _param((E, H), dtype, device, std, gen)
            if cfg.topk_method == "noaux_tc":
                # selection bias of the auxiliary-loss-free load balancing (kept in fp32, not trained by the loss)
                self.router_bias = nn.Parameter(torch.zeros(E, dtype=torch.float32, device=device), requires_grad=False)
            if cfg.ep_size > 1:     # every rank draws its own experts: decorrelate the streams by expert range
                layer_salt = int(torch.randint(0, 2 ** 30, (1,), generator=gen.gen, device=gen.gen.device).item())
                gen = _Init(layer_salt + 7919 * (cfg.ep_rank + 1), device)
            self.experts_gate_up = _param((El, 2 * I, H), dtype, device, std, gen)
            self.experts_down = _param((El, H, I), dtype, device, std, gen)
            self.ep = None          # ExpertParallel context, attached by the worker
            self.ep_pad_tokens = 0  # static token bound all ranks pad to (0: token counts are equal already)
            if cfg.shared_expert_intermediate_size > 0:
                # shared expert (Qwen2-MoE / DeepSeek style): dense, replicated on every rank
                Is = cfg.shared_expert_intermediate_size
                self.shared_gate_up_weight = _param((2 * Is, H), dtype, device, std, gen)
                self.shared_down_weight = _param((H, Is), dtype, device, std, gen)
                if cfg.shared_expert_gate:
                    self.shared_expert_gate_weight = _param((1, H), dtype, device, std, gen)
        else:
            I = cfg.intermediate_size
            self.gate_up_proj_weight = _param((2 * I, H), dtype, device, std, gen)
            self.down_proj_weight = _param((H, I), dtype, device, std, gen)

        self.lora_enabled = True
        if cfg.lora_rank > 0:
            # low-rank adapters (reference: peft LoRA, siirl/engine/fsdp_workers.py:824-895): y += (x A^T) B^T * alpha/r;
            # A is small random, B zero, so training starts at the base model; with the adapters switched off
            # (``lora_enabled = False``) the same module is the frozen reference policy
            assert not cfg.is_moe and not cfg.is_mla and cfg.lora_rank % 8 == 0, "LoRA: dense layers, rank a multiple of 8"
            r = cfg.lora_rank
            for name, (n_out, n_in) in {"qkv_proj": (cfg.qkv_width, H), "o_proj": (H, cfg.q_width),
                                        "gate_up_proj": (2 * cfg.intermediate_size, H),
                                        "down_proj": (H, cfg.intermediate_size)}.items():
                if cfg.lora_targets is not None and name not in cfg.lora_targets:
                    continue
                setattr(self, f"{name}_lora_A", _param((r, n_in), dtype, device, 1.0 / r, gen))
                setattr(self, f"{name}_lora_B", _param((n_out, r), dtype, device, 0, gen))

    def _linear(self, x: torch.Tensor, name: str, bias=None) -> torch.Tensor:
        y = ops.linear(x, getattr(self, f"{name}_weight"), bias)
        if self.cfg.lora_rank > 0 and self.lora_enabled and hasattr(self, f"{name}_lora_A"):
            a = ops.linear(x, getattr(self, f"{name}_lora_A"))
            y = y + ops.linear(a, getattr(self, f"{name}_lora_B")) * (self.cfg.lora_alpha / self.cfg.lora_rank)
        return y

    # ---- pieces shared by the training and the cached (rollout) paths --------------------------
    def qkv(self, x: torch.Tensor, positions: torch.Tensor, rope) -> torch.Tensor:
        cfg = self.cfg
        qkv = self.qkv_pre_rope(x)
        cos, sin = rope
        if cfg.mrope_section is None and positions.dim() == 2:
            positions = positions[0]            # three equal rows from a multimodal processor of a 1-D rope family
        return ops.rope(qkv, cfg.num_heads + cfg.num_kv_heads, cfg.head_dim, positions, cos, sin, cfg.mrope_section)

    def mla_latent(self, x: torch.Tensor, positions: torch.Tensor, rope):
        """Multi-head latent attention before the key / value expansion: per-head queries ``[T, nh, nope + rope]``
        (rotary part rotated), the normalised latent ``[T, kv_lora_rank]`` and the rotated shared rotary key
        ``[T, rope]``.  The latent and the rotary key are all a cache has to keep per token."""
        cfg = self.cfg
        T = x.shape[0]
        nh, dn, dr = cfg.num_heads, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim
        if cfg.q_lora_rank > 0:
            qa, _ = ops.rmsnorm(ops.linear(x, self.q_a_proj_weight), self.q_a_layernorm, cfg.rms_norm_eps)
            q = ops.linear(qa, self.q_b_proj_weight)
        else:
            q = ops.linear(x, self.q_proj_weight)
        q = q.reshape(T, nh, dn + dr)
        ckv = ops.linear(x, self.kv_a_proj_weight)
        c, k_pe = ckv[:, : cfg.kv_lora_rank], ckv[:, cfg.kv_lora_rank:]
        cn, _ = ops.rmsnorm(c.contiguous(), self.kv_a_layernorm, cfg.rms_norm_eps)
        pe = torch.cat([q[:, :, dn:], k_pe.reshape(T, 1, dr)], 1)               # [T, nh + 1, dr]
        if cfg.rope_interleave:
            # checkpoints store rotary pairs interleaved (2i, 2i+1); the rotate-half kernel wants (i, i + dr/2)
            pe = pe.reshape(T, nh + 1, dr // 2, 2).transpose(-1, -2).reshape(T, nh + 1, dr)
        if positions.dim() == 2:
            positions = positions[0]
        cos, sin = rope
        pe = ops.rope(pe.reshape(T, (nh + 1) * dr).contiguous(), nh + 1, dr, positions, cos, sin, None)
        pe = pe.reshape(T, nh + 1, dr)
        return torch.cat([q[:, :, :dn], pe[:, :nh]], -1), cn, pe[:, nh]

    def mla_qkv(self, x: torch.Tensor, positions: torch.Tensor, rope):
        """Per-head queries / keys ``[T, nh, nope + rope]`` (rotary part rotated) and values ``[T, nh, v]`` of
        multi-head latent attention (reference path: HF DeepseekV3Attention as patched by
        siirl/models/transformers/kimi_vl.py:120-225)."""
        cfg = self.cfg
        T = x.shape[0]
        nh, dn, dr, dv = cfg.num_heads, cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim
        qf, cn, k_pe = self.mla_latent(x, positions, rope)
        kv = ops.linear(cn, self.kv_b_proj_weight).reshape(T, nh, dn + dv)
        kf = torch.cat([kv[:, :, :dn], k_pe[:, None, :].expand(T, nh, dr)], -1)
        return qf, kf, kv[:, :, dn:]

    def mla_scale(self) -> float:
        cfg = self.cfg
        scale = 1.0 / math.sqrt(cfg.qk_nope_head_dim + cfg.qk_rope_head_dim)
        rs = cfg.rope_scaling or {}
        if rs.get("rope_type", rs.get("type")) == "yarn" and rs.get("mscale_all_dim"):
            from ..ops.reference import yarn_mscale
            scale *= yarn_mscale(float(rs.get("factor", 1.0)), float(rs["mscale_all_dim"])) ** 2
        return scale

    def mla_attention(self, x: torch.Tensor, positions: torch.Tensor, info: SeqInfo, rope, causal=True) -> torch.Tensor:
        from ..ops.attention import attention_wide_heads
        cfg = self.cfg
        q, k, v = self.mla_qkv(x, positions, rope)
        scale = self.mla_scale()
        sp = getattr(self, "sp", None)
        if sp is not None and sp.sp > 1:
            # Ulysses (the switch the reference patches into Kimi-VL's attention,
            # siirl/models/transformers/kimi_vl.py:172-221): rows are this rank's slice of the packed stream; one
            # all-to-all hands every rank all rows of heads / sp heads, a second one brings the outputs back
            T, nh, n = x.shape[0], cfg.num_heads, sp.sp
            dq, dv = q.shape[-1], v.shape[-1]
            packed = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], -1)
            parts = [(0, nh * dq), (nh * dq, nh * dq), (2 * nh * dq, nh * dv)]
            full = sp.seq_to_heads(packed, parts)
            Tf, hl = full.shape[0], nh // n
            qf, kf, vf = full.split([hl * dq, hl * dq, hl * dv], -1)
            a = attention_wide_heads(qf.reshape(Tf, hl, dq), kf.reshape(Tf, hl, dq), vf.reshape(Tf, hl, dv), info,
                                     causal=causal, scale=scale).reshape(Tf, hl * dv)
            return sp.heads_to_seq(a, [(0, nh * dv)])
        return attention_wide_heads(q, k, v, info, causal=causal, scale=scale).reshape(x.shape[0], -1)

    def qkv_pre_rope(self, x: torch.Tensor) -> torch.Tensor:
        """QKV projection (+ per-head q/k RMSNorm for the Qwen3 family), before rotary embedding."""
        cfg = self.cfg
        qkv = self._linear(x, "qkv_proj", self.qkv_proj_bias)
        if cfg.qk_norm:
            T = qkv.shape[0]
            nrot = cfg.num_heads + cfg.num_kv_heads
            qk = qkv[:, : nrot * cfg.head_dim].reshape(T * nrot, cfg.head_dim)
            qk = qk.reshape(T, nrot, cfg.head_dim)
            qn, _ = ops.rmsnorm(qk[:, : cfg.num_heads].reshape(-1, cfg.head_dim), self.q_norm, cfg.rms_norm_eps)
            kn, _ = ops.rmsnorm(qk[:, cfg.num_heads:].reshape(-1, cfg.head_dim), self.k_norm, cfg.rms_norm_eps)
            qkv = torch.cat([qn.reshape(T, -1), kn.reshape(T, -1), qkv[:, nrot * cfg.head_dim:]], dim=-1)
        return qkv

    def mlp(self, x: torch.Tensor) -> torch.Tensor:
        if self.is_moe:
            from .moe import moe_forward, route_deepseek
            routed = None
            if self.cfg.scoring_func == "sigmoid" or self.cfg.n_group > 1:
                routed = route_deepseek(x, self.router_weight, getattr(self, "router_bias", None), self.cfg)
            y = moe_forward(x, self.router_weight, self.experts_gate_up, self.experts_down,
                            self.cfg.num_experts_per_tok, self.cfg.norm_topk_prob, ep=self.ep,
                            pad_tokens=self.ep_pad_tokens, routed=routed)
            if self.cfg.shared_expert_intermediate_size > 0:
                s = ops.linear(ops.swiglu(ops.linear(x, self.shared_gate_up_weight)), self.shared_down_weight)
                if self.cfg.shared_expert_gate:
                    g = torch.sigmoid(x.float() @ self.shared_expert_gate_weight.float().t())
                    s = (s.float() * g).to(s.dtype)
                y = y + s
            return y
        tp = getattr(self, "tp", None)
        if tp is not None:
            from ..parallel.megatron_tp import enter_parallel_block, leave_parallel_block
            y = self._linear(ops.swiglu(self._linear(enter_parallel_block(x, tp), "gate_up_proj")), "down_proj")
            return leave_parallel_block(y, tp)
        return self._linear(ops.swiglu(self._linear(x, "gate_up_proj")), "down_proj")

    def forward(self, h: torch.Tensor, delta: Optional[torch.Tensor], positions, info: SeqInfo, rope, causal=True):
        """``h`` is the residual stream, ``delta`` the previous sub-layer output not yet added to it."""
        cfg = self.cfg
        z3 = getattr(self, "zero3", None)
        if z3 is not None:      # parameter-sharded training state: assemble this layer's weights (prefetched)
            z3.fetch(self.zero3_index)
        tp = getattr(self, "tp", None)      # tensor-parallel training: ``cfg`` holds the local head / FFN counts
        x, h = ops.rmsnorm(delta if delta is not None else h, self.input_layernorm, cfg.rms_norm_eps,
                           residual=h if delta is not None else None)
        if tp is not None:
            from ..parallel.megatron_tp import enter_parallel_block
            x = enter_parallel_block(x, tp)
        if cfg.is_mla:
            attn_out = self._linear(self.mla_attention(x, positions, info, rope, causal), "o_proj")
            x, h = ops.rmsnorm(attn_out, self.post_attention_layernorm, cfg.rms_norm_eps, residual=h)
            return h, self.mlp(x)
        qkv = self.qkv(x, positions, rope)
        sp = getattr(self, "sp", None)
        if sp is not None and sp.sp > 1:
            # Ulysses: rows are this rank's slice of the packed stream; attention sees all rows of heads / sp heads
            D, n = cfg.head_dim, sp.sp
            parts = [(0, cfg.num_heads * D), (cfg.num_heads * D, cfg.num_kv_heads * D),
                     ((cfg.num_heads + cfg.num_kv_heads) * D, cfg.num_kv_heads * D)]
            a = attention_packed(sp.seq_to_heads(qkv, parts), info, cfg.num_heads // n, cfg.num_kv_heads // n, D,
                                 causal=causal)
            a = sp.heads_to_seq(a, [(0, cfg.num_heads * D)])
        elif getattr(self, "cp", None) is not None and self.cp.cp > 1:
            # context parallel: rows are this rank's chunk of every sequence (``info`` = chunk lengths); K/V of the
            # earlier chunks come from their owners
            from ..parallel.ring_attention import ring_attention
            a = ring_attention(qkv, self.cp, info, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim)
        else:
            a = attention_packed(qkv, info, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, causal=causal)
        attn_out = self._linear(a, "o_proj")
        if tp is not None:
            from ..parallel.megatron_tp import leave_parallel_block
            attn_out = leave_parallel_block(attn_out, tp)
        x, h = ops.rmsnorm(attn_out, self.post_attention_layernorm, cfg.rms_norm_eps, residual=h)
        return h, self.mlp(x)


class DecoderLM(nn.Module):
    def __init__(self, cfg: DecoderConfig, dtype=torch.bfloat16, device="cpu", seed: int = 0,
                 gradient_checkpointing: bool = False):
        super().__init__()
        self.cfg = cfg
        self.dtype = dtype
        gen = _Init(seed, device)
        std = cfg.initializer_range
        self.embed_tokens = _param((cfg.vocab_size, cfg.hidden_size), dtype, device, std, gen)
        self.layers = nn.ModuleList([DecoderLayer(cfg, dtype, device, gen, i) for i in range(cfg.num_layers)])
        self.norm = _param((cfg.hidden_size,), dtype, device, -1, gen)
        if cfg.value_head:
            self.value_head = _param((1, cfg.hidden_size), dtype, device, std, gen)
            self.lm_head = None
        elif cfg.tie_word_embeddings:
            self.lm_head = None
        else:
            self.lm_head = _param((cfg.vocab_size, cfg.hidden_size), dtype, device, std, gen)
        self.gradient_checkpointing = gradient_checkpointing
        self._rope = None
        self.vision = None
        if cfg.vision is not None:
            from .vision import VisionTower
            self.vision = VisionTower(cfg.vision, dtype, device, gen)
        elif cfg.moonvit is not None:
            from .moonvit import MoonViT
            self.vision = MoonViT(cfg.moonvit, cfg.hidden_size, dtype, device, gen)
        elif cfg.prismatic is not None:
            from .embodied.prismatic import PrismaticVision
            self.vision = PrismaticVision(cfg.prismatic, cfg.hidden_size, dtype, device, gen)
        elif cfg.vit is not None:
            from .internvl import InternVLVision
            self.vision = InternVLVision(cfg.vit, cfg.hidden_size, cfg.downsample_ratio, dtype, device, gen)

    # ---- helpers ------------------------------------------------------------------------------
    def rope_tables(self, device, min_len: int = 0):
        need = max(min_len, 1)
        if self._rope is None or self._rope[0].device != torch.device(device) or self._rope[0].shape[0] < need:
            n = max(need, min(self.cfg.max_position_embeddings, 8192))
            self._rope = ops.rope_tables(self.cfg.rope_dim, n, self.cfg.rope_theta, device=device,
                                         scaling=self.cfg.rope_scaling)
        return self._rope

    @property
    def head_weight(self) -> torch.Tensor:
        return self.lm_head if self.lm_head is not None else self.embed_tokens

    def embed(self, input_ids: torch.Tensor, pixel_values=None, image_grid_thw=None, image_mask=None,
              zero_mask=None, extra_embeds=None) -> torch.Tensor:
        """Token embeddings with vision features written over the image placeholders.  ``image_mask`` names the
        placeholder positions explicitly; the default (ids equal to ``image_token_id``) is only safe when generated
        tokens cannot collide with the placeholder id.  Rows of ``zero_mask`` enter the model as zero vectors (the
        action placeholders of OpenVLA-OFT's parallel decoding).  ``extra_embeds = (rows, values [len(rows), H])``
        writes given vectors over further rows (OpenVLA-OFT's proprioception pseudo-token)."""
        h = ops.embedding(input_ids, self.embed_tokens)
        if zero_mask is not None:
            h = h * (~zero_mask).to(h.dtype)[:, None]
        if self.vision is not None and pixel_values is not None:
            img = self.vision(pixel_values, image_grid_thw).to(h.dtype)
            mask = image_mask if image_mask is not None else input_ids == self.cfg.image_token_id
            idx = mask.nonzero(as_tuple=True)[0]
            h = h.index_copy(0, idx, img[: idx.numel()])
        if extra_embeds is not None:
            rows, values = extra_embeds
            h = h.index_copy(0, rows.to(h.device), values.to(h.device, h.dtype))
        return h

    # ---- training / scoring path ---------------------------------------------------------------
    def forward_hidden(self, input_ids: torch.Tensor, positions: torch.Tensor, info: SeqInfo, pixel_values=None,
                       image_grid_thw=None, image_mask=None, zero_mask=None, extra_embeds=None) -> torch.Tensor:
        """Final-norm hidden states ``[T, H]`` of a packed batch.  With sequence parallelism attached
        (``self.sp``), the packed stream is padded to a multiple of the group size and this rank computes rows
        ``[rank * T/sp, (rank + 1) * T/sp)``: the result holds those rows only (see ``sp_slice``)."""
        pmax = int(positions.max().item()) + 1 if positions.numel() else 1
        rope = self.rope_tables(input_ids.device, pmax)
        if getattr(self, "pp", None) is not None and self.pp.pp > 1:
            raise RuntimeError("pipeline-parallel models are driven through forward_hidden_pp")
        sp = getattr(self, "sp", None)
        cp = getattr(self, "cp", None)
        tp = getattr(self, "tp", None)
        split = (sp is not None and sp.sp > 1) or (cp is not None and cp.cp > 1) or \
            (tp is not None and tp.sequence_parallel)
        h_pre = None
        if split and (pixel_values is not None or zero_mask is not None or extra_embeds is not None):
            # rows are about to be divided over a group: image features (and other per-row overrides) are written
            # over the whole stream first, on every rank, and divided like the token rows (the reference's
            # vision-language Ulysses patch runs the tower on every rank too,
            # siirl/models/transformers/qwen2_vl.py ulysses_flash_attn_forward)
            h_pre = self.embed(input_ids, pixel_values, image_grid_thw, image_mask, zero_mask, extra_embeds)

        def pad_rows(t, n):
            return torch.cat([t, t.new_zeros(n, *t.shape[1:])]) if t is not None and n else t

        if sp is not None and sp.sp > 1:
            lo, hi, pad = self.sp_slice(input_ids.shape[0])
            if pad:
                input_ids = torch.cat([input_ids, input_ids.new_zeros(pad)])
                positions = torch.cat([positions, positions.new_zeros(*positions.shape[:-1], pad)], dim=-1)
                info = SeqInfo(list(info.seqlens) + [pad], device=input_ids.device)
                h_pre = pad_rows(h_pre, pad)
            input_ids, positions = input_ids[lo:hi], positions[..., lo:hi].contiguous()
            h_pre = h_pre[lo:hi] if h_pre is not None else None
        if cp is not None and cp.cp > 1:
            rows, _, info = self.cp_rows(info)
            keep = rows >= 0
            safe = rows.clamp(min=0)
            input_ids = torch.where(keep, input_ids[safe], torch.zeros_like(safe))
            positions = torch.where(keep, positions[..., safe], torch.zeros_like(positions[..., safe])).contiguous()
            if h_pre is not None:
                h_pre = h_pre.index_select(0, safe) * keep.to(h_pre.dtype)[:, None]
        sp_rows = None
        if tp is not None and tp.sequence_parallel:
            # Megatron sequence parallelism: between the tensor-parallel blocks every rank keeps 1 / tp of the token
            # rows.  The packed stream is padded (one dummy sequence) to a multiple of the group size.
            sp_rows = input_ids.shape[0]
            pad = (-sp_rows) % tp.size
            if pad:
                input_ids = torch.cat([input_ids, input_ids.new_zeros(pad)])
                positions = torch.cat([positions, positions.new_zeros(*positions.shape[:-1], pad)], dim=-1)
                info = SeqInfo(list(info.seqlens) + [pad], device=input_ids.device)
                h_pre = pad_rows(h_pre, pad)
        h = h_pre if h_pre is not None else self.embed(input_ids, pixel_values, image_grid_thw, image_mask, zero_mask,
                                                       extra_embeds)
        if sp_rows is not None:
            from ..parallel.megatron_tp import take_rows_for_sp
            h = take_rows_for_sp(h, tp)
        delta = None
        offload = getattr(self, "activation_offload", None)
        ctx = offload.region() if (offload is not None and torch.is_grad_enabled()) else contextlib.nullcontext()
        z3 = getattr(self.layers[0], "zero3", None) if len(self.layers) else None
        with ctx:   # tensors saved for backward move to pinned host memory when activation offload is attached
            for li, layer in enumerate(self.layers):
                if self.gradient_checkpointing and torch.is_grad_enabled():
                    if delta is not None:
                        # fold the pending sub-layer output into the residual stream first: the checkpoint then
                        # keeps ONE [T, H] tensor per layer instead of two
                        h, delta = h + delta, None
                    if z3 is not None and z3.trainable and h.requires_grad:
                        # the layer's input gradient is the last thing its backward produces: reduce-scatter then
                        h.register_hook(z3.make_reduce_hook(li))
                    h, delta = ckpt.checkpoint(layer, h, None, positions, info, rope, use_reentrant=False)
                else:
                    h, delta = layer(h, delta, positions, info, rope)
        out, _ = ops.rmsnorm(delta, self.norm, self.cfg.rms_norm_eps, residual=h)
        if sp_rows is not None:
            from ..parallel.megatron_tp import gather_rows_from_sp
            out = gather_rows_from_sp(out, tp)[:sp_rows]
        return out

    def token_logprobs(self, hidden: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0,
                       with_entropy: bool = True):
        """``log p(label)`` and entropy from final hidden states: the fused LM-head kernel, or its vocabulary-parallel
        form when this rank holds a slice of the head (tensor-parallel training with ``vocab_parallel``)."""
        vr = getattr(self, "vocab_range", None)
        if vr is not None:
            from ..parallel.megatron_tp import vocab_parallel_logprob_entropy
            lp, ent = vocab_parallel_logprob_entropy(hidden, self.lm_head, labels, vr[0], self.tp.group, temperature)
            return lp, (ent if with_entropy else None)
        return lm_head_logprob_entropy(hidden, self.head_weight, labels, temperature, with_entropy)

    def forward_hidden_pp(self, input_ids: torch.Tensor, positions: torch.Tensor, info: SeqInfo, chunk: int = 0):
        """Pipeline-parallel forward of this rank's stage (of its local model chunk ``chunk`` under the interleaved
        schedule).  Returns ``(hidden, None)`` for the last chunk of the model (final-norm hidden states) and
        ``(None, handle)`` elsewhere, where ``handle`` is a 0-d tensor whose backward receives the gradient of the
        activations sent downstream (``None`` without gradient history)."""
        from ..parallel import pipeline as P
        pc = self.pp
        pmax = int(positions.max().item()) + 1 if positions.numel() else 1
        rope = self.rope_tables(input_ids.device, pmax)
        T, H = input_ids.shape[0], self.cfg.hidden_size
        first, last = pc.chunk_is_first(chunk), pc.chunk_is_last(chunk)
        lo, hi = pc.chunk_layers(chunk)
        if first:
            h = self.embed(input_ids)
        else:
            h = P.recv_from_prev(pc, (T, H), self.embed_tokens.dtype, input_ids.device, torch.is_grad_enabled())
        delta = None
        for layer in self.layers[lo:hi]:
            if self.gradient_checkpointing and torch.is_grad_enabled():
                if delta is not None:
                    h, delta = h + delta, None
                h, delta = ckpt.checkpoint(layer, h, None, positions, info, rope, use_reentrant=False)
            else:
                h, delta = layer(h, delta, positions, info, rope)
        if last:
            if delta is None:       # a stage without layers
                return ops.rmsnorm(h, self.norm, self.cfg.rms_norm_eps)[0], None
            return ops.rmsnorm(delta, self.norm, self.cfg.rms_norm_eps, residual=h)[0], None
        return None, P.send_to_next(pc, h + delta if delta is not None else h)

    def attach_pipeline_parallel(self, pc) -> None:
        if self.cfg.tie_word_embeddings:
            raise ValueError("pipeline parallelism needs untied input / output embeddings")
        self.pp = pc

    def sp_slice(self, T: int) -> Tuple[int, int, int]:
        """(first row, end row, padding rows) of this rank's share of a packed stream of ``T`` tokens."""
        sp = getattr(self, "sp", None)
        n = sp.sp if sp is not None else 1
        Tl = (T + n - 1) // n
        r = sp.rank if sp is not None else 0
        return r * Tl, (r + 1) * Tl, Tl * n - T

    def cp_rows(self, info: SeqInfo):
        """Context parallelism: every sequence is padded to a multiple of the number of chunks and cut into equal
        chunks; this rank holds chunk ``rank`` of each (contiguous assignment) or chunks ``rank`` and
        ``2 n - 1 - rank`` of ``2 n`` (zig-zag).  Returns (index into the unpadded packed stream of each local row,
        -1 for padding; the same for use as a mask; the ``SeqInfo`` of the local lengths)."""
        from ..parallel.ring_attention import chunk_positions
        cp = self.cp
        n, r = cp.cp, cp.rank
        zz = bool(getattr(cp, "zigzag", False))
        parts = 2 * n if zz else n
        dev = self.embed_tokens.device
        idx, lens, start = [], [], 0
        for L in info.seqlens:
            local = (L + parts - 1) // parts * (parts // n)
            j = chunk_positions([local], n, r, zz)
            idx.append(torch.where(j < L, j + start, torch.full_like(j, -1)))
            lens.append(local)
            start += L
        rows = torch.cat(idx).to(dev) if idx else torch.zeros(0, dtype=torch.int64, device=dev)
        return rows, rows >= 0, SeqInfo(lens, device=dev)

    def local_row_index(self, info: SeqInfo, T: int) -> Optional[torch.Tensor]:
        """Index into the packed stream of every row this rank computes (sequence or context parallelism), -1 for
        padding rows; ``None`` when the rank computes the whole stream."""
        sp = getattr(self, "sp", None)
        cp = getattr(self, "cp", None)
        if sp is not None and sp.sp > 1:
            lo, hi, _ = self.sp_slice(T)
            j = torch.arange(lo, hi, device=self.embed_tokens.device)
            return torch.where(j < T, j, torch.full_like(j, -1))
        if cp is not None and cp.cp > 1:
            return self.cp_rows(info)[0]
        return None

    def attach_context_parallel(self, cp) -> None:
        self.cp = cp
        for layer in self.layers:
            layer.cp = cp

    def set_lora_enabled(self, on: bool) -> None:
        for layer in self.layers:
            layer.lora_enabled = on

    def attach_sequence_parallel(self, sp) -> None:
        self.sp = sp
        for layer in self.layers:
            layer.sp = sp

    def logprobs(self, input_ids, positions, info: SeqInfo, labels, temperature: float = 1.0,
                 with_entropy: bool = True, **mm) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """``log p(labels[t] | prefix)`` and entropy for every packed position (fp32 ``[T]``)."""
        hidden = self.forward_hidden(input_ids, positions, info, **mm)
        return self.token_logprobs(hidden, labels, temperature, with_entropy)

    def values(self, input_ids, positions, info: SeqInfo, **mm) -> torch.Tensor:
        """Scalar value per packed position (critic / reward model head)."""
        hidden = self.forward_hidden(input_ids, positions, info, **mm)
        return (hidden.float() @ self.value_head.float().t()).squeeze(-1)

    def logits(self, input_ids, positions, info: SeqInfo, **mm) -> torch.Tensor:
        return lm_head_logits(self.forward_hidden(input_ids, positions, info, **mm), self.head_weight)

    # ---- rollout path (paged KV cache, no autograd) ----------------------------------------------
    @torch.no_grad()
    def forward_cached(self, input_ids: torch.Tensor, positions: torch.Tensor, cache: torch.Tensor,
                       block_table: torch.Tensor, seq_ids: torch.Tensor, *, prefill_info: Optional[SeqInfo] = None,
                       seq_lens: Optional[torch.Tensor] = None, pixel_values=None, image_grid_thw=None,
                       rope_positions: Optional[torch.Tensor] = None, prefix_lens=None,
                       prefill_slots=None) -> torch.Tensor:
        """Runs the decoder on new tokens, appending their K/V to ``cache``.

        Prefill: ``prefill_info`` describes whole prompts packed in ``input_ids`` (attention over the new tokens,
        causal).  Decode: one token per running sequence, ``seq_lens`` = context lengths including that token
        (attention against the cache).  ``positions`` are cache positions; ``rope_positions`` (default: same)
        may differ for multimodal rope.  Returns final-norm hidden states of the new tokens."""
        from ..ops import kv_cache as kvc
        cfg = self.cfg
        rp = positions if rope_positions is None else rope_positions
        pmax = int(cfg.max_position_embeddings if rp.is_cuda else rp.max().item() + 1)
        rope = self.rope_tables(input_ids.device, min(pmax, 32768))
        h = self.embed(input_ids, pixel_values, image_grid_thw)
        delta = None
        pos32 = positions.to(torch.int32).contiguous()
        if cfg.mrope_section is None and rp.dim() == 2:
            rp = rp[0]
        rp32 = rp.to(torch.int32).contiguous()
        for li, layer in enumerate(self.layers):
            x, h = ops.rmsnorm(delta if delta is not None else h, layer.input_layernorm, cfg.rms_norm_eps,
                               residual=h if delta is not None else None)
            qkv = kvc.rope_kv_append(layer.qkv_pre_rope(x), rp32, rope[0], rope[1], cfg.mrope_section, seq_ids, pos32,
                                     block_table, cache[li], cfg.num_heads, cfg.num_kv_heads, cfg.head_dim)
            if prefill_info is not None and prefix_lens is not None and any(int(p) > 0 for p in prefix_lens):
                # chunked prefill / prefix-cache hit: the chunk attends to the tokens already in the cache as well
                a = kvc.prefill_attention_with_prefix(qkv, prefill_info.seqlens, prefix_lens, prefill_slots, cache[li],
                                                      block_table, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim)
            elif prefill_info is not None:
                a = attention_packed(qkv, prefill_info, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, causal=True)
            else:
                a = kvc.decode_attention(qkv, cache[li], seq_lens, block_table, cfg.num_heads, cfg.num_kv_heads,
                                         cfg.head_dim)
            attn_out = layer._linear(a, "o_proj")
            x, h = ops.rmsnorm(attn_out, layer.post_attention_layernorm, cfg.rms_norm_eps, residual=h)
            delta = layer.mlp(x)
        out, _ = ops.rmsnorm(delta, self.norm, cfg.rms_norm_eps, residual=h)
        return out

    def named_flat_order(self) -> List[Tuple[str, nn.Parameter]]:
        return list(self.named_parameters())


def build_model(cfg: DecoderConfig, dtype=torch.bfloat16, device="cpu", seed: int = 0,
                gradient_checkpointing: bool = False) -> DecoderLM:
    return DecoderLM(cfg, dtype=dtype, device=device, seed=seed, gradient_checkpointing=gradient_checkpointing)
