"""Paged KV cache ops: append rows of a packed qkv buffer to the cache, fork blocks, decode attention (what the
reference gets from vLLM's paged attention behind siirl/engine/rollout/vllm_rollout/vllm_rollout_spmd.py:261-416).

Cache layout (one tensor for all layers): ``[layers, num_blocks, 2, Hkv, 64, D]`` bf16; ``block_table`` is
``int32 [B, max_blocks]`` (-1 = unused).  The CPU path keeps the same layout and uses plain indexing."""
from __future__ import annotations

import ctypes
import os
import math
from typing import Optional

import torch

from . import lib as _lib

BLOCK = 64


def kv_append(qkv: torch.Tensor, seq_ids: torch.Tensor, positions: torch.Tensor, block_table: torch.Tensor,
              cache_layer: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int) -> None:
    """Write the k and v parts of every row of ``qkv`` ([T, (Hq+2Hkv)*D]) to ``cache_layer`` at
    ``(sequence seq_ids[t], position positions[t])``."""
    T = qkv.shape[0]
    if qkv.is_cuda:
        L = _lib.get_lib()
        _lib.check(L.sb_kv_append(_lib.ptr(qkv), qkv.stride(0), _lib.ptr(seq_ids), _lib.ptr(positions),
                                  _lib.ptr(block_table), block_table.shape[1], _lib.ptr(cache_layer), T, n_heads,
                                  n_kv_heads, head_dim, _lib.stream()), "sb_kv_append")
        return
    valid = (seq_ids >= 0) & (positions >= 0)
    qkv, seq_ids, positions = qkv[valid], seq_ids[valid], positions[valid]
    T = qkv.shape[0]
    blk = block_table[seq_ids.long(), (positions // BLOCK).long()].long()
    off = (positions % BLOCK).long()
    k = qkv[:, n_heads * head_dim:(n_heads + n_kv_heads) * head_dim].reshape(T, n_kv_heads, head_dim)
    v = qkv[:, (n_heads + n_kv_heads) * head_dim:].reshape(T, n_kv_heads, head_dim)
    cache_layer[blk, 0, :, off] = k
    cache_layer[blk, 1, :, off] = v


def rope_kv_append(qkv: torch.Tensor, rope_positions: torch.Tensor, cos_tab: torch.Tensor, sin_tab: torch.Tensor,
                   mrope_section, seq_ids: torch.Tensor, cache_positions: torch.Tensor, block_table: torch.Tensor,
                   cache_layer: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int) -> torch.Tensor:
    """Inference-only fusion of RoPE and cache append: rotates the q and k heads of ``qkv`` IN PLACE and writes the
    rotated k and the v heads to the cache (one kernel on CUDA).  Returns ``qkv``."""
    if qkv.is_cuda and head_dim % 16 == 0:
        L = _lib.get_lib()
        pos = rope_positions.to(torch.int32).contiguous()
        rows = 1 if pos.dim() == 1 else pos.shape[0]
        s0 = s1 = 0
        if rows == 3:
            s0, s1 = mrope_section[0], mrope_section[0] + mrope_section[1]
        _lib.check(L.sb_rope_kv_append(_lib.ptr(qkv), qkv.stride(0), _lib.ptr(pos), rows, s0, s1, _lib.ptr(cos_tab),
                                       _lib.ptr(sin_tab), _lib.ptr(seq_ids), _lib.ptr(cache_positions),
                                       _lib.ptr(block_table), block_table.shape[1], _lib.ptr(cache_layer),
                                       qkv.shape[0], n_heads, n_kv_heads, head_dim, _lib.stream()),
                   "sb_rope_kv_append")
        return qkv
    from . import dense
    qkv = dense.rope(qkv, n_heads + n_kv_heads, head_dim, rope_positions, cos_tab, sin_tab, mrope_section)
    kv_append(qkv, seq_ids, cache_positions, block_table, cache_layer, n_heads, n_kv_heads, head_dim)
    return qkv


def kv_copy_blocks(cache_layer: torch.Tensor, src: torch.Tensor, dst: torch.Tensor) -> None:
    if src.numel() == 0:
        return
    if cache_layer.is_cuda:
        L = _lib.get_lib()
        block_elems = cache_layer[0].numel()
        _lib.check(L.sb_kv_copy_blocks(_lib.ptr(cache_layer), _lib.ptr(src), _lib.ptr(dst), src.numel(),
                                       ctypes.c_longlong(block_elems), _lib.stream()), "sb_kv_copy_blocks")
        return
    cache_layer[dst.long()] = cache_layer[src.long()]


# "split": persistent warp-specialised kernel with split K/V (csrc/fmha_decode_split.cu); "simple": one CTA per
# (sequence, kv head) (csrc/fmha_decode.cu)
DECODE_KERNEL = os.environ.get("SIIRL_DECODE_KERNEL", "split")      # environment override for A/B runs
_split_ws: dict = {}


def set_decode_kernel(name: str) -> None:
    global DECODE_KERNEL
    assert name in ("simple", "split")
    DECODE_KERNEL = name


def _split_workspace(device, B: int, n_heads: int, max_blocks: int, head_dim: int):
    """Partial outputs and log-sum-exps of the chunks of long sequences; one buffer per shape, allocated on first
    use (before any CUDA-graph capture replays it)."""
    chunk = int(_lib.get_lib().sb_fmha_decode_chunk_tiles())
    chunks = (max_blocks + chunk - 1) // chunk
    key = (device, B, n_heads, chunks, head_dim)
    ws = _split_ws.get(key)
    if ws is None:
        ws = (torch.empty(B * n_heads * chunks * head_dim, dtype=torch.float32, device=device),
              torch.empty(B * n_heads * chunks, dtype=torch.float32, device=device))
        _split_ws[key] = ws
    return ws


def decode_attention(q_rows: torch.Tensor, cache_layer: torch.Tensor, seq_lens: torch.Tensor,
                     block_table: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
                     scale: Optional[float] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One query token per sequence against its cached context.  ``q_rows`` is ``[B, >= Hq*D]`` with the q heads in
    the first ``Hq*D`` columns (a packed qkv row works); ``seq_lens[b]`` counts the current token.  Returns
    ``[B, Hq*D]``."""
    B = q_rows.shape[0]
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    if out is None:
        out = torch.empty(B, n_heads * head_dim, dtype=q_rows.dtype, device=q_rows.device)
    if q_rows.is_cuda:
        L = _lib.get_lib()
        assert head_dim in (64, 128), "decode attention kernel supports head_dim 64 and 128"
        if DECODE_KERNEL == "split" and q_rows.stride(0) % head_dim == 0:
            ws_o, ws_lse = _split_workspace(q_rows.device, B, n_heads, block_table.shape[1], head_dim)
            _lib.check(L.sb_fmha_decode_split(_lib.ptr(q_rows), q_rows.stride(0), _lib.ptr(cache_layer),
                                              ctypes.c_longlong(cache_layer.shape[0]), _lib.ptr(seq_lens),
                                              _lib.ptr(block_table), block_table.shape[1], _lib.ptr(out),
                                              _lib.ptr(ws_o), _lib.ptr(ws_lse), B, n_heads, n_kv_heads, head_dim,
                                              ctypes.c_float(scale), _lib.ptr(_lib.status_word(q_rows.device)),
                                              _lib.stream()), "sb_fmha_decode_split")
            return out
        _lib.check(L.sb_fmha_decode(_lib.ptr(q_rows), q_rows.stride(0), _lib.ptr(cache_layer),
                                    ctypes.c_longlong(cache_layer.shape[0]), _lib.ptr(seq_lens), _lib.ptr(block_table),
                                    block_table.shape[1], _lib.ptr(out), B, n_heads, n_kv_heads, head_dim,
                                    ctypes.c_float(scale), _lib.ptr(_lib.status_word(q_rows.device)), _lib.stream()),
                   "sb_fmha_decode")
        return out
    rep = n_heads // n_kv_heads
    for b in range(B):
        n = int(seq_lens[b])
        nb = (n + BLOCK - 1) // BLOCK
        blks = block_table[b, :nb].long()
        k = cache_layer[blks, 0].permute(1, 0, 2, 3).reshape(n_kv_heads, nb * BLOCK, head_dim)[:, :n].float()
        v = cache_layer[blks, 1].permute(1, 0, 2, 3).reshape(n_kv_heads, nb * BLOCK, head_dim)[:, :n].float()
        q = q_rows[b, : n_heads * head_dim].reshape(n_heads, head_dim).float()
        k = k.repeat_interleave(rep, dim=0)
        v = v.repeat_interleave(rep, dim=0)
        s = torch.einsum("hd,hnd->hn", q, k) * scale
        p = torch.softmax(s, -1)
        out[b] = torch.einsum("hn,hnd->hd", p, v).reshape(-1).to(out.dtype)
    return out


def prefill_attention_with_prefix(qkv: torch.Tensor, chunk_lens, prefix_lens, slots, cache_layer: torch.Tensor,
                                  block_table: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int) -> torch.Tensor:
    """Causal attention of freshly projected chunk rows against (cached prefix + chunk) -- chunked prefill and prompts
    whose first blocks were found in the prefix cache.  ``qkv [sum(chunk_lens), (Hq+2Hkv)*D]`` holds the chunk rows
    (their K/V must already be in the cache, appended by ``rope_kv_append``); sequence ``i`` sits in cache slot
    ``slots[i]`` with ``prefix_lens[i]`` earlier tokens.  K/V of all ``prefix + chunk`` positions are read back from
    the paged cache into one packed buffer, the packed-attention kernel computes only the query tiles that contain
    chunk rows, and the chunk rows of the result are returned ``[sum(chunk_lens), Hq*D]``."""
    from .attention import SeqInfo, attention_packed
    dev = qkv.device
    qw, kw = n_heads * head_dim, n_kv_heads * head_dim
    totals = [int(p) + int(c) for p, c in zip(prefix_lens, chunk_lens)]
    full = torch.zeros(sum(totals), qw + 2 * kw, dtype=qkv.dtype, device=dev)
    row, crow, keep = 0, 0, []
    for p_, c_, t_, slot in zip(prefix_lens, chunk_lens, totals, slots):
        nb = (t_ + BLOCK - 1) // BLOCK
        blks = block_table[int(slot), :nb].long()
        kv = cache_layer.index_select(0, blks)                      # [nb, 2, Hkv, 64, D]
        k = kv[:, 0].permute(0, 2, 1, 3).reshape(nb * BLOCK, kw)[:t_]
        v = kv[:, 1].permute(0, 2, 1, 3).reshape(nb * BLOCK, kw)[:t_]
        full[row:row + t_, qw:qw + kw] = k
        full[row:row + t_, qw + kw:] = v
        full[row + int(p_):row + t_, :qw] = qkv[crow:crow + int(c_), :qw]
        keep.append(torch.arange(row + int(p_), row + t_, device=dev))
        row += t_
        crow += int(c_)
    out = attention_packed(full, SeqInfo(totals, device=dev), n_heads, n_kv_heads, head_dim, causal=True,
                           q_start=[int(p) for p in prefix_lens])
    return out.index_select(0, torch.cat(keep))
