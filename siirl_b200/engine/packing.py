"""Padded ``[B, P+R]`` batches <-> packed token streams.

DAG nodes exchange the reference's padded layout (prompts left-padded to P, responses right-padded to R; Appendix
of siirl/engine/rollout/vllm_rollout/vllm_rollout_spmd.py:389-416), while every model kernel works on packed
tokens.  ``pack_batch`` builds the packed view once per micro-batch: token ids, positions, sequence boundaries,
shifted labels, and the indices that map "log-prob of response token k of row i" back into ``[B, R]``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..ops.attention import SeqInfo


@dataclass
class PackedBatch:
    input_ids: torch.Tensor        # [T]
    positions: torch.Tensor        # [T] (or [3, T] for mrope)
    info: SeqInfo
    sel: torch.Tensor              # [N] packed indices whose next-token distribution is needed
    labels: torch.Tensor           # [N] the token each selected position must predict
    out_rows: torch.Tensor         # [N] row in [B, R]
    out_cols: torch.Tensor         # [N] column in [B, R]
    batch_size: int
    response_length: int

    def scatter(self, values: torch.Tensor, fill: float = 0.0) -> torch.Tensor:
        """Place per-selected-token values into a dense ``[B, R]`` tensor (differentiable)."""
        out = torch.full((self.batch_size, self.response_length), fill, dtype=values.dtype, device=values.device)
        return out.index_put((self.out_rows, self.out_cols), values)


def pack_batch(input_ids: torch.Tensor, attention_mask: torch.Tensor, response_length: int,
               response_mask: Optional[torch.Tensor] = None, device=None) -> PackedBatch:
    """``input_ids/attention_mask`` are ``[B, P+R]``.  Selected positions are those that predict a valid response
    token: packed index of (last prompt token + k) for k in [0, r_i)."""
    B, S = input_ids.shape
    R = response_length
    P = S - R
    am = attention_mask.bool()
    lens = am.sum(-1)
    device = device or input_ids.device
    flat_ids = input_ids[am]
    pos = (torch.cumsum(am.long(), -1) - 1)[am].to(torch.int32)
    lens_cpu = lens.tolist()
    info = SeqInfo(lens_cpu, device=device)
    # packed start of every row
    starts = torch.zeros(B, dtype=torch.long, device=input_ids.device)
    if B > 1:
        starts[1:] = torch.cumsum(lens, 0)[:-1]
    p_valid = am[:, :P].sum(-1)                                   # valid prompt tokens per row
    r_valid = am[:, P:].sum(-1)
    k = torch.arange(R, device=input_ids.device)[None, :].expand(B, R)
    valid = k < r_valid[:, None]
    rows, cols = valid.nonzero(as_tuple=True)
    sel = starts[rows] + p_valid[rows] - 1 + cols
    labels = input_ids[rows, P + cols]
    return PackedBatch(flat_ids.to(device), pos.to(device), info, sel.to(device), labels.to(device),
                       rows.to(device), cols.to(device), B, R)


def get_response_mask(responses: torch.Tensor, eos_token_id, dtype=torch.int64) -> torch.Tensor:
    """1 up to and including the first EOS of each row (reference: torch_functional.py:209-229)."""
    eos_ids = eos_token_id if isinstance(eos_token_id, (list, tuple)) else [eos_token_id]
    is_eos = torch.zeros_like(responses, dtype=torch.bool)
    for e in eos_ids:
        if e is not None:
            is_eos |= responses == e
    after = (torch.cumsum(is_eos.long(), -1) - is_eos.long()) > 0
    return (~after).to(dtype)


def position_ids_from_mask(attention_mask: torch.Tensor) -> torch.Tensor:
    return torch.clamp(torch.cumsum(attention_mask.long(), -1) - 1, min=0)
