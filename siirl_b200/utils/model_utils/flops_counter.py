"""Model FLOPs and MFU (reference: siirl/utils/model_utils/flops_counter.py:33-369, whose device table has no
Blackwell entry so its MFU reads 0 on B200).  ``FlopsCounter.estimate_flops(batch_seqlens, delta_time)`` returns
``(achieved TFLOP/s, promised TFLOP/s)`` for a training pass (forward + backward = 3 x forward); ``forward_only``
gives the forward figure.  Attention FLOPs use the causal count ``sum(s^2)`` per sequence."""
from __future__ import annotations

from typing import Sequence, Tuple

import torch

from ...models.config import DecoderConfig

# dense bf16 tensor peaks in TFLOP/s (sparsity figures halved)
DEVICE_PEAK_TFLOPS = {"B200": 2250.0, "GB200": 2500.0, "B100": 1750.0, "H200": 989.0, "H100": 989.0, "H800": 989.0,
                      "H20": 148.0, "A100": 312.0, "A800": 312.0, "L40": 181.0, "L20": 119.5, "910B": 354.0}


def get_device_peak_tflops(name: str = None) -> float:
    if name is None:
        name = torch.cuda.get_device_name() if torch.cuda.is_available() else "cpu"
    for key, val in DEVICE_PEAK_TFLOPS.items():
        if key in name:
            return val
    return float("inf")


class FlopsCounter:
    def __init__(self, cfg: DecoderConfig):
        self.cfg = cfg

    def _attention_params(self) -> int:
        c = self.cfg
        if c.is_mla:
            nh, dn, dr, dv, R = c.num_heads, c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim, c.kv_lora_rank
            q = c.hidden_size * c.q_lora_rank + c.q_lora_rank * nh * (dn + dr) if c.q_lora_rank > 0 else \
                c.hidden_size * nh * (dn + dr)
            return q + c.hidden_size * (R + dr) + R * nh * (dn + dv) + nh * dv * c.hidden_size
        return c.hidden_size * c.qkv_width + c.q_width * c.hidden_size

    def _mlp_params(self, layer: int) -> int:
        """GEMM parameters one token touches in layer ``layer``'s MLP: a mixture-of-experts layer counts the router,
        the active routed experts and the shared experts; the first ``first_k_dense_replace`` layers of the
        DeepSeek-V3 family are dense."""
        c = self.cfg
        dense_first = int(getattr(c, "first_k_dense_replace", 0) or 0)
        if c.is_moe and layer >= dense_first:
            mlp = c.num_experts_per_tok * 3 * c.hidden_size * c.moe_intermediate_size + c.num_experts * c.hidden_size
            return mlp + 3 * c.hidden_size * int(getattr(c, "shared_expert_intermediate_size", 0) or 0)
        return 3 * c.hidden_size * c.intermediate_size

    def dense_params_per_token(self) -> int:
        """Parameters touched by one token in the GEMMs (MoE counts the active experts only)."""
        c = self.cfg
        head = c.hidden_size * (1 if c.value_head else c.vocab_size)
        return c.num_layers * self._attention_params() + sum(self._mlp_params(i) for i in range(c.num_layers)) + head

    def forward_flops(self, batch_seqlens: Sequence[int]) -> float:
        c = self.cfg
        tokens = float(sum(batch_seqlens))
        dense = 2.0 * self.dense_params_per_token() * tokens
        pairs = sum(0.5 * s * s for s in batch_seqlens)              # causal (query, key) pairs
        if c.is_mla:
            per_pair = c.num_heads * (c.qk_nope_head_dim + c.qk_rope_head_dim + c.v_head_dim)   # scores + values
        else:
            per_pair = 2.0 * c.num_heads * c.head_dim
        return dense + 2.0 * c.num_layers * per_pair * pairs

    def estimate_flops(self, batch_seqlens: Sequence[int], delta_time: float,
                       forward_only: bool = False) -> Tuple[float, float]:
        flops = self.forward_flops(batch_seqlens) * (1.0 if forward_only else 3.0)
        return flops / max(delta_time, 1e-9) / 1e12, get_device_peak_tflops()

    def mfu(self, batch_seqlens: Sequence[int], delta_time: float, forward_only: bool = False,
            n_gpus: int = 1) -> float:
        achieved, peak = self.estimate_flops(batch_seqlens, delta_time, forward_only)
        return achieved / n_gpus / peak if peak != float("inf") else 0.0
