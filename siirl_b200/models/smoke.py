"""Tiny end-to-end exercise of the flagship path on one GPU: packed decoder forward + backward through the
tcgen05 GEMM / attention / LM-head kernels, one sharded-AdamW step, and a short paged-KV rollout."""
from __future__ import annotations

import torch

from ..engine.rollout.native_engine import RolloutEngine, SamplingParams
from ..ops import lib
from ..ops.attention import SeqInfo
from ..parallel.flat_params import FlatParamStore
from .config import get_config
from .decoder import build_model


def run_smoke(device: torch.device) -> dict:
    torch.cuda.set_device(device)
    cfg = get_config("tiny-gpu")
    model = build_model(cfg, dtype=torch.bfloat16, device=device, seed=0, gradient_checkpointing=True)
    store = FlatParamStore(model)
    info = SeqInfo([96, 200, 33], device=device)
    ids = torch.randint(3, cfg.vocab_size, (info.total,), device=device)
    logp, ent = model.logprobs(ids, info.positions, info, torch.roll(ids, -1), temperature=1.0)
    loss = -(logp.mean()) - 0.01 * ent.mean()
    loss.backward()
    norm = store.step(lr=1e-4)
    eng = RolloutEngine(model, max_num_seqs=8, max_model_len=256, num_blocks=32, sync_interval=4)
    outs = eng.generate([[5, 6, 7, 8], list(range(10, 90))], SamplingParams(n=2, temperature=1.0, max_new_tokens=12))
    torch.cuda.synchronize()
    lib.check_status()
    assert torch.isfinite(loss).item() and torch.isfinite(norm).item()
    assert len(outs) == 4 and all(len(o.token_ids) == 12 for o in outs)
    res = {"loss": float(loss.detach()), "grad_norm": float(norm.detach()), "kernel_launches": lib.launch_count()}
    print(f"smoke ok: {res}")
    return res
