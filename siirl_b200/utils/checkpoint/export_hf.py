"""Turn a sharded training checkpoint into a Hugging Face directory, offline and on CPU.

    python -m siirl_b200.utils.checkpoint.export_hf --checkpoint ckpt/global_step_100/actor_agent_0 --out exported/

A training checkpoint holds one slice of the flat bf16 parameter buffer per rank
(``model_world_size_<W>_rank_<r>.pt``) plus a manifest with the parameter offsets and the model configuration.  This
reads all slices in one process, rebuilds the model and writes ``config.json`` + safetensors under the family's
checkpoint names (``models/hf_io.py``), the same files ``checkpoint.contents=[..., hf_model]`` writes during
training.  ``--tokenizer`` copies a tokenizer directory beside the weights.  Expert-parallel, parameter-sharded
(``sharding=zero3``) and tensor-parallel checkpoints keep per-rank files that only the layout that wrote them can
read: export those from the training job with ``hf_model`` in ``checkpoint.contents``.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Optional


def export(checkpoint: str, out: str, tokenizer: Optional[str] = None, dtype: str = "bfloat16") -> str:
    import torch

    from ...models.config import DecoderConfig
    from ...models.decoder import build_model
    from ...models.hf_io import save_hf_model
    from ...parallel.flat_params import FlatParamStore
    from .checkpoint_manager import ShardedCheckpointManager
    with open(os.path.join(checkpoint, "manifest.json")) as f:
        manifest = json.load(f)
    if manifest.get("expert_parallel"):
        raise ValueError("expert-parallel or parameter-sharded (sharding=zero3) checkpoint: part of the weights lives "
                         "in per-rank files of the layout that wrote them; export from the training job with "
                         "hf_model in checkpoint.contents")
    if os.path.isdir(os.path.join(checkpoint, "tp_rank_0")):
        raise ValueError("tensor-parallel training checkpoint (tp_rank_* directories): export from the training job")
    if manifest.get("model_config") is None or manifest.get("offsets") is None:
        raise ValueError(f"{checkpoint}: the manifest holds no model configuration / parameter offsets")
    missing = [r for r in range(int(manifest["world_size"])) if not os.path.exists(
        os.path.join(checkpoint, f"model_world_size_{manifest['world_size']}_rank_{r}.pt"))]
    if missing:
        raise FileNotFoundError(f"{checkpoint}: parameter slices of rank(s) {missing} are missing")
    cfg = DecoderConfig.from_dict(manifest["model_config"])
    model = build_model(cfg, dtype=getattr(torch, dtype), device="cpu", seed=0)
    store = FlatParamStore(model, optimizer_state=False, with_grad=False)
    ShardedCheckpointManager(model, store, cfg).load(checkpoint, contents=["model"])
    tok = None
    if tokenizer:
        from ...data_coordinator.dataloader.tokenizer import load_tokenizer
        tok = load_tokenizer(tokenizer, cfg.vocab_size)
    save_hf_model(model, out, tokenizer=tok)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--checkpoint", required=True, help="a role directory of a checkpoint, e.g. global_step_N/actor_agent_0")
    ap.add_argument("--out", required=True)
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "float16"])
    args = ap.parse_args(argv)
    out = export(args.checkpoint, args.out, args.tokenizer, args.dtype)
    print(f"wrote {out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
