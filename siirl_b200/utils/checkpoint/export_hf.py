"""Turn a sharded training checkpoint into a Hugging Face directory, offline and on CPU.

    python -m siirl_b200.utils.checkpoint.export_hf --checkpoint ckpt/global_step_100/actor_agent_0 --out exported/

A training checkpoint holds one slice of the flat bf16 parameter buffer per rank
(``model_world_size_<W>_rank_<r>.pt``) plus a manifest with the parameter offsets and the model configuration.  This
reads all slices in one process, rebuilds the model and writes ``config.json`` + safetensors under the family's
checkpoint names (``models/hf_io.py``), the same files ``checkpoint.contents=[..., hf_model]`` writes during
training.  ``--tokenizer`` copies a tokenizer directory beside the weights.

Parameter-sharded checkpoints (``sharding=zero3``) are reassembled too: the replicated remainder (embedding, final
norm, head, vision tower) from its slices, every decoder layer from the ranks' pieces of its flat unit (the layout of
``parallel/sharded_params.py``: parameters packed at 128-element boundaries, unit length rounded up to a multiple of
``128 x world``, rank r holds elements ``[r, r + 1) x unit / world`` of every unit).  Expert-parallel, hybrid-sharded
and tensor-parallel checkpoints keep per-rank files that only the layout that wrote them can read: export those from
the training job with ``hf_model`` in ``checkpoint.contents``.
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
    cfg = DecoderConfig.from_dict(manifest["model_config"]) if manifest.get("model_config") else None
    sharded_layers = bool(manifest.get("expert_parallel"))
    if sharded_layers and (cfg is None or cfg.is_moe):
        raise ValueError("expert-parallel checkpoint: the experts live in per-rank files of the layout that wrote "
                         "them; export from the training job with hf_model in checkpoint.contents")
    if os.path.isdir(os.path.join(checkpoint, "tp_rank_0")):
        raise ValueError("tensor-parallel training checkpoint (tp_rank_* directories): export from the training job")
    if manifest.get("model_config") is None or manifest.get("offsets") is None:
        raise ValueError(f"{checkpoint}: the manifest holds no model configuration / parameter offsets")
    missing = [r for r in range(int(manifest["world_size"])) if not os.path.exists(
        os.path.join(checkpoint, f"model_world_size_{manifest['world_size']}_rank_{r}.pt"))]
    if missing:
        raise FileNotFoundError(f"{checkpoint}: parameter slices of rank(s) {missing} are missing")
    model = build_model(cfg, dtype=getattr(torch, dtype), device="cpu", seed=0)
    if sharded_layers:
        _load_layer_units(model, checkpoint, int(manifest["world_size"]))
        store = FlatParamStore(model, optimizer_state=False, with_grad=False,
                               param_filter=lambda n: not n.startswith("layers."))
    else:
        store = FlatParamStore(model, optimizer_state=False, with_grad=False)
    ShardedCheckpointManager(model, store, cfg).load(checkpoint, contents=["model"])
    tok = None
    if tokenizer:
        from ...data_coordinator.dataloader.tokenizer import load_tokenizer
        tok = load_tokenizer(tokenizer, cfg.vocab_size)
    save_hf_model(model, out, tokenizer=tok)
    return out


def _load_layer_units(model, checkpoint: str, world: int) -> None:
    """Decoder layers of a parameter-sharded checkpoint: rank r's file holds, for every layer, elements
    ``[r * piece, (r + 1) * piece)`` of the layer's flat unit."""
    import torch

    from ...parallel.flat_params import _ALIGN, _round_up
    layers = list(model.layers)
    tables, unit_len = [], 0
    for layer in layers:
        off, table = 0, []
        for name, p in layer.named_parameters():
            table.append((p, off, p.numel()))
            off = _round_up(off + p.numel(), _ALIGN)
        tables.append(table)
        unit_len = max(unit_len, off)
    unit_len = _round_up(unit_len, _ALIGN * world)
    piece = unit_len // world
    flats = []
    for r in range(world):
        path = os.path.join(checkpoint, f"experts_world_size_{world}_rank_{r}.pt")
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path}: the layer pieces of rank {r} are missing")
        flat = torch.load(path, map_location="cpu", weights_only=False)["flat"]
        if flat.numel() != len(layers) * piece:
            raise ValueError(f"{path}: {flat.numel()} elements, expected {len(layers)} layers x {piece} (a hybrid-"
                             f"sharded or differently laid out checkpoint: export from the training job)")
        flats.append(flat)
    with torch.no_grad():
        for i, table in enumerate(tables):
            unit = torch.cat([f[i * piece:(i + 1) * piece] for f in flats])
            for p, off, k in table:
                p.copy_(unit[off:off + k].view(p.shape).to(p.dtype))


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
