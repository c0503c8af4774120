"""Rollout of a multi-head-latent-attention model: the latent-cache engine against cache-free recomputation.

    python -m siirl_b200.benchmarks.mla_rollout --model moonlight-16b-a3b --layers 8 --prompts 16 --n 4 \
        --prompt-len 256 --response 64

Builds a random-init decoder (optionally truncated to ``--layers`` layers), generates ``--response`` tokens for
``--prompts x --n`` sequences with each engine and prints one JSON line with the device times (CUDA events around the
whole ``generate`` call, after one warm-up call) and the share of tokens on which the two engines agree."""
from __future__ import annotations

import argparse
import json

import torch

from ..engine.rollout.latent_engine import LatentCacheEngine
from ..engine.rollout.native_engine import SamplingParams
from ..engine.rollout.recompute_engine import RecomputeEngine
from ..models.config import get_config
from ..models.decoder import build_model
from ..ops import lib


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="moonlight-16b-a3b")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--prompts", type=int, default=16)
    ap.add_argument("--n", type=int, default=4)
    ap.add_argument("--prompt-len", type=int, default=256)
    ap.add_argument("--response", type=int, default=64)
    ap.add_argument("--skip-recompute", action="store_true")
    args = ap.parse_args()
    cfg = get_config(args.model, {"num_layers": args.layers} if args.layers else None)
    dev = torch.device("cuda")
    model = build_model(cfg, dtype=torch.bfloat16, device=dev, seed=0)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 1000, (args.prompt_len - (i % 7),), generator=g).tolist() for i in range(args.prompts)]
    sp = SamplingParams(n=args.n, temperature=0.0, max_new_tokens=args.response, ignore_eos=True)
    B = args.prompts * args.n

    def timed(engine):
        engine.wake_up()
        engine.generate(prompts[:2], SamplingParams(n=1, temperature=0.0, max_new_tokens=4, ignore_eos=True))
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        outs = engine.generate(prompts, sp)
        b.record()
        torch.cuda.synchronize()
        lib.check_status()
        engine.sleep()
        return a.elapsed_time(b) / 1e3, outs

    lat = LatentCacheEngine(model, max_num_seqs=B, max_model_len=args.prompt_len + args.response + 8)
    t_lat, o_lat = timed(lat)
    res = {"model": args.model, "layers": cfg.num_layers, "sequences": B, "prompt_len": args.prompt_len,
           "response": args.response, "latent_cache_s": round(t_lat, 3),
           "latent_cache_tokens_per_s": round(B * args.response / t_lat, 1),
           "latent_cache_gb": round(lat.cache_bytes() / 2 ** 30, 3),
           "expanded_kv_cache_gb": round(cfg.num_layers * B * (args.prompt_len + args.response + 8) * cfg.num_heads
                                         * (cfg.qk_nope_head_dim + cfg.qk_rope_head_dim + cfg.v_head_dim) * 2 / 2 ** 30, 3)}
    if not args.skip_recompute:
        t_rec, o_rec = timed(RecomputeEngine(model, max_num_seqs=B, max_model_len=args.prompt_len + args.response + 8))
        same = sum(int(x == y) for p, q in zip(o_lat, o_rec) for x, y in zip(p.token_ids, q.token_ids))
        res.update({"recompute_s": round(t_rec, 3), "speedup": round(t_rec / t_lat, 2),
                    "greedy_token_agreement": round(same / (B * args.response), 4)})
    print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
