"""Rollout of a multi-head-latent-attention model: the latent-cache engine against cache-free recomputation.

    python -m siirl_b200.benchmarks.mla_rollout --model moonlight-16b-a3b --layers 8 --prompts 16 --n 4 \
        --prompt-len 256 --response 64

Builds a random-init decoder (optionally truncated to ``--layers`` layers), generates ``--response`` tokens for
``--prompts x --n`` sequences with each engine and prints one JSON line with the device times (CUDA events around the
whole ``generate`` call, after one warm-up call), the share of greedy tokens on which the two engines agree (with
random weights the logits are nearly flat, so one rounding difference flips an arg-max and the sequences part: low
agreement says little), and the check that does not depend on that: the engine's log-probs of its own tokens against
the packed training forward over prompt + response.
"""
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
    ap.add_argument("--dense", action="store_true", help="replace every mixture-of-experts layer by the dense MLP "
                    "(isolates the attention path: expert choices flip on rounding differences)")
    args = ap.parse_args()
    over = {"num_layers": args.layers} if args.layers else {}
    if args.dense:
        over["first_k_dense_replace"] = args.layers or get_config(args.model).num_layers
    cfg = get_config(args.model, over or None)
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
    res = {"model": args.model + (" (dense MLPs)" if args.dense else ""), "layers": cfg.num_layers, "sequences": B, "prompt_len": args.prompt_len,
           "response": args.response, "latent_cache_s": round(t_lat, 3),
           "latent_cache_tokens_per_s": round(B * args.response / t_lat, 1),
           "latent_cache_gb": round(lat.cache_bytes() / 2 ** 30, 3),
           "expanded_kv_cache_gb": round(cfg.num_layers * B * (args.prompt_len + args.response + 8) * cfg.num_heads
                                         * (cfg.qk_nope_head_dim + cfg.qk_rope_head_dim + cfg.v_head_dim) * 2 / 2 ** 30, 3)}
    # teacher-forced check: log-probs the engine reported for its tokens vs. the training forward of the same sequences
    from ..ops.attention import SeqInfo
    worst, total, count = 0.0, 0.0, 0
    with torch.no_grad():
        for at in range(0, len(o_lat), 16):
            part = o_lat[at:at + 16]
            seqs = [prompts[o.prompt_index] + o.token_ids for o in part]
            ids = torch.tensor([t for q in seqs for t in q], device=dev)
            info = SeqInfo([len(q) for q in seqs], device=dev)
            labels = torch.roll(ids, -1)
            lp, _ = model.logprobs(ids, info.positions, info, labels, with_entropy=False)
            start = 0
            for o, q in zip(part, seqs):
                pl = len(q) - len(o.token_ids)
                mine = lp[start + pl - 1:start + len(q) - 1].float().cpu()
                d = (mine - torch.tensor(o.logprobs)).abs()
                worst, total, count = max(worst, float(d.max())), total + float(d.sum()), count + d.numel()
                start += len(q)
    res.update({"logprob_vs_training_forward_mean_abs": round(total / max(count, 1), 5),
                "logprob_vs_training_forward_max_abs": round(worst, 4)})
    if not args.skip_recompute:
        t_rec, o_rec = timed(RecomputeEngine(model, max_num_seqs=B, max_model_len=args.prompt_len + args.response + 8))
        same = sum(int(x == y) for p, q in zip(o_lat, o_rec) for x, y in zip(p.token_ids, q.token_ids))
        first = [abs(p.logprobs[0] - q.logprobs[0]) for p, q in zip(o_lat, o_rec)]
        res.update({"recompute_s": round(t_rec, 3), "speedup": round(t_rec / t_lat, 2),
                    "greedy_token_agreement": round(same / (B * args.response), 4),
                    "first_token_logprob_max_abs_diff": round(max(first), 4)})
    print(json.dumps(res), flush=True)


if __name__ == "__main__":
    main()
