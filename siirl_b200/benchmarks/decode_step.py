"""Decode-step micro-benchmark of the rollout engine (used for the launch list / ncu captures under profiles/).

    python -m siirl_b200.benchmarks.decode_step --model qwen2.5-7b --layers 4 --seqs 64 --context 640 --steps 8

Builds a random-init decoder (optionally truncated to ``--layers`` layers so a capture stays small), prefills
``--seqs`` prompts of ``--context`` tokens and times ``--steps`` eager decode steps (no CUDA graph, so every kernel
is visible to a profiler) and the same steps replayed from a CUDA graph."""
from __future__ import annotations

import argparse
import json

import torch

from ..engine.rollout.native_engine import RolloutEngine, SamplingParams
from ..models.config import get_config
from ..models.decoder import build_model
from ..ops import lib


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--seqs", type=int, default=64)
    ap.add_argument("--context", type=int, default=640)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--decode-kernel", default="", choices=["", "simple", "split"],
                    help="decode attention kernel (default: the package's)")
    ap.add_argument("--max-model-len", type=int, default=0, help="engine limit (0: just enough for this run); the "
                    "training configuration uses prompt + response = 5120")
    ap.add_argument("--n", type=int, default=1, help="samples per prompt (prefix blocks shared by the n samples)")
    args = ap.parse_args()
    if args.decode_kernel:
        from ..ops import kv_cache
        kv_cache.set_decode_kernel(args.decode_kernel)
    cfg = get_config(args.model, {"num_layers": args.layers} if args.layers else None)
    dev = torch.device("cuda")
    model = build_model(cfg, dtype=torch.bfloat16, device=dev, seed=0)
    res = {"model": args.model, "layers": cfg.num_layers, "seqs": args.seqs, "context": args.context,
           "max_model_len": args.max_model_len, "n": args.n, "decode_kernel": args.decode_kernel or "default"}
    # prompts are prefilled at most 256 k tokens per engine iteration (a whole 256 x 2700 batch would need a 24 GB MLP
    # intermediate); every sequence decodes `extra` more rounds than the three of a single-batch prefill, so that a
    # round exists in which all sequences are active (the one that is reported)
    total_prompt = args.seqs // args.n * args.context
    batched = max(8192, min(total_prompt, 262144))
    extra = (total_prompt + batched - 1) // batched - 1
    for graph in ([False] if args.no_graph else [False, True]):
        eng = RolloutEngine(model, max_num_seqs=args.seqs,
                            max_model_len=args.max_model_len or args.context + (4 + extra) * args.steps + 64,
                            use_cuda_graph=graph, sync_interval=args.steps, max_num_batched_tokens=batched)
        g = torch.Generator().manual_seed(0)
        prompts = [torch.randint(3, cfg.vocab_size, (args.context,), generator=g).tolist()
                   for _ in range(args.seqs // args.n)]
        sp = SamplingParams(n=args.n, temperature=1.0, max_new_tokens=1 + (3 + extra) * args.steps, eos_token_id=None)
        # generate = prefill + first token + 3 rounds of `steps` decode steps; time the last round only
        times = []
        orig = eng._run_decode_steps

        def timed(k, *a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            orig(k, *a, **kw)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) / k)

        eng._run_decode_steps = timed
        eng.generate(prompts, sp)
        lib.check_status()
        # rounds 0 .. extra-1 run while later prompts are still being prefilled; round extra + 2 is the third with every
        # sequence active and none finished
        res["graph_ms_per_step" if graph else "eager_ms_per_step"] = times[min(extra + 2, len(times) - 1)]
        eng.sleep()
    print(json.dumps(res))


if __name__ == "__main__":
    main()
