"""Library arm of the headline benchmark (``python bench.py --impl library``): the same GRPO step through the stack the
reference would use on this box -- vLLM for rollout, Hugging Face transformers + flash-attn + ``torch.optim.AdamW`` for
the two scoring passes and the update (the reference: siirl/engine/fsdp_workers.py:1090-1150 and
siirl/engine/rollout/vllm_rollout/vllm_rollout_spmd.py:261-416).  Nothing of ``siirl_b200`` runs on this path except
the architecture preset (to write the HF ``config.json``) and the synthetic prompt generator.

It is NOT the reference (that arm stays ``--impl reference``); it is a bar on the same box: ``impl`` is printed as
``"library"``.  One process, one GPU.  What it leaves out, all in the library stack's favour: no train -> rollout
weight synchronisation (the engine keeps its own random weights), no FSDP wrapping, no Ray.

Step: vLLM generates ``n`` samples per prompt (``ignore_eos``, temperature 1), then the HF policy scores them (old
log-probs), a second HF copy scores them (reference log-probs), rewards / group advantages are computed, and the policy
takes one clipped-loss + KL AdamW step over micro-batches with activation checkpointing.  The engine sleeps
(``enable_sleep_mode``) while the trainer works, like the reference's hybrid engine.
"""
from __future__ import annotations

import json
import os
import tempfile
import time


def run(args, process_start: float) -> int:
    import torch

    from siirl_b200.models.config import get_config

    def elapsed() -> float:
        return time.time() - process_start

    dev = torch.device("cuda:0")
    cfg = get_config(args.model)
    tmp = tempfile.mkdtemp(prefix="library_arm_")
    hf_cfg = cfg.to_hf_config()
    hf_cfg["max_position_embeddings"] = max(8192, args.prompt_max + args.max_response + 64)
    with open(os.path.join(tmp, "config.json"), "w") as f:
        json.dump(hf_cfg, f)
    try:
        from vllm import LLM, SamplingParams
        import transformers
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "library", "unavailable": f"{type(e).__name__}: {e}"[:300]}), flush=True)
        return 0

    # ---- rollout engine --------------------------------------------------------------------------------------------
    max_len = args.prompt_max + args.max_response + 8
    try:
        llm = LLM(model=tmp, skip_tokenizer_init=True, load_format="dummy", dtype="bfloat16", seed=0,
                  gpu_memory_utilization=0.45, max_model_len=max_len, enable_sleep_mode=True,
                  max_num_seqs=args.prompts_per_gpu * args.n, enable_prefix_caching=True)
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "library", "unavailable": f"vLLM engine did not start: {type(e).__name__}: {e}"[:300]}),
              flush=True)
        return 0
    sp = SamplingParams(n=args.n, temperature=1.0, top_p=1.0, max_tokens=args.max_response, ignore_eos=True,
                        detokenize=False)
    llm.sleep(level=1)

    # ---- trainer ---------------------------------------------------------------------------------------------------
    hcfg = transformers.AutoConfig.from_pretrained(tmp)
    try:
        hcfg._attn_implementation = "flash_attention_2"
    except Exception:  # noqa: BLE001
        pass
    torch.manual_seed(0)

    def build():
        with torch.device(dev):
            m = transformers.AutoModelForCausalLM.from_config(hcfg, dtype=torch.bfloat16,
                                                              attn_implementation="flash_attention_2")
        return m
    policy, ref = build(), build()
    ref.load_state_dict(policy.state_dict())
    ref.requires_grad_(False)
    policy.gradient_checkpointing_enable()
    policy.config.use_cache = False
    opt = torch.optim.AdamW(policy.parameters(), lr=1e-6, fused=True)

    def token_logprobs(model, ids, mask, resp_len, grad: bool):
        """``ids, mask [B, L]`` right-aligned prompts + responses -> log-probs of the last ``resp_len`` tokens."""
        ctx = torch.enable_grad() if grad else torch.no_grad()
        with ctx:
            hidden = model.model(input_ids=ids, attention_mask=mask).last_hidden_state[:, -resp_len - 1:-1]
            labels = ids[:, -resp_len:]
            out = []
            for c0 in range(0, resp_len, 1024):                  # vocabulary logits one chunk of positions at a time

                def chunk(h, y):
                    lg = model.lm_head(h).float()
                    return torch.log_softmax(lg, -1).gather(-1, y[..., None])[..., 0]
                h, y = hidden[:, c0:c0 + 1024], labels[:, c0:c0 + 1024]
                out.append(torch.utils.checkpoint.checkpoint(chunk, h, y, use_reentrant=False) if grad else chunk(h, y))
            return torch.cat(out, 1)

    gen = torch.Generator().manual_seed(1234)

    def make_prompts():
        lens = torch.randint(args.prompt_min, args.prompt_max + 1, (args.prompts_per_gpu,), generator=gen).tolist()
        return [torch.randint(3, 1000, (n,), generator=gen).tolist() for n in lens]

    def one_step():
        t0 = time.time()
        split = {}
        prompts = make_prompts()
        llm.wake_up()
        ta = time.time()
        outs = llm.generate([{"prompt_token_ids": p} for p in prompts], sp, use_tqdm=False)
        llm.sleep(level=1)
        torch.cuda.synchronize()
        split["rollout"] = time.time() - ta
        rows = [(p, list(c.token_ids)) for p, o in zip(prompts, outs) for c in o.outputs]
        R = max(len(r) for _, r in rows)
        P = max(len(p) for p, _ in rows)
        B = len(rows)
        ids = torch.zeros(B, P + R, dtype=torch.int64)
        mask = torch.zeros(B, P + R, dtype=torch.int64)
        rmask = torch.zeros(B, R)
        for i, (p, r) in enumerate(rows):                       # left-padded prompt, right-padded response
            ids[i, P - len(p):P] = torch.tensor(p)
            ids[i, P:P + len(r)] = torch.tensor(r)
            mask[i, P - len(p):P + len(r)] = 1
            rmask[i, :len(r)] = 1
        tokens = int(mask.sum())
        reward = torch.tensor([float(r[-1] % 2 == 0) for _, r in rows])
        grp = reward.view(-1, args.n)
        adv = ((grp - grp.mean(1, keepdim=True)) / (grp.std(1, keepdim=True) + 1e-6)).reshape(-1)
        mb = args.micro_batch

        def scoring(model, key):
            ta = time.time()
            vals = []
            for i in range(0, B, mb):
                vals.append(token_logprobs(model, ids[i:i + mb].to(dev), mask[i:i + mb].to(dev), R, False))
            torch.cuda.synchronize()
            split[key] = time.time() - ta
            return torch.cat(vals)
        old = scoring(policy, "old_log_prob")
        refp = scoring(ref, "ref_log_prob")
        ta = time.time()
        opt.zero_grad(set_to_none=True)
        for i in range(0, B, mb):
            lp = token_logprobs(policy, ids[i:i + mb].to(dev), mask[i:i + mb].to(dev), R, True)
            m = rmask[i:i + mb].to(dev)
            a = adv[i:i + mb].to(dev)[:, None]
            ratio = torch.exp(lp - old[i:i + mb])
            pg = -torch.minimum(ratio * a, ratio.clamp(0.8, 1.2) * a)
            d = refp[i:i + mb] - lp
            kl = torch.exp(d) - d - 1
            loss = ((pg + 0.001 * kl) * m).sum() / m.sum().clamp(min=1) * (min(mb, B - i) / B)
            loss.backward()
        torch.nn.utils.clip_grad_norm_(policy.parameters(), 1.0)
        opt.step()
        torch.cuda.synchronize()
        split["actor_train"] = time.time() - ta
        split["step"] = time.time() - t0
        return tokens, split

    # ---- warm-up and timed steps under the wall-clock budget ------------------------------------------------------
    t_first = time.time()
    one_step()
    t_full = time.time() - t_first
    warm_done = 1
    while warm_done < args.warmup and elapsed() + 2.2 * t_full < args.budget_s:
        one_step()
        warm_done += 1
    K = max(1, min(args.steps, int((args.budget_s - elapsed()) // max(t_full, 1e-3))))
    tokens, wall, done, split = 0, 0.0, 0, {}
    for _ in range(K):
        torch.cuda.synchronize()
        ta = time.time()
        tk, split = one_step()
        torch.cuda.synchronize()
        wall += time.time() - ta
        tokens += tk
        done += 1
        print(json.dumps({
            "metric": "grpo_tokens_per_second", "value": tokens / wall, "unit": "tokens/s", "n_gpus": 1, "steps": done,
            "warmup": warm_done, "requested_steps": args.steps, "requested_warmup": args.warmup,
            "ms_per_step": wall * 1e3 / done, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (random token prompts, random-init weights)", "impl": "library",
            "partial": done < K,
            "config": {"model": args.model, "global_batch": args.prompts_per_gpu * args.n,
                       "prompts": args.prompts_per_gpu, "samples_per_prompt": args.n,
                       "seq_len": f"prompt {args.prompt_min}-{args.prompt_max} + response <= {args.max_response}",
                       "parallelism": "1 GPU: vLLM rollout (sleep mode) + transformers / flash-attn / fused AdamW, "
                                      "no weight synchronisation", "micro_batch": args.micro_batch,
                       "timing": "host clock with device synchronisation around each step"},
            "step_split_s": {k: round(v, 3) for k, v in split.items()},
        }), flush=True)
    return 0
