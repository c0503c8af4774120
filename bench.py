"""Headline benchmark: GRPO end-to-end throughput (rollout + reward + advantage + old/ref log-probs + actor update)
of a Qwen2.5-7B-architecture model with random-init bf16 weights and synthetic prompts.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 3 --warmup 3

One rank per GPU (weak scaling: ``--prompts-per-gpu`` prompts x ``--n`` samples on every rank).  Every step goes
through the user-facing call ``DAGWorker.train_step()``: the dataloader's batch sits in pinned host memory, is copied
to the device, walks the DAG (rollout, reward, log-probs, advantage, update) and its result tensors and metrics are
read back to the host.  The same steps give both numbers of the JSON line: ``value`` is all ranks' tokens divided by
the CUDA-event time of the timed steps (max over ranks), ``e2e.value`` the same tokens divided by the host clock
around the same calls.

``--steps`` / ``--warmup`` are upper bounds under a wall-clock budget (``--budget-s``, counted from process start and
including the model build): one step of the named configuration takes minutes, so the script measures its first
full-size warm-up step and then runs as many timed steps as fit (at least one).  When a full-size step is expected
to take longer than a minute, all warm-up steps but the last run with short responses (they exercise every kernel,
the allocator and the collectives; the last, full-size one captures the decode graphs at their final shapes).  Rank 0
prints the cumulative JSON line after every finished timed step; the last line printed is the result.

``--impl reference`` is the arm that would run the unmodified reference; it reports why it cannot run here.
``--impl library`` (one GPU) runs the same step through vLLM, transformers, flash-attn and ``torch.optim.AdamW``
(``baseline/library_arm.py``) and prints ``"impl": "library"``.
"""
from __future__ import annotations

import time

_T_PROCESS_START = time.time()

import os

# one GPU holds weights, reference copy, fp32 gradients and the whole Adam state (151 GB of 180): growing segments
# instead of fixed-size blocks keeps the remaining memory usable for the 41k-token micro-batches
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

import argparse
import json
import statistics
import subprocess
import sys
import threading

METRIC = "grpo_tokens_per_second"
BASELINE_TOKENS_PER_S_PER_GPU = 3473.837  # reference quick-start log (Qwen2.5-0.5B, 1 GPU, step 2)
SHORT_RESPONSE = 128                       # response limit of the short warm-up steps
AUTO_SHARDS_PARAMS = True                  # what --param-sharding auto means on two or more GPUs (the named configuration)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "library"],
                    help="library: the same step through vLLM + transformers + flash-attn + torch AdamW (1 GPU), a bar "
                         "on this box that is not the reference")
    ap.add_argument("--budget-s", type=float, default=600.0,
                    help="wall-clock budget of the whole run, from process start; --steps/--warmup are upper bounds")
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--prompts-per-gpu", type=int, default=32)  # 256 prompts on 8 GPUs
    ap.add_argument("--n", type=int, default=8)
    ap.add_argument("--prompt-min", type=int, default=256)
    ap.add_argument("--prompt-max", type=int, default=1024)
    ap.add_argument("--max-response", type=int, default=4096)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--rollout-tp", type=int, default=0,
                    help="rollout tensor-parallel size; 0 = the named configuration (2 on two or more GPUs, else 1)")
    ap.add_argument("--param-sharding", default="auto", choices=["auto", "replicated", "sharded"],
                    help="actor / reference weights: sharded over the ranks and gathered per layer, or replicated")
    ap.add_argument("--offload", action="store_true", help="keep activation checkpoints in pinned host memory")
    return ap.parse_args()


def reference_arm(args) -> int:
    """The reference (installed with --no-deps under baseline/_ref) needs ray, omegaconf/hydra, tensordict, dacite,
    vllm-compatible torch and more; none can be installed offline, so its public entry point cannot start."""
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, os.path.join(here, "baseline", "_ref"))
    why = None
    try:
        import importlib
        importlib.import_module("siirl.main_dag")
    except Exception as e:  # noqa: BLE001
        why = f"reference entry point siirl.main_dag does not import offline: {type(e).__name__}: {e}"
    if why is None:
        why = "reference imports but its Ray/vLLM runtime cannot be started without network-installed dependencies"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}), flush=True)
    return 0


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of this rank's GPU while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "500", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 8:
                self.rows.append(parts)

    def summary(self):
        sm, reasons, smax = [], set(), None
        for r in list(self.rows):
            try:
                sm.append(float(r[1]))
                smax = float(r[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        busy = [x for x in sm if smax is None or x > 0.3 * smax] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": smax,
                "reasons": sorted(reasons), "samples": len(sm)}

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return self.summary()


def resolve_parallelism(args, world: int):
    tp = args.rollout_tp if args.rollout_tp > 0 else (2 if world >= 2 else 1)
    if world % tp:
        tp = 1
    sharded = args.param_sharding == "sharded" or (args.param_sharding == "auto" and world >= 2 and
                                                   AUTO_SHARDS_PARAMS)
    return tp, sharded


def build_config(args, world: int):
    from siirl_b200.params import parse_config
    bs = args.prompts_per_gpu * world
    tp, sharded = resolve_parallelism(args, world)
    ov = [
        "algorithm.adv_estimator=grpo",
        "data.synthetic=arith", f"data.synthetic_size={max(64, bs * 8)}",
        f"data.synthetic_min_prompt={args.prompt_min}", f"data.synthetic_max_prompt={args.prompt_max}",
        f"data.max_prompt_length={args.prompt_max}", f"data.max_response_length={args.max_response}",
        f"data.train_batch_size={bs}", "data.shuffle=True",
        f"actor_rollout_ref.model.arch_preset={args.model}", "actor_rollout_ref.model.random_init=True",
        "actor_rollout_ref.model.enable_gradient_checkpointing=True",
        f"actor_rollout_ref.model.enable_activation_offload={bool(args.offload)}",
        # single GPU: the whole Adam state (8 bytes per parameter) is idle during rollout; in pinned host memory it
        # leaves room for the KV blocks of all 256 sequences of the step
        f"actor_rollout_ref.actor.fsdp_config.optimizer_offload={world == 1}",
        f"actor_rollout_ref.actor.fsdp_config.sharding={'zero3' if sharded else 'zero2'}",
        f"actor_rollout_ref.rollout.n={args.n}", "actor_rollout_ref.rollout.temperature=1.0",
        f"actor_rollout_ref.rollout.tensor_model_parallel_size={tp}",
        # a tensor-parallel replica serves the prompts of all its ranks
        f"actor_rollout_ref.rollout.max_num_seqs={args.prompts_per_gpu * args.n * tp}",
        "actor_rollout_ref.rollout.gpu_memory_utilization=0.85", "actor_rollout_ref.rollout.free_cache_engine=True",
        "actor_rollout_ref.rollout.enforce_eager=False", "actor_rollout_ref.rollout.ignore_eos=False",
        f"actor_rollout_ref.actor.ppo_mini_batch_size={bs}",
        f"actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu={args.micro_batch}",
        f"actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu={args.micro_batch}",
        f"actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu={args.micro_batch}",
        "actor_rollout_ref.actor.use_kl_loss=True", "actor_rollout_ref.actor.kl_loss_type=low_var_kl",
        "actor_rollout_ref.actor.optim.lr=1e-6",
        f"trainer.n_gpus_per_node={world}", "trainer.nnodes=1", "trainer.val_before_train=False",
        "trainer.resume_mode=disable", "trainer.save_freq=-1", "trainer.test_freq=-1", "trainer.logger=[]",
        "trainer.total_training_steps=1000000",
    ]
    return parse_config(ov)


def main() -> int:
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.impl == "library":
        if int(os.environ.get("WORLD_SIZE", "1")) > 1:
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "library", "unavailable": "the library arm runs on one GPU"}), flush=True)
            return 0
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from baseline.library_arm import run as library_run
        return library_run(args, _T_PROCESS_START)
    import torch
    import torch.distributed as dist

    from siirl_b200.dag_worker.dagworker import DAGWorker
    from siirl_b200.main_dag import init_distributed, plan
    from siirl_b200.ops import lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun for N > 1"
    cfg = build_config(args, world)
    tp, sharded = resolve_parallelism(args, world)
    torch.cuda.set_device(local)
    init_distributed(cfg)
    _, assignment, pgm = plan(cfg, world)
    comm = None
    if world > 1:
        try:
            from siirl_b200.parallel.symm import SymmComm
            comm = SymmComm.create(dist.group.WORLD)
        except Exception as e:  # noqa: BLE001
            if rank == 0:
                print(f"[bench] peer-memory communicator unavailable ({e}); NCCL collectives", file=sys.stderr)
    worker = DAGWorker(cfg, pgm, assignment, comm=comm)
    worker.init_graph()
    dev = worker.device

    def elapsed() -> float:
        return time.time() - _T_PROCESS_START

    def agree(x: float, op) -> float:
        """The same decision on every rank (step counts drive collectives)."""
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=op)
        return float(t.item())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def one_step(short: bool = False):
        """One GRPO step through the public call; returns (tokens of this rank, h2d bytes, d2h bytes, wall s)."""
        worker.rollout_meta_overrides = {"response_length": min(SHORT_RESPONSE, args.max_response)} if short else {}
        t0 = time.perf_counter()
        try:
            m = worker.train_step()
        finally:
            worker.rollout_meta_overrides = {}
        assert m is not None
        return (int(worker.last_step_tokens), int(worker.last_h2d_bytes), int(worker.last_d2h_bytes),
                time.perf_counter() - t0)

    # ---- warm-up ---------------------------------------------------------------------------------------------
    avg_len = (args.prompt_min + args.prompt_max) / 2 + args.max_response
    from siirl_b200.engine.workers import resolve_model_config
    from siirl_b200.utils.model_utils.flops_counter import FlopsCounter
    seqs = args.prompts_per_gpu * args.n
    fwd_pflop = FlopsCounter(resolve_model_config(cfg.actor_rollout_ref.model)).forward_flops([avg_len] * seqs) / 1e15
    # rough a-priori step time: two scoring passes and the update (4 forward-equivalents with recompute) at about
    # 1 PFLOP/s, and a decode phase about as long as those together
    est_step_s = fwd_pflop * 6 * 2
    heavy = est_step_s > 60.0
    n_warm = max(args.warmup, 1)
    n_short = n_warm - 1 if heavy else 0
    for _ in range(n_short):
        one_step(short=True)
    full_warm = 0
    t_full = 0.0
    for i in range(n_warm - n_short):
        t_full = agree(one_step()[3], dist.ReduceOp.MAX if world > 1 else None)
        full_warm += 1
        # another full warm-up step only if it still leaves room for the requested timed steps
        left = args.budget_s - elapsed()
        if left < t_full * (1 + max(1, min(args.steps, 2))):
            break
    lib.check_status()
    margin = 20.0 + 0.05 * t_full
    k_fit = int((args.budget_s - elapsed() - margin) // max(t_full, 1e-3))
    K = int(agree(float(max(1, min(args.steps, k_fit))), dist.ReduceOp.MIN if world > 1 else None))

    # ---- timed steps -----------------------------------------------------------------------------------------
    sampler = ClockSampler(local)
    barrier()
    if rank == 0:
        sampler.start()
    launches0 = lib.launch_count()
    e0 = torch.cuda.Event(enable_timing=True)
    e0.record()
    wall0 = time.perf_counter()
    tokens = h2d = d2h = 0
    done = 0

    def report(final: bool):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(ev)
        wall = time.perf_counter() - wall0
        t = torch.tensor([ms, wall, float(tokens), float(lib.launch_count() - launches0)], dtype=torch.float64,
                         device=dev)
        if world > 1:
            mx, sm = t.clone(), t.clone()
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            dist.all_reduce(sm, op=dist.ReduceOp.SUM)
            ms, wall, tokens_all, launches = mx[0].item(), mx[1].item(), sm[2].item(), int(sm[3].item())
        else:
            tokens_all, launches = t[2].item(), int(t[3].item())
        if rank != 0:
            return
        value = tokens_all / (ms / 1e3)
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": done,
            "warmup": n_short + full_warm, "requested_steps": args.steps, "requested_warmup": args.warmup,
            "ms_per_step": ms / done, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / world) / BASELINE_TOKENS_PER_S_PER_GPU,
            "dtype": "bf16", "data": "synthetic (seeded a+b digit prompts, random-init weights)",
            "tokens_per_second_per_gpu": value / world,
            "config": {"model": args.model, "global_batch": args.prompts_per_gpu * world * args.n,
                       "prompts": args.prompts_per_gpu * world, "samples_per_prompt": args.n,
                       "seq_len": f"prompt {args.prompt_min}-{args.prompt_max} + response <= {args.max_response}",
                       "parallelism": f"dp{world}, actor and reference weights "
                                      f"{'sharded over the ranks (gathered per layer)' if sharded else 'replicated'}, "
                                      f"fp32 master / Adam state sharded, rollout tp{tp}",
                       "rollout_tp": tp, "param_sharding": "sharded" if sharded else "replicated",
                       "micro_batch": args.micro_batch, "l2": "inputs larger than L2 (15 GB of weights per pass)",
                       "warmup_detail": {"short_steps": n_short, "short_response_limit": SHORT_RESPONSE,
                                         "full_steps": full_warm, "full_step_s": round(t_full, 2)},
                       "budget_s": args.budget_s, "elapsed_s": round(elapsed(), 1),
                       "memory_plan": {"kv_arena_borrows_idle_grad_buffer": True,
                                       "adam_moments_in_pinned_host_memory_during_rollout": world == 1,
                                       "activation_checkpointing": True, "activation_offload": bool(args.offload)},
                       "baseline_note": "vs_baseline divides tokens/s/GPU by the reference's only published absolute "
                                        "number (3473.8 tokens/s/GPU, Qwen2.5-0.5B, 1 GPU of unstated type)"},
            "clocks": sampler.summary() if not final else clocks_final[0], "gpu_launches": launches,
            "impl": "native", "partial": not final,
            "step_split_s": {k: round(v, 4) for k, v in worker.timing_raw.items()},
            "engine_stats": {k: (round(v, 3) if isinstance(v, float) else v) for w_ in worker.workers.values()
                             for k, v in getattr(getattr(w_, "engine", None), "stats", {}).items()},
            "e2e": {"value": tokens_all / wall, "unit": "tokens/s", "ms_per_step": wall * 1e3 / done, "steps": done,
                    "h2d_bytes_per_step": h2d // done, "d2h_bytes_per_step": d2h // done,
                    "clock": "host perf_counter around DAGWorker.train_step (pinned host batch -> device, DAG walk, "
                             "result tensors and metrics read back), same steps as value"},
        }
        print(json.dumps(out), flush=True)

    clocks_final = [None]
    for i in range(K):
        tk, a, b, _ = one_step()
        tokens += tk
        h2d += a
        d2h += b
        done += 1
        if i + 1 < K:
            report(final=False)
    barrier()
    clocks_final[0] = sampler.stop() if rank == 0 else None
    lib.check_status()
    report(final=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
