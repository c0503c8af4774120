"""Headline benchmark: GRPO end-to-end throughput (rollout + reward + advantage + old/ref log-probs + actor update)
of a Qwen2.5-7B-architecture model with random-init bf16 weights and synthetic prompts.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench.py --gpus 8 --steps 3 --warmup 3

One rank per GPU (weak scaling: ``--prompts-per-gpu`` prompts x ``--n`` samples on every rank).  Rank 0 prints one
JSON line.  ``value`` is the whole-job tokens/s (prompt + response tokens of all ranks / step time) timed on the
device with CUDA events, max over ranks, with the step's prompt batch already resident on the GPU; ``e2e.value`` is
the same metric through the user-facing path (DAGWorker step: dataloader batch in pinned host memory -> H2D copy ->
... -> metrics read back to the host).  ``--impl reference`` is the arm that would run the unmodified reference; it
reports why it cannot run here.
"""
from __future__ import annotations

import os

# one GPU holds weights, reference copy, fp32 gradients and the whole Adam state (151 GB of 180): growing segments
# instead of fixed-size blocks keeps the remaining memory usable for the 41k-token micro-batches
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

METRIC = "grpo_tokens_per_second"
BASELINE_TOKENS_PER_S_PER_GPU = 3473.837  # reference quick-start log (Qwen2.5-0.5B, 1 GPU, step 2)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--prompts-per-gpu", type=int, default=32)  # 256 prompts on 8 GPUs
    ap.add_argument("--n", type=int, default=8)
    ap.add_argument("--prompt-min", type=int, default=256)
    ap.add_argument("--prompt-max", type=int, default=1024)
    ap.add_argument("--max-response", type=int, default=4096)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--rollout-tp", type=int, default=1)
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--offload", action="store_true", help="keep activation checkpoints in pinned host memory")
    ap.add_argument("--e2e-steps", type=int, default=0, help="steps of the end-to-end region (0: 1 when a step takes "
                    "longer than a minute, else --steps)")
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
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}))
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
                                          "-lms", "200", "-i", str(self.gpu)], stdout=subprocess.PIPE,
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

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = []
        reasons = set()
        smax = None
        for r in self.rows:
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


def build_config(args, world: int):
    from siirl_b200.params import parse_config
    bs = args.prompts_per_gpu * world
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
        f"actor_rollout_ref.rollout.n={args.n}", "actor_rollout_ref.rollout.temperature=1.0",
        f"actor_rollout_ref.rollout.tensor_model_parallel_size={args.rollout_tp}",
        f"actor_rollout_ref.rollout.max_num_seqs={args.prompts_per_gpu * args.n}",
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
    import torch
    import torch.distributed as dist

    from siirl_b200.dag_worker.dagworker import DAGWorker
    from siirl_b200.data_coordinator import preprocess_dataloader
    from siirl_b200.main_dag import init_distributed, plan
    from siirl_b200.ops import lib

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun for N > 1"
    cfg = build_config(args, world)
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

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    split = {}

    def run_steps(k: int, prestaged: bool):
        """Runs k GRPO steps; returns (tokens on this rank, h2d bytes, d2h bytes)."""
        tokens = h2d = d2h = 0
        real_run = worker.dataloader.run
        for _ in range(k):
            if prestaged:
                staged = preprocess_dataloader(real_run(), args.n).to(dev)
                torch.cuda.synchronize()
                worker.dataloader.run = lambda *a, **kw: staged
                worker._bench_prestaged = True
            m = worker._run_training_step(0, 0)
            worker.dataloader.run = real_run
            worker._bench_prestaged = False
            worker.global_steps += 1
            tokens += int(worker.last_step_tokens)
            split.clear()
            split.update({k: round(v, 4) for k, v in worker.timing_raw.items()})
            h2d += int(worker.last_h2d_bytes)
            d2h += int(worker.last_d2h_bytes)
            assert m is not None
        return tokens, h2d, d2h

    # warm-up (also captures the decode CUDA graphs and grows the allocator pools)
    run_steps(args.warmup, prestaged=True)
    lib.check_status()

    def timed(prestaged: bool, steps: int = 0):
        steps = steps or args.steps
        sampler = ClockSampler(local)
        barrier()
        if rank == 0:
            sampler.start()
        launches0 = lib.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        tokens, h2d, d2h = run_steps(steps, prestaged)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        barrier()
        clocks = sampler.stop() if rank == 0 else None
        t = torch.tensor([ms, float(tokens), float(lib.launch_count() - launches0)], dtype=torch.float64, device=dev)
        if world > 1:
            mx = t.clone()
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            sm = t.clone()
            dist.all_reduce(sm, op=dist.ReduceOp.SUM)
            ms, tokens_all, launches = mx[0].item(), sm[1].item(), int(sm[2].item())
        else:
            ms, tokens_all, launches = t[0].item(), t[1].item(), int(t[2].item())
        return ms, tokens_all, launches, h2d, d2h, clocks

    ms, tokens_all, launches, _, _, clocks = timed(prestaged=True)
    value = tokens_all / (ms / 1e3)
    step_split = dict(split)
    e2e = None
    if not args.skip_e2e:
        k2 = args.e2e_steps or (1 if ms / args.steps > 60e3 else args.steps)
        ms2, tokens2, _, h2d, d2h, _ = timed(prestaged=False, steps=k2)
        e2e = {"value": tokens2 / (ms2 / 1e3), "unit": "tokens/s", "ms_per_step": ms2 / k2, "steps": k2,
               "h2d_bytes_per_step": h2d // k2, "d2h_bytes_per_step": d2h // k2}
    lib.check_status()
    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / world) / BASELINE_TOKENS_PER_S_PER_GPU,
            "dtype": "bf16", "data": "synthetic (seeded a+b digit prompts, random-init weights)",
            "tokens_per_second_per_gpu": value / world,
            "config": {"model": args.model, "global_batch": args.prompts_per_gpu * world * args.n,
                       "prompts": args.prompts_per_gpu * world, "samples_per_prompt": args.n,
                       "seq_len": f"prompt {args.prompt_min}-{args.prompt_max} + response <= {args.max_response}",
                       "parallelism": f"dp{world} (replicated bf16 params, sharded fp32 master/Adam), "
                                      f"rollout tp{args.rollout_tp}",
                       "micro_batch": args.micro_batch, "l2": "inputs larger than L2 (15 GB of weights per pass)",
                       "memory_plan": {"kv_arena_borrows_idle_grad_buffer": True,
                                       "adam_moments_in_pinned_host_memory_during_rollout": world == 1,
                                       "activation_checkpointing": True, "activation_offload": bool(args.offload)},
                       "baseline_note": "vs_baseline divides tokens/s/GPU by the reference's only published absolute "
                                        "number (3473.8 tokens/s/GPU, Qwen2.5-0.5B, 1 GPU of unstated type)"},
            "clocks": clocks, "gpu_launches": launches, "impl": "native", "step_split_s": step_split,
        }
        if e2e is not None:
            out["e2e"] = e2e
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
