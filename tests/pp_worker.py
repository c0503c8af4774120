"""Body of the pipeline-schedule check, one process per stage (torchrun env, gloo).

Micro-batches go through a pipeline under the 1F1B order (``PP_VIRTUAL=1``) or the interleaved order with
``PP_VIRTUAL`` model chunks per stage, with asynchronous sends on the direction groups; every stage's accumulated
parameter gradients must equal those of the whole model run on one process."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from siirl_b200.models.config import get_config  # noqa: E402
from siirl_b200.models.decoder import build_model  # noqa: E402
from siirl_b200.ops.attention import SeqInfo  # noqa: E402
from siirl_b200.parallel.pipeline import PipelineContext, schedule_1f1b, schedule_interleaved  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    ranks = list(range(world))
    g, gf, gb = dist.new_group(ranks), dist.new_group(ranks), dist.new_group(ranks)
    wf, wb = dist.new_group(ranks), dist.new_group(ranks)
    V = int(os.environ.get("PP_VIRTUAL", "1"))
    cfg = get_config("tiny", {"num_layers": 2 * world * V - (1 if V > 1 else 0)})   # uneven last chunk when interleaved
    full = build_model(cfg, dtype=torch.float32, device="cpu", seed=5)
    staged = build_model(cfg, dtype=torch.float32, device="cpu", seed=5)
    pc = PipelineContext(g, cfg.num_layers, gf, gb, virtual=V, wrap_fwd_group=wf, wrap_bwd_group=wb)
    assert pc.pipelined
    staged.attach_pipeline_parallel(pc)
    for n, p in staged.named_parameters():
        if not pc.owns_param(n):
            p.requires_grad_(False)
    gen = torch.Generator().manual_seed(7)         # same micro-batches on every stage
    M = 5 if V == 1 else 2 * world + int(os.environ.get("PP_EXTRA", "0"))
    mbs = []
    for _ in range(M):
        lens = [int(x) for x in torch.randint(5, 20, (3,), generator=gen)]
        ids = torch.randint(3, cfg.vocab_size, (sum(lens),), generator=gen)
        labels = torch.randint(3, cfg.vocab_size, (sum(lens),), generator=gen)
        mbs.append((lens, ids, labels))
    # whole model, one process: reference gradients
    for lens, ids, labels in mbs:
        info = SeqInfo(lens)
        lp, _ = full.logprobs(ids, info.positions, info, labels)
        (-lp.mean()).backward()
    if V == 1:
        order = schedule_1f1b(pc.stage, pc.pp, M)
        assert [i for op, i in order if op == "F"] == list(range(M)) and [i for op, i in order if op == "B"] == list(range(M))
        assert max(sum(1 for op, j in order[:k + 1] if op == "F") - sum(1 for op, j in order[:k + 1] if op == "B")
                   for k in range(len(order))) == min(world - rank, M)   # micro-batches in flight on this stage
    order = schedule_interleaved(pc.stage, pc.pp, M, V)
    assert sorted((i, c) for op, i, c in order if op == "F") == [(i, c) for i in range(M) for c in range(V)]
    assert sorted((i, c) for op, i, c in order if op == "B") == [(i, c) for i in range(M) for c in range(V)]
    inflight = {}
    for op, i, c in order:
        lens, ids, labels = mbs[i]
        if op == "F":
            info = SeqInfo(lens)
            hidden, handle = staged.forward_hidden_pp(ids, info.positions, info, chunk=c)
            if pc.chunk_is_last(c):
                lp, _ = staged.token_logprobs(hidden, labels, 1.0, False)
                inflight[i, c] = -lp.mean()
            else:
                inflight[i, c] = handle
        else:
            inflight.pop((i, c)).backward()
    pc.drain()
    worst = 0.0
    pf = dict(full.named_parameters())
    for n, p in staged.named_parameters():
        if not pc.owns_param(n):
            assert p.grad is None and getattr(p, "main_grad", None) is None
            continue
        got = p.grad if p.grad is not None else p.main_grad
        want = pf[n].grad if pf[n].grad is not None else pf[n].main_grad
        worst = max(worst, (got.float() - want.float()).abs().max().item())
    assert worst < 1e-5, worst
    dist.barrier()
    if rank == 0:
        print("PP_1F1B_OK", V, worst)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
