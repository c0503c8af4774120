"""Body of the parameter-sharding checks, one process per rank (torchrun env).  ``Z3_DEVICE=cpu`` runs on gloo ranks
(library collectives), ``Z3_DEVICE=cuda`` on NCCL ranks with the peer-memory gather / reduce kernels.

The sharded store (parameters, gradients and optimizer state split over the ranks, layers gathered on demand) must
train exactly like the replicated store: same losses, same gradient norms, same parameters after three optimizer
steps of two micro-batches each, and the same scores from a no-grad pass afterwards."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from siirl_b200.models.config import get_config  # noqa: E402
from siirl_b200.models.decoder import build_model  # noqa: E402
from siirl_b200.ops.attention import SeqInfo  # noqa: E402
from siirl_b200.parallel.flat_params import FlatParamStore  # noqa: E402
from siirl_b200.parallel.sharded_params import ShardedParamStore  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    cuda = os.environ.get("Z3_DEVICE", "cpu") == "cuda"
    comm = None
    if cuda:
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        dist.init_process_group("nccl")
        dev = torch.device("cuda", torch.cuda.current_device())
        from siirl_b200.ops import lib
        from siirl_b200.parallel.symm import SymmComm
        comm = SymmComm.create(dist.group.WORLD)
    else:
        dist.init_process_group("gloo")
        dev = torch.device("cpu")
    dtype = torch.bfloat16 if cuda else torch.float32
    cfg = get_config("tiny-gpu" if cuda else "tiny")
    ma = build_model(cfg, dtype=dtype, device=dev, seed=3, gradient_checkpointing=True)
    mb = build_model(cfg, dtype=dtype, device=dev, seed=3, gradient_checkpointing=True)
    sa = FlatParamStore(ma, group=dist.group.WORLD, comm=comm)
    hybrid = int(os.environ.get("Z3_HYBRID", "0"))
    shard_group, replica_group, hybrid_flat = dist.group.WORLD, None, None
    if hybrid > 1:
        # hybrid sharding: blocks of `hybrid` consecutive ranks shard, the same index across blocks replicates
        assert not cuda
        world = dist.get_world_size()
        for b in range(world // hybrid):
            grp = dist.new_group(list(range(b * hybrid, (b + 1) * hybrid)))
            if b == rank // hybrid:
                shard_group = grp
        for i in range(hybrid):
            grp = dist.new_group(list(range(i, world, hybrid)))
            if i == rank % hybrid:
                replica_group = grp
        mh = build_model(cfg, dtype=dtype, device=dev, seed=3, gradient_checkpointing=True)
        hybrid_flat = (mh, FlatParamStore(mh, group=shard_group, replica_group=replica_group))
    sb = ShardedParamStore(mb, group=shard_group, comm=comm, replica_group=replica_group)
    assert next(mb.layers[0].parameters()).numel() == 0, "layer weights must not stay resident"
    g = torch.Generator().manual_seed(100 + rank)
    tol = 2e-2 if cuda else 1e-5
    for step in range(3):
        sa.zero_grad()
        sb.zero_grad()
        for _mb in range(2):
            lens = [70 + 8 * rank, 130, 40] if cuda else [9, 14, 7]
            ids = torch.randint(3, cfg.vocab_size, (sum(lens),), generator=g).to(dev)
            labels = torch.randint(3, cfg.vocab_size, (sum(lens),), generator=g).to(dev)
            info = SeqInfo(lens, device=dev)
            losses = []
            for m in (ma, mb) + ((hybrid_flat[0],) if hybrid_flat else ()):
                lp, ent = m.logprobs(ids, info.positions, info, labels)
                loss = -(lp.mean()) + 0.01 * ent.mean()
                loss.backward()
                losses.append(loss.item())
            assert abs(losses[0] - losses[1]) < tol * max(1.0, abs(losses[0])), (step, losses)
        na, nb = float(sa.step(1e-3)), float(sb.step(1e-3))
        assert abs(na - nb) < (5e-2 if cuda else 1e-4) * max(1.0, na), (step, na, nb)
        if hybrid_flat:
            nh = float(hybrid_flat[1].step(1e-3))
            hybrid_flat[1].zero_grad()
            assert abs(na - nh) < 1e-4 * max(1.0, na), (step, na, nh)
    if cuda:
        torch.cuda.synchronize()
        lib.check_status()
    # whole weights, regathered for the rollout engine, equal the replicated store's
    sb.materialize_full()
    pa, pb = dict(ma.named_parameters()), dict(mb.named_parameters())
    worst = max((pa[n].data.float() - pb[n].data.float()).abs().max().item() for n in pa)
    # (hybrid: the gradient sum runs in another order, and Adam turns a last-bit difference of a near-zero gradient
    # element into a fraction of the learning rate)
    assert worst < (2e-2 if cuda else (3e-4 if hybrid > 1 else 1e-5)), worst
    sb.release_full()
    assert next(mb.layers[0].parameters()).numel() == 0
    if hybrid_flat:
        ph = dict(hybrid_flat[0].named_parameters())
        assert max((pa[n].data.float() - ph[n].data.float()).abs().max().item() for n in pa) < 3e-4
    with torch.no_grad():       # scoring pass: layers are gathered one ahead in forward order
        lens = [33, 50]
        ids = torch.randint(3, cfg.vocab_size, (sum(lens),), generator=g).to(dev)
        info = SeqInfo(lens, device=dev)
        la, _ = ma.logprobs(ids, info.positions, info, ids)
        lb, _ = mb.logprobs(ids, info.positions, info, ids)
        assert (la - lb).abs().max().item() < (0.15 if cuda else (1e-2 if hybrid > 1 else 1e-5))
    # a frozen sharded model (reference policy): no gradient or optimizer memory
    mc = build_model(cfg, dtype=dtype, device=dev, seed=3)
    for p in mc.parameters():
        p.requires_grad_(False)
    sc = ShardedParamStore(mc, group=shard_group, comm=comm, optimizer_state=False, trainable=False)
    assert sc.grad_slots is None and sc.local.master is None
    md = build_model(cfg, dtype=dtype, device=dev, seed=3)
    with torch.no_grad():
        lc, _ = mc.logprobs(ids, info.positions, info, ids)
        ld, _ = md.logprobs(ids, info.positions, info, ids)
        assert (lc - ld).abs().max().item() < (0.05 if cuda else 1e-5)
    if cuda:
        torch.cuda.synchronize()
        lib.check_status()
    dist.barrier()
    if rank == 0:
        print("ZERO3_OK", worst)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
