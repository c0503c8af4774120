"""Body of the multi-GPU checks; launched by tests/test_gpu_multi.py with one process per GPU (torchrun env)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from siirl_b200.models.config import get_config  # noqa: E402
from siirl_b200.models.decoder import build_model  # noqa: E402
from siirl_b200.ops import lib  # noqa: E402
from siirl_b200.ops.attention import SeqInfo  # noqa: E402
from siirl_b200.parallel.flat_params import FlatParamStore  # noqa: E402
from siirl_b200.parallel.symm import SymmComm  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    dev = torch.device("cuda", torch.cuda.current_device())
    comm = SymmComm.create(dist.group.WORLD)
    comm.barrier()
    comm.barrier()

    # 1. fused reduce-scatter + AdamW + all-gather equals the NCCL path
    cfg = get_config("tiny-gpu")
    stores = []
    for use_comm in (True, False):
        model = build_model(cfg, dtype=torch.bfloat16, device=dev, seed=3)
        store = FlatParamStore(model, group=dist.group.WORLD, comm=comm if use_comm else None)
        stores.append((model, store))
    info = SeqInfo([64 + 16 * rank, 100], device=dev)
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    ids = torch.randint(3, cfg.vocab_size, (info.total,), device=dev, generator=g)
    ids_train = ids
    norms = []
    for step in range(2):
        for model, store in stores:
            store.zero_grad()
            lp, _ = model.logprobs(ids, info.positions, info, torch.roll(ids, -1), with_entropy=False)
            (-lp.mean()).backward()
            norms.append(store.step(lr=1e-3, max_grad_norm=1.0))
    torch.cuda.synchronize()
    lib.check_status()
    a, b = stores[0][1].flat_param.float(), stores[1][1].flat_param.float()
    err = (a - b).abs().max().item()
    assert err < 1e-2, f"fused vs NCCL parameters differ by {err}"
    assert abs(norms[-2].item() - norms[-1].item()) < 1e-2 * max(1.0, norms[-1].item())
    # replicas agree across ranks
    chk = stores[0][1].flat_param.float().sum().reshape(1).clone()
    parts = [torch.zeros_like(chk) for _ in range(world)]
    dist.all_gather(parts, chk)
    assert all(torch.equal(parts[0], p) for p in parts), "replicas diverged"

    # 2. row all-to-all-v through peer memory
    row = 32
    counts = [[(s + d) % 3 + 1 for d in range(world)] for s in range(world)]
    send = torch.cat([torch.full((counts[rank][d], row), float(rank * 100 + d), device=dev) for d in range(world)])
    staging = comm.alloc(64 * row, torch.float32)
    got = comm.alltoallv_rows(send, counts[rank], staging, counts)
    want = torch.cat([torch.full((counts[s][rank], row), float(s * 100 + rank), device=dev) for s in range(world)])
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    lib.check_status()

    # 3. Data Coordinator redistribution through peer memory: every rank publishes samples of different lengths,
    #    a collective get re-partitions them (balanced) and each rank receives its share bit-exactly
    from siirl_b200.data_coordinator import DataCoordinator
    from siirl_b200.data_coordinator.sample import Sample, SampleInfo
    dc = DataCoordinator(1, 0, world, group=dist.group.WORLD, comm=comm)
    per_rank = 6
    infos, samples = [], []
    for i in range(per_rank):
        n = 5 + 3 * i + rank
        ids = torch.arange(n, device=dev) + 1000 * rank + 100 * i
        samples.append(Sample({"input_ids": ids, "score": torch.tensor([float(rank * 10 + i)], device=dev)},
                              {"tag": f"r{rank}s{i}"}, {}))
        infos.append(SampleInfo(sum_tokens=n, dict_info={"key": "k"}))
    dc.put_batch(infos, samples, caller_node_id="k")
    got_s = dc.get_batch_collective(per_rank, rank, world, lambda info: info.dict_info.get("key") == "k")
    assert len(got_s) == per_rank
    seen = []
    for smp in got_s:
        tag = smp.non_tensors["tag"]
        r, i = int(tag[1]), int(tag[3])
        n = 5 + 3 * i + r
        assert smp.tensors["input_ids"].is_cuda
        assert torch.equal(smp.tensors["input_ids"].cpu(), torch.arange(n) + 1000 * r + 100 * i), tag
        assert float(smp.tensors["score"]) == float(r * 10 + i)
        seen.append(tag)
    all_seen = [None] * world
    dist.all_gather_object(all_seen, seen)
    flat = sorted(t for part in all_seen for t in part)
    assert flat == sorted(f"r{r}s{i}" for r in range(world) for i in range(per_rank)), "a sample was lost or duplicated"
    torch.cuda.synchronize()
    lib.check_status()

    # 4. adversarial arrival order: every rank sleeps a different, random time on the host before each flag barrier and
    #    before each fused optimizer step (up to 150 ms, far above a kernel's duration but below the bounded waits).
    #    Epoch-tagged flags must never let a late rank pass on a stale flag: after every barrier each rank reads what
    #    its left neighbour wrote into symmetric memory just before arriving.
    import random
    import time
    rng = random.Random(1000 + rank)
    box = comm.alloc(16, torch.int64)
    peers = comm.peers_of(box)
    left = (rank - 1) % world
    for it in range(12):
        time.sleep(rng.random() * 0.15)
        box.fill_(1000 * it + rank)
        torch.cuda.synchronize()
        comm.barrier()
        seen_left = torch.empty(16, dtype=torch.int64, device=dev)
        lib.check(lib.get_lib().sb_segment_pull(peers.ptr_array, world, lib.ptr(torch.tensor(
            [[0, 0, 128, left]], dtype=torch.int64, device=dev)), 1, lib.ptr(seen_left), lib.stream()),
            "sb_segment_pull")
        torch.cuda.synchronize()
        assert int(seen_left[0]) == 1000 * it + left, (it, int(seen_left[0]))
        comm.barrier()                      # nobody overwrites its box before every reader is done
    model, store = stores[0]
    ref_model, ref_store = stores[1]
    for it in range(4):
        for m_, st_ in ((model, store), (ref_model, ref_store)):
            st_.zero_grad()
            lp, _ = m_.logprobs(ids_train, info.positions, info, torch.roll(ids_train, -1), with_entropy=False)
            (-lp.mean()).backward()
        time.sleep(rng.random() * 0.15)
        n1 = store.step(lr=1e-3, max_grad_norm=1.0)
        n2 = ref_store.step(lr=1e-3, max_grad_norm=1.0)
        assert abs(n1.item() - n2.item()) < 1e-2 * max(1.0, n2.item()), (it, n1.item(), n2.item())
    torch.cuda.synchronize()
    lib.check_status()
    err = (store.flat_param.float() - ref_store.flat_param.float()).abs().max().item()
    assert err < 2e-2, f"skewed arrival: fused vs NCCL parameters differ by {err}"
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
