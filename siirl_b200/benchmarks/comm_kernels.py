"""Benchmarks of the kernels fused with a collective, against the same op done with library collectives.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node=N --master-addr 127.0.0.1 --master-port 29577 \
        -m siirl_b200.benchmarks.comm_kernels [--case optimizer|gemm_ar|all] [--numel 1e9]

One JSON line per case from rank 0.  Times are CUDA-event times on the launching stream after 3 warm-up iterations,
median of the timed iterations, MAX over ranks.  Rooflines: a fused kernel's target time is the slower of
FLOPs / measured cuBLAS bf16 throughput and bytes crossing NVLink / 770 GB/s (measured peer-copy bandwidth per
direction per GPU on this pool)."""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from .kernels import peaks

NVLINK_GBS = 770.0


def timeit(fn, iters=10, warm=3) -> float:
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def emit(**kw):
    if dist.get_rank() == 0:
        print(json.dumps(kw), flush=True)


def bench_optimizer(comm, numel: int):
    from ..parallel.flat_params import FlatParamStore
    world = dist.get_world_size()

    class _M(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.p = torch.nn.Parameter(torch.zeros(numel, device="cuda", dtype=torch.bfloat16))

    res = {}
    for name, c in (("fused_peer_memory", comm), ("nccl", None)):
        store = FlatParamStore(_M(), group=dist.group.WORLD, comm=c)
        store.flat_grad.normal_()
        res[name] = timeit(lambda: store.step(1e-4), iters=5)
        del store
        torch.cuda.empty_cache()
    shard = numel / world
    link_bytes = (world - 1) * shard * 4 + (world - 1) * shard * 2      # pulled fp32 grads + pushed bf16 params
    hbm_bytes = numel * 4 / world * world + shard * (4 * 3 * 2 + 4) + numel * 2
    target = max(link_bytes / NVLINK_GBS / 1e6, hbm_bytes / peaks()["hbm_gbs"] / 1e6)
    emit(case="reduce_scatter+adamw+all_gather", numel=numel, world=world, fused_ms=round(res["fused_peer_memory"], 3),
         nccl_ms=round(res["nccl"], 3), speedup=round(res["nccl"] / res["fused_peer_memory"], 3),
         roofline_ms=round(target, 3), frac_of_roofline=round(target / res["fused_peer_memory"], 3))


def bench_gemm_ar(comm):
    from .. import ops
    from ..parallel.tensor_parallel import TPContext
    world = dist.get_world_size()
    H = 3584
    ctx = TPContext(dist.group.WORLD, comm, max_rows=8192, max_cols=H, max_tiles=64 * 28 + 8,
                    fused_max_rows=1 << 30)     # measure the fused kernel at every size
    pk = peaks()
    for M, K, what in ((64, 18944, "decode down_proj"), (64, 3584, "decode o_proj"), (128, 18944, "decode down_proj"),
                       (256, 18944, "decode down_proj"), (512, 18944, "decode down_proj"), (512, 3584, "decode o_proj"),
                       (4096, 18944, "prefill down_proj"), (8192, 3584, "prefill o_proj")):
        ks = K // world // 64 * 64
        x = torch.randn(M, ks, device="cuda", dtype=torch.bfloat16)
        w = (0.02 * torch.randn(H, ks, device="cuda")).to(torch.bfloat16)
        fused = timeit(lambda: ctx.row_parallel_linear(x, w))

        def lib_path():
            y = ops.linear(x, w)
            dist.all_reduce(y)
            return y

        nccl = timeit(lib_path)
        flops = 2.0 * M * H * ks
        link = (world - 1) / world * M * H * (4 + 2)
        hbm = H * ks * 2
        target = max(flops / pk["tflops"] / 1e9, link / NVLINK_GBS / 1e6, hbm / pk["hbm_gbs"] / 1e6)
        emit(case="gemm+all_reduce", shape=what, protocol="push (one shot)" if M <= ctx.one_shot_rows else "owner pull",
             M=M, N=H, K_per_rank=ks, world=world, fused_ms=round(fused, 4),
             gemm_plus_nccl_ms=round(nccl, 4), speedup=round(nccl / fused, 3), roofline_ms=round(target, 4),
             frac_of_roofline=round(target / fused, 3))


def bench_ag_gemm(comm):
    from .. import ops
    from ..parallel.ag_gemm import AgLinear
    world = dist.get_world_size()
    pk = peaks()
    for M, N, K, what in ((8192, 18944 * 2 // 256 // world * 256 * world, 3584, "gate_up (weights sharded by rows)"),
                          (8192, 3584 // (256 * world) * 256 * world, 18944, "down_proj (weights sharded by rows)")):
        ag = AgLinear(dist.group.WORLD, comm, N, K)
        ag.load_shard((0.02 * torch.randn(ag.rows, K, device="cuda")).to(torch.bfloat16))
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        fused = timeit(lambda: ag(x))
        full = torch.empty(N * K, device="cuda", dtype=torch.bfloat16)

        def lib_path():
            dist.all_gather_into_tensor(full, ag.shard.reshape(-1))
            return ops.linear(x, full.view(N, K))

        nccl = timeit(lib_path)
        flops = 2.0 * M * N * K
        link = (world - 1) / world * N * K * 2
        target = max(flops / pk["tflops"] / 1e9, link / NVLINK_GBS / 1e6)
        emit(case="all_gather+gemm", shape=what, M=M, N=N, K=K, world=world, fused_ms=round(fused, 4),
             nccl_all_gather_plus_gemm_ms=round(nccl, 4), speedup=round(nccl / fused, 3),
             roofline_ms=round(target, 4), frac_of_roofline=round(target / fused, 3))
        del ag, full
        torch.cuda.empty_cache()


def bench_moe_ep(comm):
    """Expert-parallel dispatch + combine of one MoE layer (Qwen3-30B-A3B shape) by peer pulls, against the same token
    exchange done with NCCL all_to_all_single plus index_select / index_add permutation kernels."""
    from ..ops import moe as M
    world, rank = dist.get_world_size(), dist.get_rank()
    T, H, E, k = 8192, 2048, 128, 8
    ep = M.ExpertParallel(dist.group.WORLD, comm, max_tokens=T, hidden=H, max_slots=world * T * k + (E // world + 1) * 128)
    x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
    idx = torch.stack([torch.randperm(E, device="cuda")[:k] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, k, device="cuda")
    all_idx = ep.all_gather(idx)
    lay = M.build_layout(all_idx, E, world, rank)
    pr, ps = lay.my_pairs()

    def fused():
        xs = ep.gather_rows(x, lay.slot_src_rank, lay.slot_src_row, None)
        return ep.combine(xs, pr, ps, w, T, k)          # (the expert GEMMs would sit in between)

    # library path: sort pairs by destination rank, exchange counts (precomputed), all_to_all rows both ways
    dest = (idx.long() // (E // world)).reshape(-1)
    order = torch.argsort(dest, stable=True)
    send_counts = torch.bincount(dest, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts)
    sc, rc = send_counts.tolist(), recv_counts.tolist()

    def library():
        rows = x.index_select(0, order // k)
        recv = torch.empty(sum(rc), H, device="cuda", dtype=torch.bfloat16)
        dist.all_to_all_single(recv, rows, rc, sc)
        back = torch.empty_like(rows)
        dist.all_to_all_single(back, recv, sc, rc)
        out = torch.zeros(T, H, device="cuda", dtype=torch.float32)
        out.index_add_(0, order // k, back.float() * w.reshape(-1)[order][:, None])
        return out.to(torch.bfloat16)

    t_f, t_l = timeit(fused, iters=5), timeit(library, iters=5)
    link = 2.0 * (world - 1) / world * T * k * H * 2
    emit(case="moe dispatch+combine", T=T, top_k=k, H=H, world=world, fused_ms=round(t_f, 4),
         nccl_all_to_all_ms=round(t_l, 4), speedup=round(t_l / t_f, 3),
         roofline_ms=round(link / NVLINK_GBS / 1e6, 4), frac_of_roofline=round(link / NVLINK_GBS / 1e6 / t_f, 3))


def bench_ulysses(comm):
    """Sequence <-> head layout switch of Ulysses SP (Qwen2.5-7B qkv width) by one strided pull kernel, against
    NCCL all_to_all_single with the pack / unpack copies the reference does around it."""
    from ..parallel.ulysses import UlyssesSP
    world = dist.get_world_size()
    hq, hkv, D = 28 // world * world, 4 // world * world or world, 128
    Tl = 32768 // world
    W = (hq + 2 * hkv) * D
    parts = [(0, hq * D), (hq * D, hkv * D), ((hq + hkv) * D, hkv * D)]
    sp = UlyssesSP(dist.group.WORLD, comm, max_elems=Tl * W)
    x = torch.randn(Tl, W, device="cuda", dtype=torch.bfloat16)

    def fused():
        return sp.heads_to_seq(sp.seq_to_heads(x, parts), parts)

    def library():
        y = x
        for _ in range(2):      # there and back: pack by destination, exchange, unpack
            packed = torch.cat([torch.cat([y[:, c0 + r * (w // world): c0 + (r + 1) * (w // world)] for c0, w in parts], 1)
                                for r in range(world)], 0).contiguous()
            out = torch.empty_like(packed)
            dist.all_to_all_single(out, packed)
            y = out.reshape(world, Tl, W // world).permute(1, 0, 2).reshape(Tl, W).contiguous()
        return y

    t_f, t_l = timeit(fused), timeit(library)
    link = 2.0 * (world - 1) / world * Tl * W * 2
    emit(case="ulysses seq<->head switch (there and back)", tokens_per_rank=Tl, width=W, world=world,
         fused_ms=round(t_f, 4), nccl_all_to_all_ms=round(t_l, 4), speedup=round(t_l / t_f, 3),
         roofline_ms=round(link / NVLINK_GBS / 1e6, 4), frac_of_roofline=round(link / NVLINK_GBS / 1e6 / t_f, 3))


def bench_samples(comm):
    """Data Coordinator redistribution: 2048 samples of 300-5000 tokens re-partitioned over the ranks, peer-memory
    path against the object-collective path."""
    import random

    from ..data_coordinator import DataCoordinator
    from ..data_coordinator.sample import Sample, SampleInfo
    world, rank = dist.get_world_size(), dist.get_rank()
    per = 2048 // world
    rng = random.Random(rank)
    res = {}
    for name, c in (("peer_memory", comm), ("object_collectives", None)):
        ts = []
        for it in range(4):
            dc = DataCoordinator(1, 0, world, group=dist.group.WORLD, comm=c)
            infos, samples = [], []
            for i in range(per):
                n = rng.randint(300, 5000)
                samples.append(Sample({"input_ids": torch.randint(0, 1000, (n,), device="cuda"),
                                       "logp": torch.randn(n, device="cuda")}, {"i": i}, {}))
                infos.append(SampleInfo(sum_tokens=n, dict_info={"key": "k"}))
            dc.put_batch(infos, samples, caller_node_id="k")
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            got = dc.get_batch_collective(per, rank, world, lambda info: info.dict_info.get("key") == "k")
            e1.record()
            torch.cuda.synchronize()
            assert len(got) == per
            if it:
                ts.append(e0.elapsed_time(e1))
        t = torch.tensor([sorted(ts)[len(ts) // 2]], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res[name] = float(t.item())
    emit(case="sample redistribution (2048 samples, 300-5000 tokens)", world=world,
         fused_ms=round(res["peer_memory"], 3), object_collectives_ms=round(res["object_collectives"], 3),
         speedup=round(res["object_collectives"] / res["peer_memory"], 3))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all", choices=["all", "optimizer", "gemm_ar", "ag_gemm", "moe_ep", "ulysses",
                                                     "samples"])
    ap.add_argument("--numel", type=float, default=1e9)
    a = ap.parse_args()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl")
    from ..ops import lib
    from ..parallel.symm import SymmComm
    comm = SymmComm.create(dist.group.WORLD)
    emit(peaks=peaks(), world=dist.get_world_size(), nvlink_gbs_per_direction=NVLINK_GBS)
    if a.case in ("all", "gemm_ar"):
        bench_gemm_ar(comm)
    if a.case in ("all", "ag_gemm"):
        bench_ag_gemm(comm)
    if a.case in ("all", "moe_ep"):
        bench_moe_ep(comm)
    if a.case in ("all", "ulysses"):
        bench_ulysses(comm)
    if a.case in ("all", "samples"):
        bench_samples(comm)
    if a.case in ("all", "optimizer"):
        n = int(a.numel) // (8 * dist.get_world_size()) * (8 * dist.get_world_size())
        bench_optimizer(comm, n)
    torch.cuda.synchronize()
    lib.check_status()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
