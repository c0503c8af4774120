"""One-GPU run of the one-sided collective kernels: the buffers of W emulated ranks live on ONE device and the kernels
read / write them through the same pointer tables they get from the peer-memory communicator.

This is what a profiler can capture on this pool (it wraps single-GPU commands only): the kernels' own memory
behaviour -- bytes moved per launch against the measured copy bandwidth -- without the NVLink hop.  Only kernels that
never wait on another rank are run here (reduce-scatter pull + AdamW / all-gather push, segment pull); the kernels
that spin on peers' flags are measured across GPUs by ``benchmarks/comm_kernels.py``.

    python -m siirl_b200.benchmarks.comm_loopback [--world 2] [--numel 2.5e8] [--small]
"""
from __future__ import annotations

import argparse
import ctypes
import json

import numpy as np
import torch

from ..ops import lib as _lib
from .kernels import peaks as load_peaks
from .kernels import timeit


def ptr_table(tensors):
    """Host pointer table, the form the communicator hands to the launchers."""
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--world", type=int, default=2)
    ap.add_argument("--numel", type=float, default=2.5e8, help="parameters (whole model) of the optimizer case")
    ap.add_argument("--small", action="store_true", help="a few hundred MB on the device: profiler capture size")
    a = ap.parse_args()
    dev = torch.device("cuda")
    L = _lib.get_lib()
    peaks = load_peaks()
    print(json.dumps({"peaks": peaks, "device": torch.cuda.get_device_name(0)}))
    W = a.world
    n = int(6.4e7 if a.small else a.numel) // (256 * W) * (256 * W)
    shard = n // W
    ll, f = ctypes.c_longlong, ctypes.c_float
    grads = [torch.randn(n, device=dev) for _ in range(W)]                       # fp32 gradient buffers of the W ranks
    params = [torch.zeros(n, dtype=torch.bfloat16, device=dev) for _ in range(W)]
    gt, pt = ptr_table(grads), ptr_table(params)
    out = torch.empty(shard, device=dev)
    sumsq, norm = torch.zeros(1, device=dev), torch.zeros(1, device=dev)
    master, m, v = torch.randn(shard, device=dev), torch.zeros(shard, device=dev), torch.zeros(shard, device=dev)
    status = _lib.status_word(dev)

    def rs():
        sumsq.zero_()
        _lib.check(L.sb_rs_reduce(gt, W, 0, ll(0), ll(shard), _lib.ptr(out), _lib.ptr(sumsq),
                                  _lib.ptr(status), _lib.stream()), "sb_rs_reduce")

    def ag():
        _lib.check(L.sb_adamw_allgather(_lib.ptr(master), _lib.ptr(m), _lib.ptr(v), _lib.ptr(out), pt, W,
                                        _lib.ptr(sumsq), _lib.ptr(norm), ll(0), ll(shard), f(1e-5), f(0.9), f(0.999),
                                        f(1e-8), f(0.01), 1, f(1.0), f(1.0 / W), _lib.stream()), "sb_adamw_allgather")
    rs()
    want = sum(g[:shard].double() for g in grads)
    assert torch.allclose(out.double(), want, atol=1e-4), "rs_reduce loopback numerics"
    ms = timeit(rs)
    moved = shard * 4 * W + shard * 4
    print(json.dumps({"kernel": "rs_reduce (pull W fp32 shards, sum, write shard, squared norm)", "world": W,
                      "shard_elems": shard, "ms": round(ms, 4), "gbs": round(moved / ms / 1e6, 1),
                      "frac_of_measured_copy_bw": round(moved / ms / 1e6 / peaks["hbm_gbs"], 3)}))
    ms = timeit(ag)
    moved = shard * (4 * 3 * 2 + 4) + shard * 2 * W
    print(json.dumps({"kernel": "adamw_allgather (update shard, push bf16 to W replicas)", "world": W,
                      "shard_elems": shard, "ms": round(ms, 4), "gbs": round(moved / ms / 1e6, 1),
                      "frac_of_measured_copy_bw": round(moved / ms / 1e6 / peaks["hbm_gbs"], 3)}))
    # segment pull: a layer of the parameter-sharded store (W pieces of a 233 M-element layer, bf16) into a gather slot
    unit = int(2.33e8 if not a.small else 3.2e7) // (256 * W) * (256 * W)
    piece = unit // W
    pieces = [torch.randn(piece, device=dev).to(torch.bfloat16) for _ in range(W)]
    bt = ptr_table(pieces)
    slot = torch.empty(unit, dtype=torch.bfloat16, device=dev)
    tab = np.zeros((W, 4), dtype=np.int64)
    for q in range(W):
        tab[q] = (0, q * piece * 2, piece * 2, q)
    segs = torch.from_numpy(tab).to(dev)

    def pull():
        _lib.check(L.sb_segment_pull(bt, W, _lib.ptr(segs), W, _lib.ptr(slot), _lib.stream()),
                   "sb_segment_pull")
    pull()
    assert torch.equal(slot[piece:2 * piece], pieces[1]), "segment_pull loopback numerics"
    ms = timeit(pull)
    moved = unit * 2 * 2
    print(json.dumps({"kernel": "segment_pull (gather one sharded layer into a slot)", "world": W, "bytes": unit * 2,
                      "ms": round(ms, 4), "gbs": round(moved / ms / 1e6, 1),
                      "frac_of_measured_copy_bw": round(moved / ms / 1e6 / peaks["hbm_gbs"], 3)}))
    torch.cuda.synchronize()
    _lib.check_status()


if __name__ == "__main__":
    main()
