"""Bounded device-side waits report through the status word and leave the context usable.

One GPU plays both ends: the flag barrier of a two-rank group is launched with two local buffers standing in for the
peers' flag arrays and the second "rank" never arrives, so the wait runs out after its (short) limit.  Nothing faults:
the kernel returns, the host reads the status, and later launches work."""
import ctypes

import pytest
import torch

from siirl_b200.ops import lib

pytestmark = pytest.mark.gpu


def _ptr_array(*tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def test_flag_wait_runs_out_and_the_host_sees_it():
    L = lib.get_lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    status = lib.status_word(dev)
    status.zero_()
    flags0 = torch.zeros(64, dtype=torch.int32, device=dev)     # this rank's flag array
    flags1 = torch.zeros(64, dtype=torch.int32, device=dev)     # the absent peer's flag array
    peers = _ptr_array(flags0, flags1)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    lib.check(L.sb_flag_barrier(peers, 2, 0, 1, lib.ptr(status), ctypes.c_longlong(5), lib.stream()),
              "sb_flag_barrier")
    t1.record()
    torch.cuda.synchronize()
    assert 4.0 < t0.elapsed_time(t1) < 500.0            # waited about the 5 ms limit, not forever
    assert int(flags1[0].item()) == 1                   # the arrival was published before the wait
    with pytest.raises(lib.KernelStatusError) as err:
        lib.check_status(dev)
    assert err.value.code == 4
    # the status word was cleared by the read and the context still runs kernels
    lib.check_status(dev)
    x = torch.randn(256, 256, device=dev, dtype=torch.bfloat16)
    from siirl_b200.ops.dense import gemm
    y = gemm(x, x)
    torch.testing.assert_close(y.float(), (x.float() @ x.float().t()), rtol=2e-2, atol=2e-1)
    # a barrier whose peer did arrive completes without touching the status word
    flags0[1] = 2
    lib.check(L.sb_flag_barrier(peers, 2, 0, 2, lib.ptr(status), ctypes.c_longlong(5), lib.stream()),
              "sb_flag_barrier")
    torch.cuda.synchronize()
    lib.check_status(dev)


def test_gradient_reduction_poisons_the_norm_after_a_timed_out_wait():
    """The fused optimizer step must not apply gradients that a timed-out barrier may have left incomplete: the
    reduce-scatter kernel turns a non-zero status word into an infinite squared norm, which every rank's AdamW
    kernel reads (after the norm all-reduce) as "skip this step"."""
    L = lib.get_lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    status = lib.status_word(dev)
    n = 4096
    grad = torch.randn(n, device=dev)
    out = torch.empty(n, device=dev)
    sumsq = torch.zeros(1, device=dev)
    ll = ctypes.c_longlong
    status.zero_()
    lib.check(L.sb_rs_reduce(_ptr_array(grad), 1, 0, ll(0), ll(n), lib.ptr(out), lib.ptr(sumsq), lib.ptr(status),
                             lib.stream()), "sb_rs_reduce")
    torch.cuda.synchronize()
    torch.testing.assert_close(sumsq[0], grad.double().pow(2).sum().float(), rtol=1e-4, atol=1e-3)
    torch.testing.assert_close(out, grad)
    status.fill_(4)
    sumsq.zero_()
    lib.check(L.sb_rs_reduce(_ptr_array(grad), 1, 0, ll(0), ll(n), lib.ptr(out), lib.ptr(sumsq), lib.ptr(status),
                             lib.stream()), "sb_rs_reduce")
    torch.cuda.synchronize()
    assert torch.isinf(sumsq).all()
    status.zero_()
