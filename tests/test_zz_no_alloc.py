"""The allocation-free GRPO advantage entry point, called through its exported C symbol.

Collected last on purpose (file name): if it fails, a run that stops at the first failure has already run every
other test.  The entry point is meant for callers that cannot get device memory at the time of the call — a host
program under a fixed memory budget without PyTorch, or a step that runs while the KV-cache arena and the trainer
own all free HBM — so it keeps its scratch in a fixed device array inside the library.  Checked here: two calls in a
row (the second reuses the scratch the first one dirtied) agree with the regular entry point, and sizes beyond the
built-in scratch are refused."""
import ctypes

import pytest
import torch

from siirl_b200.ops import lib, rl

pytestmark = pytest.mark.gpu


def _call(cdll, rewards, mask, gid, G, eps=1e-6, norm=1):
    B, R = rewards.shape
    adv = torch.empty_like(rewards)
    fn = cdll.sb_grpo_group_adv_noalloc
    fn.restype = ctypes.c_int
    rc = fn(ctypes.c_void_p(rewards.data_ptr()), ctypes.c_void_p(mask.data_ptr()), ctypes.c_void_p(gid.data_ptr()),
            ctypes.c_void_p(adv.data_ptr()), B, R, G, ctypes.c_float(eps), norm,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, adv


def test_noalloc_entry_point_matches_regular_one_twice():
    assert lib.lib_path().exists()
    cdll = ctypes.CDLL(str(lib.lib_path()))
    torch.manual_seed(0)
    for B, R, G in [(48, 64, 13), (200, 33, 50)]:      # second call has other sizes and reuses dirty scratch
        lens = torch.randint(1, R + 1, (B,))
        mask = (torch.arange(R)[None, :] < lens[:, None]).float().cuda()
        rewards = torch.zeros(B, R)
        rewards[torch.arange(B), lens - 1] = torch.rand(B)
        rewards = rewards.cuda()
        gid = torch.randint(0, G, (B,), dtype=torch.int32).cuda()
        rc, got = _call(cdll, rewards, mask, gid, G)    # first call on the device also resolves the scratch address
        assert rc == 0
        # A further call must not take device memory from the driver.  torch's allocator statistics would not see a
        # cudaMalloc made inside the library, so compare the driver's own free-memory figure around a call whose
        # output tensor comes out of torch's cache (same size as the one just freed).
        del got
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc, got = _call(cdll, rewards, mask, gid, G)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert rc == 0
        assert free_after >= free_before, (free_before, free_after)
        want = rl.grpo_group_advantage(rewards, mask, gid, G)
        torch.cuda.synchronize()
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
        rc2, got2 = _call(cdll, rewards, mask, gid, G, norm=0)
        want2 = rl.grpo_group_advantage(rewards, mask, gid, G, norm_by_std=False)
        assert rc2 == 0
        torch.testing.assert_close(got2, want2, rtol=1e-4, atol=1e-5)


def test_noalloc_entry_point_rejects_oversize():
    cdll = ctypes.CDLL(str(lib.lib_path()))
    x = torch.zeros(4, 4, device="cuda")
    gid = torch.zeros(4, dtype=torch.int32, device="cuda")
    rc, _ = _call(cdll, x, x, gid, 16385)
    assert rc == -4
    big = torch.zeros(16385, 1, device="cuda")
    rc, _ = _call(cdll, big, big, torch.zeros(16385, dtype=torch.int32, device="cuda"), 4)
    assert rc == -4
