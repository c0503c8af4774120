"""The debug-bounds build of the native library: compiles for sm_100a without a GPU and exports one reader per
translation unit that checks data-dependent indices; on a GPU an out-of-range token id is recorded (unit, site, index,
limit) while the kernel's own clamp keeps the access in range."""
import os
import subprocess
import sys

import pytest


def test_debug_bounds_build_exports_the_readers():
    from siirl_b200 import build_ext
    path = build_ext.build(debug_bounds=True)
    assert path.name == "libsiirl_b200_dbg.so" and path.exists()
    syms = subprocess.run(["nm", "-D", str(path)], capture_output=True, text=True).stdout
    assert "sb_bounds_read_elementwise" in syms and "sb_bounds_read_kv_cache" in syms
    normal = subprocess.run(["nm", "-D", str(build_ext.build())], capture_output=True, text=True).stdout
    assert "sb_bounds_read_" not in normal


@pytest.mark.gpu
def test_out_of_range_token_id_is_recorded_not_dereferenced():
    code = """
import torch
from siirl_b200 import ops
from siirl_b200.ops import lib
table = torch.randn(64, 32, device="cuda").to(torch.bfloat16)
ids = torch.tensor([3, 70, 5], device="cuda")
out = ops.embedding(ids, table)
torch.cuda.synchronize()
assert torch.equal(out[1], table[63])            # clamped by the kernel
v = lib.bounds_violations()
assert v == [("elementwise", 1, 70, 64)], v
assert lib.bounds_violations() == []             # reading clears the record
ok = ops.embedding(torch.tensor([1, 2], device="cuda"), table)
torch.cuda.synchronize()
assert lib.bounds_violations() == []
print("BOUNDS_OK")
"""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, SIIRL_DEBUG_BOUNDS="1", PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0 and "BOUNDS_OK" in out.stdout, out.stdout[-1000:] + out.stderr[-2000:]
