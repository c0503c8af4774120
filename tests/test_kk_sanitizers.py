"""The host-only C++ of the native library (Karmarkar-Karp partitioning) under AddressSanitizer and
UndefinedBehaviorSanitizer: built as its own small program with ``g++ -fsanitize=address,undefined`` and run on random
workloads (also the degenerate ones), its output compared with the Python statement of the same algorithm."""
import os
import random
import shutil
import subprocess

import pytest

from siirl_b200.utils.model_utils.seqlen_balancing import _kk_python

DRIVER = r"""
#include <cstdio>
#include <vector>
extern "C" int sb_kk_partition(const long long* workloads, int n, int k, int equal_size, int* out_part);
int main() {
  int cases;
  if (scanf("%d", &cases) != 1) return 2;
  for (int c = 0; c < cases; ++c) {
    int n, k, eq;
    if (scanf("%d %d %d", &n, &k, &eq) != 3) return 2;
    std::vector<long long> w(n);
    for (int i = 0; i < n; ++i) if (scanf("%lld", &w[i]) != 1) return 2;
    std::vector<int> part(n > 0 ? n : 1, -1);
    int rc = sb_kk_partition(w.data(), n, k, eq, part.data());
    printf("%d", rc);
    for (int i = 0; i < n; ++i) printf(" %d", part[i]);
    printf("\n");
  }
  return 0;
}
"""


@pytest.mark.skipif(shutil.which("g++") is None, reason="no host compiler")
def test_kk_partition_under_asan_and_ubsan(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.path.join(root, "siirl_b200", "csrc", "host", "kk_partition.cpp")
    drv = tmp_path / "driver.cpp"
    drv.write_text(DRIVER)
    exe = tmp_path / "kk_san"
    build = subprocess.run(["g++", "-std=c++17", "-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=all",
                            "-fno-omit-frame-pointer", src, str(drv), "-o", str(exe)], capture_output=True, text=True)
    if build.returncode != 0 and "sanitize" in build.stderr:
        pytest.skip("this toolchain has no sanitizer runtime: " + build.stderr[-200:])
    assert build.returncode == 0, build.stderr[-2000:]
    rng = random.Random(0)
    cases = [(0, 2, 0, []), (1, 1, 0, [5]), (3, 5, 0, [1, 2, 3]), (4, 2, 1, [7, 7, 7, 7]), (5, 2, 1, [1, 2, 3, 4, 5]),
             (6, 3, 1, [0, 0, 0, 0, 0, 0])]
    for _ in range(60):
        k = rng.randint(1, 8)
        eq = rng.random() < 0.5
        n = k * rng.randint(1, 12) if eq else rng.randint(1, 90)
        cases.append((n, k, int(eq), [rng.randint(1, 4096) ** 2 for _ in range(n)]))
    text = [str(len(cases))] + [f"{n} {k} {eq} " + " ".join(map(str, w)) for n, k, eq, w in cases]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    run = subprocess.run([str(exe)], input="\n".join(text) + "\n", capture_output=True, text=True, env=env, timeout=120)
    assert run.returncode == 0, run.stderr[-3000:]
    assert "runtime error" not in run.stderr and "AddressSanitizer" not in run.stderr, run.stderr[-3000:]
    lines = run.stdout.strip().splitlines()
    assert len(lines) == len(cases)
    for (n, k, eq, w), line in zip(cases, lines):
        vals = list(map(int, line.split()))
        if eq and n % k:
            assert vals[0] == -3
            continue
        assert vals[0] == 0, (n, k, eq, vals[0])
        part = vals[1:]
        assert len(part) == n and all(0 <= p < k for p in part)
        sums = [sum(w[i] for i in range(n) if part[i] == j) for j in range(k)]
        want = _kk_python(w, k, bool(eq)) if n else [[] for _ in range(k)]
        assert sorted(sums) == sorted(sum(w[i] for i in s) for s in want), (n, k, eq)
        if eq:
            assert all(part.count(j) == n // k for j in range(k))
