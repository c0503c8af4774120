"""Code-generation scorer: run the model's program against test cases in a child process with a time and memory
limit (reference: siirl/utils/reward_score/prime_code/*, which ports the APPS / TACO harness).  Ground truth is a
JSON object ``{"inputs": [...], "outputs": [...]}`` (stdin / stdout pairs) or ``{"fn_name": ..., "inputs": [...],
"outputs": [...]}`` (call a function).  Score = fraction of passed tests (or all-or-nothing with
``continuous=False``)."""
from __future__ import annotations

import json
import os
import re
import subprocess
import sys
import tempfile
from typing import Any, Dict, Tuple

_RUNNER = r'''
import json, sys, resource
resource.setrlimit(resource.RLIMIT_AS, ({mem}, {mem}))
src = open(sys.argv[1]).read()
spec = json.load(open(sys.argv[2]))
ns = {{"__name__": "__solution__"}}
exec(compile(src, "solution.py", "exec"), ns)
fn = ns[spec["fn_name"]]
out = []
for args in spec["inputs"]:
    try:
        out.append(fn(*args) if isinstance(args, list) else fn(args))
    except Exception as e:
        out.append({{"__error__": repr(e)}})
print(json.dumps(out, default=str))
'''


def extract_code(text: str) -> str:
    m = re.findall(r"```(?:python|py)?\n(.*?)```", text, flags=re.S)
    return m[-1] if m else text


def _run(cmd, stdin: str, timeout: float) -> Tuple[int, str]:
    try:
        p = subprocess.run(cmd, input=stdin, capture_output=True, text=True, timeout=timeout,
                           env={"PATH": os.environ.get("PATH", ""), "PYTHONHASHSEED": "0"})
        return p.returncode, p.stdout
    except subprocess.TimeoutExpired:
        return -9, ""


def compute_score(solution_str: str, ground_truth: Any, continuous: bool = True, timeout: float = 5.0,
                  memory_bytes: int = 1 << 30) -> Dict[str, Any]:
    spec = json.loads(ground_truth) if isinstance(ground_truth, str) else dict(ground_truth)
    code = extract_code(solution_str)
    inputs, outputs = list(spec.get("inputs", [])), list(spec.get("outputs", []))
    if not inputs:
        return {"score": 0.0, "passed": 0, "total": 0}
    passed = 0
    with tempfile.TemporaryDirectory() as d:
        src = os.path.join(d, "solution.py")
        with open(src, "w") as f:
            f.write(code)
        if spec.get("fn_name"):
            sp = os.path.join(d, "spec.json")
            with open(sp, "w") as f:
                json.dump({"fn_name": spec["fn_name"], "inputs": inputs}, f)
            rn = os.path.join(d, "runner.py")
            with open(rn, "w") as f:
                f.write(_RUNNER.format(mem=memory_bytes))
            rc, out = _run([sys.executable, rn, src, sp], "", timeout * max(1, len(inputs)))
            try:
                got = json.loads(out.strip().splitlines()[-1]) if rc == 0 else []
            except (ValueError, IndexError):
                got = []
            for g, w in zip(got, outputs):
                w = w[0] if isinstance(w, list) and len(w) == 1 and not isinstance(g, list) else w
                passed += int(json.dumps(g, default=str) == json.dumps(w, default=str))
        else:
            for x, w in zip(inputs, outputs):
                rc, out = _run([sys.executable, src], x if isinstance(x, str) else "\n".join(map(str, x)), timeout)
                want = w if isinstance(w, str) else "\n".join(map(str, w))
                passed += int(rc == 0 and out.split() == want.split())
    total = len(inputs)
    score = passed / total if continuous else float(passed == total)
    return {"score": score, "passed": passed, "total": total}
