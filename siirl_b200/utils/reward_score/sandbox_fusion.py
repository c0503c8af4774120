"""Remote code sandbox scorer (reference: siirl/utils/reward_score/sandbox_fusion/*): POST the program and each
test's stdin to a Sandbox-Fusion compatible ``run_code`` endpoint, compare stdout.  Concurrency is bounded by a
semaphore like the reference's ``concurrent_semaphore``; connection errors count as failed tests, never raise."""
from __future__ import annotations

import json
import threading
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Dict, Optional

from .prime_code import extract_code


def _call(url: str, code: str, stdin: str, timeout: float, language: str) -> Optional[str]:
    import urllib.request
    body = json.dumps({"code": code, "stdin": stdin, "language": language, "run_timeout": timeout}).encode()
    req = urllib.request.Request(url, data=body, headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=timeout + 5) as r:
            res = json.loads(r.read().decode())
        run = res.get("run_result") or {}
        return run.get("stdout") if res.get("status") == "Success" else None
    except Exception:  # noqa: BLE001
        return None


def compute_score(sandbox_fusion_url: str, concurrent_semaphore: Optional[threading.Semaphore], solution_str: str,
                  ground_truth: Any, continuous: bool = True, timeout: float = 10.0,
                  language: str = "python") -> Dict[str, Any]:
    spec = json.loads(ground_truth) if isinstance(ground_truth, str) else dict(ground_truth)
    code = extract_code(solution_str)
    inputs, outputs = list(spec.get("inputs", [])), list(spec.get("outputs", []))
    sem = concurrent_semaphore or threading.Semaphore(8)

    def one(pair):
        x, w = pair
        with sem:
            out = _call(sandbox_fusion_url, code, x if isinstance(x, str) else "\n".join(map(str, x)), timeout, language)
        want = w if isinstance(w, str) else "\n".join(map(str, w))
        return int(out is not None and out.split() == want.split())

    with ThreadPoolExecutor(max_workers=8) as ex:
        passed = sum(ex.map(one, zip(inputs, outputs)))
    total = max(len(inputs), 1)
    return {"score": passed / total if continuous else float(passed == len(inputs)), "passed": passed,
            "total": len(inputs)}
