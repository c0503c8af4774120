"""MATH-style scorers: last ``\\boxed{...}`` answer, normalised string equality (fractions, units, spacing).
Behaviour of siirl/utils/reward_score/math.py, math_dapo.py and geo3k.py in the reference."""
import re
from typing import Optional


def last_boxed_only_string(s: str) -> Optional[str]:
    idx = s.rfind("\\boxed")
    if idx < 0:
        idx = s.rfind("\\fbox")
        if idx < 0:
            return None
    i, depth, end = idx, 0, None
    while i < len(s):
        if s[i] == "{":
            depth += 1
        elif s[i] == "}":
            depth -= 1
            if depth == 0:
                end = i
                break
        i += 1
    return None if end is None else s[idx:end + 1]


def remove_boxed(s: str) -> str:
    if s.startswith("\\boxed "):
        return s[len("\\boxed "):]
    left = "\\boxed{"
    if s.startswith(left) and s.endswith("}"):
        return s[len(left):-1]
    return s


def _fix_fracs(s: str) -> str:
    return re.sub(r"\\frac(\d)(\d)", r"\\frac{\1}{\2}", s)


def strip_string(s: str) -> str:
    s = str(s).replace("\n", "").replace("\\!", "").replace("\\\\", "\\")
    s = s.replace("tfrac", "frac").replace("dfrac", "frac").replace("\\left", "").replace("\\right", "")
    s = s.replace("^{\\circ}", "").replace("^\\circ", "").replace("\\$", "").replace("$", "")
    s = re.sub(r"\\text\{\s*[a-zA-Z ]+\}$", "", s)
    s = s.replace("\\%", "").replace("%", "")
    s = s.replace(" .", " 0.").replace("{.", "{0.")
    if s.startswith("."):
        s = "0" + s
    if len(s.split("=")) == 2 and len(s.split("=")[0]) <= 2:
        s = s.split("=")[1]
    s = s.replace(" ", "")
    s = _fix_fracs(s)
    if s == "0.5":
        s = "\\frac{1}{2}"
    m = re.fullmatch(r"(-?\d+)/(\d+)", s)
    if m:
        s = f"\\frac{{{m.group(1)}}}{{{m.group(2)}}}"
    return s


def is_equiv(a: Optional[str], b: Optional[str]) -> bool:
    if a is None or b is None:
        return a is None and b is None
    try:
        return strip_string(a) == strip_string(b)
    except Exception:  # noqa: BLE001
        return a == b


def compute_score(solution_str: str, ground_truth: str) -> float:
    boxed = last_boxed_only_string(solution_str)
    if boxed is None:
        return 0.0
    return 1.0 if is_equiv(remove_boxed(boxed), ground_truth) else 0.0


def compute_score_dapo(solution_str: str, ground_truth: str) -> dict:
    """DAPO convention: answer after ``Answer:`` (last 300 chars) or boxed; +1 / -1 reward, ``acc`` flag."""
    tail = solution_str[-300:]
    m = re.findall(r"(?i)Answer\s*:\s*([^\n]+)", tail)
    pred = m[-1].strip() if m else None
    if pred is None:
        boxed = last_boxed_only_string(tail)
        pred = remove_boxed(boxed) if boxed else None
    correct = pred is not None and is_equiv(pred, str(ground_truth))
    return {"score": 1.0 if correct else -1.0, "acc": bool(correct), "pred": pred}


def compute_score_geo3k(solution_str: str, ground_truth: str) -> float:
    fmt = 1.0 if re.fullmatch(r".*<think>.*</think>.*\\boxed\{.*\}.*", solution_str, re.DOTALL) else 0.0
    acc = compute_score(solution_str, ground_truth)
    return 0.9 * acc + 0.1 * fmt
