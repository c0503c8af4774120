"""Exact-match QA scorer (Search-R1 style): answer inside the last ``<answer>...</answer>`` block."""
import re
import string


def normalize_answer(s: str) -> str:
    s = s.lower()
    s = "".join(ch for ch in s if ch not in set(string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return " ".join(s.split())


def extract_solution(solution_str: str):
    m = re.findall(r"<answer>(.*?)</answer>", solution_str, re.DOTALL)
    return m[-1].strip() if m else None


def compute_score(solution_str: str, ground_truth, format_score: float = 0.0, score: float = 1.0) -> float:
    ans = extract_solution(solution_str)
    if ans is None:
        return 0.0
    targets = ground_truth.get("target", ground_truth) if isinstance(ground_truth, dict) else ground_truth
    if isinstance(targets, str):
        targets = [targets]
    return score if any(normalize_answer(ans) == normalize_answer(str(t)) for t in targets) else format_score
