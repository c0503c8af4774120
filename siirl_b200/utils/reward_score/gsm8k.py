"""GSM8K scorer: the final answer follows ``####`` (strict) or is the last number in the text (flexible)."""
import re

_STRICT = re.compile(r"#### (\-?[0-9\.\,]+)")
_NUM = re.compile(r"(\-?[0-9\.\,]+)")


def extract_solution(solution_str: str, method: str = "strict"):
    assert method in ("strict", "flexible")
    tail = solution_str[-300:]
    if method == "strict":
        m = _STRICT.findall(tail)
        if not m:
            return None
        return m[-1].replace(",", "").replace("$", "")
    nums = [n for n in _NUM.findall(tail) if n not in ("", ".")]
    return nums[-1].replace(",", "") if nums else None


def compute_score(solution_str: str, ground_truth: str, method: str = "strict", format_score: float = 0.0,
                  score: float = 1.0) -> float:
    ans = extract_solution(solution_str, method)
    if ans is None:
        return 0.0
    return score if ans == str(ground_truth) else format_score
