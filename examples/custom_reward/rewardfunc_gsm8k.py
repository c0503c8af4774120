"""A user-supplied reward for GSM8K, in the batched form (``reward_model.reward_manager=batch``).

The function named by ``custom_reward_function.path`` / ``.name`` receives the whole batch as lists and returns one
score (or one dict with a ``"score"`` entry) per sample.  The per-sample form
``compute_score(data_source, solution_str, ground_truth, extra_info=None)`` works with the other reward managers."""
import re

_STRICT = re.compile(r"#### (-?[0-9.,]+)")
_NUMBER = re.compile(r"-?[0-9][0-9.,]*")


def final_answer(text: str, method: str = "strict"):
    if method == "strict":                       # the model must also follow the "#### <number>" format
        m = _STRICT.search(text)
        return m.group(1).replace(",", "").rstrip(".") if m else None
    numbers = [n.replace(",", "").rstrip(".") for n in _NUMBER.findall(text)]
    numbers = [n for n in numbers if n]
    return numbers[-1] if numbers else None


def compute_score(data_sources, solution_strs, ground_truths, extra_infos, method="strict", format_score=0.0,
                  score=1.0, **kwargs):
    out = []
    for text, truth in zip(solution_strs, ground_truths):
        ans = final_answer(text, method)
        if ans is None:
            out.append(0.0)
        else:
            out.append(score if ans == str(truth).replace(",", "") else format_score)
    return out
