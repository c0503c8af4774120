"""Example user reward function (selected with ``custom_reward_function.path=<this file>``).
Any function with the signature below can be plugged in; it may return a float or a dict with ``"score"``."""
from siirl_b200.utils.reward_score import gsm8k


def compute_score(data_source, solution_str, ground_truth, extra_info=None, **kwargs):
    strict = gsm8k.compute_score(solution_str, ground_truth, method="strict")
    flexible = gsm8k.compute_score(solution_str, ground_truth, method="flexible")
    return {"score": max(strict, 0.1 * flexible), "acc": bool(strict > 0)}
