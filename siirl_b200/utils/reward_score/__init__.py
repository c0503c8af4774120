"""Rule-based scorers and the ``data_source`` dispatch.

Signature kept from the reference (siirl/utils/reward_score/__init__.py:19-98):
``compute_score(data_source, solution_str, ground_truth, extra_info=None) -> float | dict`` (a dict must hold
``"score"``).  Scorers: gsm8k, math (boxed answers, normalised string match), math_dapo, geo3k, math_verify / prime_math
(numeric and element-wise equivalence), search-R1 style exact match, plus the synthetic tasks of the benchmark configurations (arith, parity, bernoulli, length)."""
from __future__ import annotations

import random
import re
from typing import Any, Dict, Optional, Union

from . import gsm8k, math as math_score, qa_em


def _arith(solution_str: str, ground_truth: str) -> float:
    digits = re.findall(r"\d+", solution_str)
    return 1.0 if digits and digits[0] == str(ground_truth) else 0.0


def _bernoulli(extra_info: Optional[Dict[str, Any]]) -> float:
    seed = int((extra_info or {}).get("seed", 0))
    return 1.0 if random.Random(seed).random() < 0.5 else 0.0


def _length_score(solution_str: str, extra_info: Optional[Dict[str, Any]]) -> float:
    seed = int((extra_info or {}).get("seed", 0))
    return random.Random(seed).random()


def default_compute_score(data_source: str, solution_str: str, ground_truth: Any,
                          extra_info: Optional[Dict[str, Any]] = None, **kwargs) -> Union[float, Dict[str, Any]]:
    ds = str(data_source)
    if ds in ("openai/gsm8k", "gsm8k"):
        return gsm8k.compute_score(solution_str, ground_truth, **{k: v for k, v in kwargs.items()
                                                                   if k in ("method", "format_score", "score")})
    if ds in ("lighteval/MATH", "DigitalLearningGmbH/MATH-lighteval", "math", "HuggingFaceH4/MATH-500"):
        return math_score.compute_score(solution_str, ground_truth)
    if ds in ("math_dapo", "aime") or ds.startswith("aime"):
        return math_score.compute_score_dapo(solution_str, ground_truth)
    if ds in ("hiyouga/geometry3k", "geo3k", "mm_eureka"):
        return math_score.compute_score_geo3k(solution_str, ground_truth)
    if ds in ("searchR1_nq", "searchR1_triviaqa", "searchR1_popqa", "searchR1_hotpotqa", "searchR1_2wikimultihopqa",
              "searchR1_musique", "searchR1_bamboogle", "qa_em"):
        return qa_em.compute_score(solution_str, ground_truth)
    if ds in ("numina_aops_forum", "numina_synthetic_math", "numina_amc_aime", "numina_synthetic_amc", "numina_cn_k12",
              "numina_olympiads", "prime_math", "math_verify"):
        # the reference scores these with sympy / math-verify; here: string, exact-rational / numeric and
        # element-wise (tuple, set, interval) equivalence from math_verify.py
        from . import math_verify
        return math_verify.compute_score(solution_str, ground_truth)
    if ds in ("codecontests", "apps", "codeforces", "taco", "prime_code"):
        url = kwargs.get("sandbox_fusion_url")
        if url:
            from . import sandbox_fusion
            return sandbox_fusion.compute_score(url, kwargs.get("concurrent_semaphore"), solution_str, ground_truth,
                                                continuous=True)
        from . import prime_code
        return prime_code.compute_score(solution_str, ground_truth, continuous=True)
    if ds == "synthetic/arith":
        return _arith(solution_str, ground_truth)
    if ds == "synthetic/bernoulli":
        return _bernoulli(extra_info)
    if ds == "synthetic/random":
        return _length_score(solution_str, extra_info)
    if ds == "synthetic/parity":
        # decided on token ids by the reward manager (needs the raw ids, not text)
        return float((extra_info or {}).get("last_token_even", 0.0))
    raise NotImplementedError(f"Reward function is not implemented for data_source={data_source!r}")


compute_score = default_compute_score
