"""Answer equivalence for math tasks without a computer-algebra dependency.

The reference scores ``math_verify`` / ``prime_math`` / numina sources with the ``math-verify`` and sympy packages
(siirl/utils/reward_score/math_verify.py:24-39, prime_math/__init__.py).  Neither is a dependency here: answers are
compared (1) as normalised strings, (2) as exact rationals / floats after translating the common LaTeX forms
(``\\frac{a}{b}``, ``\\sqrt{x}``, ``\\pi``, ``^``, ``\\cdot``, ``\\times``, percent, thousands separators, mixed
numbers, scientific notation) into arithmetic that a restricted AST evaluator computes, (3) element-wise for tuples,
sets and intervals.  Expressions with free variables fall back to the string comparison."""
from __future__ import annotations

import ast
import math
import re
from fractions import Fraction
from typing import List, Optional, Sequence, Union

from .math import last_boxed_only_string, remove_boxed, strip_string

Number = Union[Fraction, float]

_TEXT = re.compile(r"\\(?:text|mathrm|textbf|mathbf|mbox)\{([^{}]*)\}")
_UNITS = re.compile(r"(?<=[0-9)])\s*(?:cm|mm|km|kg|mph|meters?|inches|inch|feet|foot|units?|degrees?|dollars?|cents?"
                    r"|hours?|minutes?|seconds?|days?|years?|sq|square)\b.*$", re.I)


def _balanced(s: str, start: int) -> int:
    """Index just past the ``}`` that closes the ``{`` at ``start``; -1 if unbalanced."""
    depth = 0
    for i in range(start, len(s)):
        if s[i] == "{":
            depth += 1
        elif s[i] == "}":
            depth -= 1
            if depth == 0:
                return i + 1
    return -1


def _group(s: str, i: int):
    """A LaTeX argument at position i: ``{...}`` or a single character.  Returns (content, next index)."""
    while i < len(s) and s[i] == " ":
        i += 1
    if i >= len(s):
        return None, i
    if s[i] == "{":
        j = _balanced(s, i)
        if j < 0:
            return None, i
        return s[i + 1:j - 1], j
    return s[i], i + 1


def latex_to_expr(s: str) -> str:
    """Translate the arithmetic subset of LaTeX into a Python expression string."""
    s = s.strip().strip("$").strip()
    s = _TEXT.sub(lambda m: m.group(1), s)
    s = s.replace("\\!", "").replace("\\,", "").replace("\\;", "").replace("\\ ", " ").replace("\\$", "")
    s = s.replace("\\left", "").replace("\\right", "").replace("\\dfrac", "\\frac").replace("\\tfrac", "\\frac")
    s = s.replace("\\cdot", "*").replace("\\times", "*").replace("\\div", "/").replace("\\%", "%")
    s = s.replace("^\\circ", "").replace("^{\\circ}", "").replace("°", "")
    s = _UNITS.sub("", s)
    out: List[str] = []
    i = 0
    while i < len(s):
        if s.startswith("\\frac", i):
            a, j = _group(s, i + 5)
            b, k = _group(s, j)
            if a is None or b is None:
                raise ValueError("malformed \\frac")
            out.append(f"(({latex_to_expr(a)})/({latex_to_expr(b)}))")
            i = k
        elif s.startswith("\\sqrt", i):
            j = i + 5
            root = None
            if j < len(s) and s[j] == "[":
                e = s.index("]", j)
                root = s[j + 1:e]
                j = e + 1
            a, k = _group(s, j)
            if a is None:
                raise ValueError("malformed \\sqrt")
            out.append(f"(({latex_to_expr(a)})**(1/({latex_to_expr(root)})))" if root else f"sqrt({latex_to_expr(a)})")
            i = k
        elif s.startswith("\\pi", i):
            out.append("pi")
            i += 3
        elif s[i] == "^":
            a, k = _group(s, i + 1)
            if a is None:
                raise ValueError("malformed exponent")
            out.append(f"**({latex_to_expr(a)})")
            i = k
        elif s[i] == "{":
            j = _balanced(s, i)
            if j < 0:
                raise ValueError("unbalanced braces")
            out.append(f"({latex_to_expr(s[i + 1:j - 1])})")
            i = j
        elif s[i] == "\\":
            raise ValueError(f"unsupported LaTeX command at {s[i:i + 12]!r}")
        else:
            out.append(s[i])
            i += 1
    expr = "".join(out).strip()
    expr = re.sub(r"(?<=\d),(?=\d{3}(?:\D|$))", "", expr)                 # 1,234,567
    expr = re.sub(r"^(\d+)\s*\(\((\d+)\)/\((\d+)\)\)$", r"(\1+(\2)/(\3))", expr) if not expr.startswith("-") \
        else re.sub(r"^-(\d+)\s*\(\((\d+)\)/\((\d+)\)\)$", r"(-(\1+(\2)/(\3)))", expr)   # mixed numbers: 1 \frac12
    if expr.endswith("%"):
        expr = f"({expr[:-1]})/100"
    # implicit multiplication: 2pi, 3sqrt(2), )(, 2(
    expr = re.sub(r"(\d|\))\s*(?=pi|sqrt|\()", r"\1*", expr)
    expr = re.sub(r"(pi)\s*(?=\d|\(|sqrt)", r"\1*", expr)
    return expr


_ALLOWED_BIN = {ast.Add: lambda a, b: a + b, ast.Sub: lambda a, b: a - b, ast.Mult: lambda a, b: a * b}


def _eval(node) -> Number:
    if isinstance(node, ast.Expression):
        return _eval(node.body)
    if isinstance(node, ast.Constant):
        if isinstance(node.value, bool) or not isinstance(node.value, (int, float)):
            raise ValueError("not a number")
        return Fraction(node.value) if isinstance(node.value, int) else Fraction(repr(node.value))
    if isinstance(node, ast.UnaryOp) and isinstance(node.op, (ast.USub, ast.UAdd)):
        v = _eval(node.operand)
        return -v if isinstance(node.op, ast.USub) else v
    if isinstance(node, ast.BinOp):
        a, b = _eval(node.left), _eval(node.right)
        if type(node.op) in _ALLOWED_BIN:
            return _ALLOWED_BIN[type(node.op)](a, b)
        if isinstance(node.op, ast.Div):
            if b == 0:
                raise ValueError("division by zero")
            return a / b
        if isinstance(node.op, ast.Pow):
            if isinstance(b, Fraction) and b.denominator == 1 and abs(b) <= 64 and isinstance(a, Fraction):
                if a == 0 and b < 0:
                    raise ValueError("division by zero")
                return a ** int(b)
            fa, fb = float(a), float(b)
            if fa < 0 and fb != int(fb):
                raise ValueError("complex result")
            if abs(fb) > 256:
                raise ValueError("exponent too large")
            return math.pow(fa, fb)
        raise ValueError("operator not allowed")
    if isinstance(node, ast.Name) and node.id == "pi":
        return math.pi
    if isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and node.func.id == "sqrt" \
            and len(node.args) == 1 and not node.keywords:
        v = _eval(node.args[0])
        if v < 0:
            raise ValueError("complex result")
        if isinstance(v, Fraction):
            n, d = math.isqrt(v.numerator), math.isqrt(v.denominator)
            if n * n == v.numerator and d * d == v.denominator:
                return Fraction(n, d)
        return math.sqrt(float(v))
    raise ValueError("expression not allowed")


def to_number(text: str) -> Optional[Number]:
    """The numeric value of an answer string, or ``None`` if it is not a closed arithmetic expression."""
    try:
        expr = latex_to_expr(text)
        if not expr or len(expr) > 256:
            return None
        return _eval(ast.parse(expr, mode="eval"))
    except (ValueError, SyntaxError, ZeroDivisionError, OverflowError, RecursionError, TypeError):
        return None


def numbers_equal(a: Number, b: Number, rel_tol: float = 1e-6) -> bool:
    if isinstance(a, Fraction) and isinstance(b, Fraction):
        return a == b
    fa, fb = float(a), float(b)
    return math.isclose(fa, fb, rel_tol=rel_tol, abs_tol=1e-9)


def _split_top_level(s: str) -> List[str]:
    """Split on commas that are not inside braces / brackets / parentheses (and not thousands separators)."""
    parts, depth, cur = [], 0, []
    for i, ch in enumerate(s):
        if ch in "{[(":
            depth += 1
        elif ch in "}])":
            depth -= 1
        if ch == "," and depth == 0 and not (i > 0 and s[i - 1].isdigit() and len(s[i + 1:i + 4]) == 3
                                               and s[i + 1:i + 4].isdigit() and not s[i + 4:i + 5].isdigit()):
            parts.append("".join(cur).strip())
            cur = []
        else:
            cur.append(ch)
    parts.append("".join(cur).strip())
    return [p for p in parts if p]


def _strip_assignment(s: str) -> str:
    """``x = 5`` -> ``5`` (a short left-hand side only, so that equations as answers are left alone)."""
    m = re.match(r"^\s*[A-Za-z](?:_\{?\w+\}?)?\s*=\s*(.+)$", s)
    return m.group(1) if m else s


def _single_equal(pred: str, truth: str) -> bool:
    pred, truth = _strip_assignment(pred), _strip_assignment(truth)
    pred, truth = _TEXT.sub(lambda m: m.group(1), pred).strip(), _TEXT.sub(lambda m: m.group(1), truth).strip()
    try:
        if strip_string(pred) == strip_string(truth):
            return True
    except Exception:  # noqa: BLE001 - the normaliser is best effort on malformed model output
        if pred.strip() == truth.strip():
            return True
    a, b = to_number(pred), to_number(truth)
    if a is None or b is None:
        return False
    if numbers_equal(a, b):
        return True
    # one side is a rounded decimal of the other ("0.6667" for 2/3): accept within half a unit of its last digit,
    # from two decimals on
    for text in (pred, truth):
        m = re.fullmatch(r"\s*-?\d*\.(\d{2,})\s*", text.replace("$", ""))
        if m and abs(float(a) - float(b)) <= 0.5000001 * 10.0 ** (-len(m.group(1))):
            return True
    return False


def is_equiv(pred: Optional[str], truth: Optional[str]) -> bool:
    """String, numeric, or element-wise (tuples, sets, intervals; sets are order-free) equivalence."""
    if pred is None or truth is None:
        return False
    p, t = pred.strip().strip("$").strip(), truth.strip().strip("$").strip()
    p = p.replace("\\left", "").replace("\\right", "")
    t = t.replace("\\left", "").replace("\\right", "")
    if _single_equal(p, t):
        return True
    openers = {"(": ")", "[": "]", "\\{": "\\}"}
    for o in ("\\{", "(", "["):
        if p.startswith(o) and t.startswith(o):
            pc = next((c for c in ("\\}", ")", "]") if p.endswith(c)), None)
            tc = next((c for c in ("\\}", ")", "]") if t.endswith(c)), None)
            if pc is None or pc != tc:
                return False              # (a, b) vs (a, b] are different intervals
            pe, te = _split_top_level(p[len(o):-len(pc)]), _split_top_level(t[len(o):-len(tc)])
            if len(pe) != len(te) or len(pe) < 2:
                return False
            if o == "\\{":
                rest = list(te)
                for x in pe:
                    hit = next((y for y in rest if _single_equal(x, y)), None)
                    if hit is None:
                        return False
                    rest.remove(hit)
                return True
            return all(_single_equal(x, y) for x, y in zip(pe, te))
    del openers
    # unordered lists without brackets: "1, 3" vs "3, 1"
    pe, te = _split_top_level(p), _split_top_level(t)
    if len(pe) == len(te) >= 2:
        rest = list(te)
        for x in pe:
            hit = next((y for y in rest if _single_equal(x, y)), None)
            if hit is None:
                return False
            rest.remove(hit)
        return True
    return False


def extract_answer(solution_str: str) -> Optional[str]:
    """The last ``\\boxed{...}`` of the solution; else what follows the last "answer is" / "Answer:"."""
    boxed = last_boxed_only_string(solution_str)
    if boxed is not None:
        try:
            return remove_boxed(boxed)
        except Exception:  # noqa: BLE001
            return None
    m = re.findall(r"(?:answer is|Answer:)\s*([^\n]+)", solution_str)
    if m:
        return m[-1].strip().rstrip(".").strip()
    return None


def compute_score(solution_str: str, ground_truth: Union[str, Sequence[str]], **_) -> float:
    pred = extract_answer(solution_str)
    if pred is None:
        return 0.0
    truths = [ground_truth] if isinstance(ground_truth, (str, int, float)) else list(ground_truth)
    for t in truths:
        t = str(t)
        if "\\boxed" in t:
            b = last_boxed_only_string(t)
            t = remove_boxed(b) if b else t
        if is_equiv(pred, t):
            return 1.0
    return 0.0
