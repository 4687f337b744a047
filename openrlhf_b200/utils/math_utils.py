"""Answer extraction and grading for math-style rule rewards: ``extract_boxed_answer`` and ``grade_answer`` (string
normalisation in the MATH style, then symbolic equivalence with sympy under a time limit). Same entry points as
openrlhf/utils/math_utils.py:285-425; the normalisation rules are written for this project."""
from __future__ import annotations

import re
import signal
import threading

_UNITS = ("degrees", "degree", "cm", "centimeters", "meters", "meter", "mph", "inches", "inch", "feet", "foot", "units",
          "unit", "square", "sq", "dollars", "dollar", "cents", "cent", "percent", "hours", "hour", "minutes", "minute",
          "seconds", "second", "miles", "mile", "points", "point")


class _SympyTimeout(Exception):
    pass


def last_boxed_only_string(string: str):
    """The last ``\\boxed{...}`` (or ``\\fbox{...}``) group including its braces, or None."""
    idx = max(string.rfind("\\boxed"), string.rfind("\\fbox"))
    if idx < 0:
        return None
    depth, start = 0, string.find("{", idx)
    if start < 0:
        return None
    for i in range(start, len(string)):
        if string[i] == "{":
            depth += 1
        elif string[i] == "}":
            depth -= 1
            if depth == 0:
                return string[idx:i + 1]
    return None


def remove_boxed(value: str):
    if value is None:
        return None
    m = re.match(r"\\(?:boxed|fbox)\s*\{(.*)\}\s*$", value, flags=re.S)
    return m.group(1) if m else None


def extract_boxed_answer(solution: str):
    """Content of the last \\boxed{} in a model response (None when there is none)."""
    return remove_boxed(last_boxed_only_string(solution))


def _fix_fracs(s: str) -> str:
    # \frac12 -> \frac{1}{2}; \frac1{72} -> \frac{1}{72}
    s = re.sub(r"\\[dt]frac", r"\\frac", s)
    s = re.sub(r"\\frac(\d)(\d)", r"\\frac{\1}{\2}", s)
    s = re.sub(r"\\frac(\d)\{", r"\\frac{\1}{", s)
    s = re.sub(r"\\frac\{([^{}]+)\}(\d)", r"\\frac{\1}{\2}", s)
    return s


def _fix_sqrt(s: str) -> str:
    return re.sub(r"\\sqrt(\w)", r"\\sqrt{\1}", s)


def _strip_string(s: str) -> str:
    s = str(s).replace("\n", "").replace("\\!", "").replace("\\\\", "\\")
    s = s.replace("\\left", "").replace("\\right", "").replace("^{\\circ}", "").replace("^\\circ", "")
    s = s.replace("\\$", "").replace("$", "").replace("\\%", "").replace("%", "")
    s = re.sub(r"\\text\{\s*([^{}]*)\}", r"\1", s)
    s = re.sub(r"\\mbox\{\s*([^{}]*)\}", r"\1", s)
    for u in _UNITS:
        s = re.sub(rf"(?<=[\d}}])\s*{u}\b", "", s)
    s = s.replace(" .", " 0.").replace("{.", "{0.")
    if s.startswith("."):
        s = "0" + s
    if "=" in s and len(s.split("=")[0]) <= 2:
        s = s.split("=", 1)[1]
    s = _fix_sqrt(s)
    s = s.replace(" ", "")
    s = _fix_fracs(s)
    if s == "0.5":
        s = "\\frac{1}{2}"
    m = re.fullmatch(r"(-?\d+)/(-?\d+)", s)
    if m:
        s = f"\\frac{{{m.group(1)}}}{{{m.group(2)}}}"
    return s


def mathd_normalize_answer(answer):
    if answer is None:
        return None
    answer = answer.strip()
    m = re.search(r"^\\text\{(?P<text>.+?)\}$", answer)
    if m:
        answer = m.group("text").strip()
    try:
        return _strip_string(answer)
    except Exception:  # noqa: BLE001
        return answer


def _normalize(expr):
    """Looser normalisation used before the symbolic comparison."""
    if expr is None:
        return None
    expr = mathd_normalize_answer(expr)
    expr = expr.replace("\\cdot", "*").replace("\\times", "*").replace("\\pi", "pi").replace("\\infty", "oo")
    expr = re.sub(r"\\frac\{([^{}]+)\}\{([^{}]+)\}", r"((\1)/(\2))", expr)
    expr = re.sub(r"\\sqrt\{([^{}]+)\}", r"sqrt(\1)", expr)
    expr = expr.replace("^", "**").replace("{", "(").replace("}", ")")
    expr = re.sub(r"(\d),(\d{3})", r"\1\2", expr)
    expr = re.sub(r"(\d)\s*\(", r"\1*(", expr)
    expr = re.sub(r"(\d)([a-zA-Z])", r"\1*\2", expr)
    return expr.strip().lower() if len(expr) > 1 else expr.strip()


def count_unknown_letters_in_expr(expr: str) -> int:
    """Distinct letters that are not part of a known function or constant name: free symbols sympy would have to carry."""
    return len(set(re.findall(r"[a-zA-Z]", re.sub(r"sqrt|frac|pi|oo", "", expr))))


def should_allow_eval(expr: str) -> bool:
    """Expressions handed to sympy stay small: at most two free symbols, no braced / parenthesised or chained powers,
    no exponent of two or more digits (a tower like 9^99^9 would run until the time limit), no Python syntax."""
    if count_unknown_letters_in_expr(expr) > 2:
        return False
    if any(b in expr for b in ("^{", "^(", "__", "import", "lambda")):
        return False
    return re.search(r"\^[0-9]+\^|\^[0-9][0-9]+", expr) is None


def are_equal_under_sympy(ground_truth_normalized: str, given_normalized: str, timeout: int = 120) -> bool:
    def handler(signum, frame):
        raise _SympyTimeout()

    use_alarm = threading.current_thread() is threading.main_thread() and hasattr(signal, "SIGALRM")
    old = None
    try:
        if use_alarm:
            old = signal.signal(signal.SIGALRM, handler)
            signal.alarm(timeout)
        import sympy
        from sympy.parsing.sympy_parser import parse_expr

        expr = f"({ground_truth_normalized})-({given_normalized})"
        if not should_allow_eval(expr):
            return False
        return sympy.simplify(parse_expr(expr)) == 0
    except Exception:  # noqa: BLE001  (includes the timeout)
        return False
    finally:
        if use_alarm:
            signal.alarm(0)
            if old is not None:
                signal.signal(signal.SIGALRM, old)


def split_tuple(expr: str) -> list[str]:
    expr = expr.strip()
    if len(expr) > 2 and expr[0] in "([" and expr[-1] in ")]" and "," in expr:
        return [e.strip() for e in expr[1:-1].split(",")]
    return [expr]


def grade_answer_mathd(given_answer: str, ground_truth: str) -> bool:
    return mathd_normalize_answer(ground_truth) == mathd_normalize_answer(given_answer)


def grade_answer_sympy(given_answer: str, ground_truth: str) -> bool:
    gt, gv = _normalize(ground_truth), _normalize(given_answer)
    if gt is None or gv is None or len(gv) == 0:
        return False
    if gt == gv:
        return True
    a, b = split_tuple(gt), split_tuple(gv)
    if len(a) != len(b) or (len(a) > 1 and (gt[0] != gv[0] or gt[-1] != gv[-1])):
        return False
    return all(x == y or are_equal_under_sympy(x, y) for x, y in zip(a, b))


def grade_answer(given_answer: str, ground_truth: str) -> bool:
    """True when the answers agree after normalisation or are symbolically equal."""
    if given_answer is None:
        return False
    return grade_answer_mathd(given_answer, ground_truth) or grade_answer_sympy(given_answer, ground_truth)
