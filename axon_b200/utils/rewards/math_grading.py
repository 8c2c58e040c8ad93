"""Grading of free-form mathematical answers (reference: axon/utils/rewards/math_utils/utils.py - string
normalisation in the style of the MATH dataset's checker, then symbolic equality; math_reward.py picks the last boxed
answer and accepts a list of ground truths).

Three stages, cheapest first; an answer is right as soon as one stage says so:

  1. ``normalize_answer``: LaTeX cosmetics removed (``\\left`` / ``\\right``, thin spaces, ``\\text{...}`` wrappers,
     ``\\dfrac`` -> ``\\frac``, ``\\frac12`` -> ``\\frac{1}{2}``, ``a/b`` -> ``\\frac{a}{b}`` for integers, degrees, percent and
     currency signs, trailing units, thousands separators, ``x = ...`` prefixes, leading zero of decimals) and the strings compared;
  2. numeric comparison when both sides evaluate to numbers (fractions, percentages, scientific notation);
  3. symbolic comparison with sympy on a LaTeX -> expression translation of both sides (``simplify(a - b) == 0``),
     element-wise for tuples, intervals (bracket types must agree) and sets written as comma lists. Expressions that
     would make sympy expand towers of powers or that contain too many distinct unknowns are not evaluated.
"""
from __future__ import annotations

import re

_UNITS = ("degrees", "degree", "cm", "centimeters", "meters", "meter", "mph", "inches", "inch", "feet", "foot", "units", "unit",
          "square", "sq", "dollars", "dollar", "cents", "cent", "hours", "hour", "minutes", "minute", "seconds", "second",
          "days", "day", "points", "point", "percent", "mm", "km", "kg", "grams", "gram", "ounces", "ounce", "pounds", "pound")
_WORD_NUMBERS = {"zero": "0", "one": "1", "two": "2", "three": "3", "four": "4", "five": "5", "six": "6", "seven": "7", "eight": "8",
                 "nine": "9", "ten": "10", "eleven": "11", "twelve": "12"}


def last_boxed(text: str) -> str | None:
    """Content of the last ``\\boxed{...}`` / ``\\fbox{...}`` (balanced braces), or of ``\\boxed x``."""
    i = max(text.rfind("\\boxed"), text.rfind("\\fbox"))
    if i < 0:
        return None
    j = text.find("{", i)
    if j < 0 or text[i:j].strip() not in ("\\boxed", "\\fbox"):
        tail = text[i:].split()
        return tail[1].rstrip("$.") if len(tail) > 1 else None
    depth = 0
    for k in range(j, len(text)):
        if text[k] == "{":
            depth += 1
        elif text[k] == "}":
            depth -= 1
            if depth == 0:
                return text[j + 1:k]
    return None


def extract_answer(text: str) -> str | None:
    """The answer a solution text commits to: the last boxed expression, else what follows a final ``answer is`` /
    ``Answer:`` (up to the end of that line, trailing period dropped)."""
    b = last_boxed(text)
    if b is not None:
        return b
    m = None
    for m in re.finditer(r"(?:final answer|answer)\s*(?:is|:)\s*(.+)", text, flags=re.I):
        pass
    if m:
        return m.group(1).strip().split("\n")[0].rstrip(". ").strip("$ ")
    return None


def _fix_fracs(s: str) -> str:
    """``\\frac12`` -> ``\\frac{1}{2}``, ``\\frac1{72}`` -> ``\\frac{1}{72}``, ``\\frac{a}b`` -> ``\\frac{a}{b}``."""
    out, i = [], 0
    while i < len(s):
        if s.startswith("\\frac", i):
            out.append("\\frac")
            i += 5
            for _ in range(2):
                if i < len(s) and s[i] == "{":
                    depth, j = 0, i
                    while j < len(s):
                        depth += s[j] == "{"
                        depth -= s[j] == "}"
                        j += 1
                        if depth == 0:
                            break
                    out.append(s[i:j])
                    i = j
                elif i < len(s):
                    out.append("{" + s[i] + "}")
                    i += 1
            continue
        out.append(s[i])
        i += 1
    return "".join(out)


def _fix_sqrt(s: str) -> str:
    return re.sub(r"\\sqrt(\w)", r"\\sqrt{\1}", s)


def normalize_answer(ans: str | None) -> str | None:
    if ans is None:
        return None
    s = str(ans).strip()
    m = re.fullmatch(r"\\text\{(.*)\}", s)
    if m:
        s = m.group(1).strip()
    s = s.replace("\n", "").replace("\\!", "").replace("\\,", "").replace("\\;", "").replace("\\:", "").replace("\\ ", " ")
    s = s.replace("\\left", "").replace("\\right", "").replace("\\displaystyle", "")
    s = s.replace("\\dfrac", "\\frac").replace("\\tfrac", "\\frac").replace("\\cdot", "*").replace("\\times", "*")
    s = s.replace("^\\circ", "").replace("^{\\circ}", "").replace("°", "")
    s = s.replace("\\$", "").replace("$", "").replace("\\%", "%")
    s = re.sub(r"\\text\{\s*([^{}]*)\}", r" \1", s)
    s = re.sub(r"\\mbox\{\s*([^{}]*)\}", r" \1", s)
    s = re.sub(r"\\(?:mathrm|textbf|mathbf|mathit)\{([^{}]*)\}", r"\1", s)
    low = s.strip().lower()
    if low in _WORD_NUMBERS:
        return _WORD_NUMBERS[low]
    # trailing units ("5 cm", "12 square units", "30 degrees", "4 cm^2")
    units = "|".join(sorted(_UNITS, key=len, reverse=True))
    m = re.fullmatch(rf"(.*\d[\d\s.,/)}}]*?)((?:\s*(?:{units})(?:\^\{{?\d\}}?)?)+)\.?", s.strip(), flags=re.I)
    if m:
        s = m.group(1)
    s = s.strip().rstrip(".")
    if re.fullmatch(r"[A-Za-z]\s*=\s*[^=]+", s):            # "x = 5" -> "5"
        s = s.split("=", 1)[1]
    s = re.sub(r"(\d),(?=\d{3}(?:\D|$))", r"\1", s)           # 1,234,567 -> 1234567
    s = s.replace(" ", "")
    s = _fix_sqrt(_fix_fracs(s))
    m = re.fullmatch(r"(-?\d+)/(-?\d+)", s)
    if m:
        s = f"\\frac{{{m.group(1)}}}{{{m.group(2)}}}"
    if s.startswith("."):
        s = "0" + s
    s = re.sub(r"(?<=\D)\.(?=\d)", "0.", s) if not s[:1].isdigit() else s
    s = re.sub(r"(\d+\.\d*?)0+(?=\D|$)", lambda mm: mm.group(1).rstrip("."), s)      # 2.50 -> 2.5, 3.0 -> 3
    if s.endswith("%"):
        s = s[:-1]
    return s


def _to_number(s: str) -> float | None:
    s = s.replace("\\frac{", "(").replace("}{", ")/(").replace("}", ")") if s.startswith("\\frac{") or "\\frac{" in s else s
    s = s.replace("^", "**")
    if not re.fullmatch(r"[-+*/().\deE ]+", s):
        return None
    if "**" in s and len(s) > 20:
        return None
    try:
        return float(eval(s, {"__builtins__": {}}, {}))       # digits and arithmetic signs only (checked above)
    except Exception:  # noqa: BLE001
        return None


def latex_to_expr(s: str) -> str:
    """A sympy-parsable rendering of the LaTeX subset answers use."""
    s = _fix_sqrt(_fix_fracs(s))
    for _ in range(8):                                       # innermost fractions / roots first
        new = re.sub(r"\\frac\{([^{}]*)\}\{([^{}]*)\}", r"((\1)/(\2))", s)
        new = re.sub(r"\\sqrt\[([^\[\]]*)\]\{([^{}]*)\}", r"((\2)**(1/(\1)))", new)
        new = re.sub(r"\\sqrt\{([^{}]*)\}", r"sqrt(\1)", new)
        if new == s:
            break
        s = new
    s = s.replace("\\pi", "pi").replace("\\infty", "oo").replace("\\cdot", "*").replace("\\times", "*").replace("\\div", "/")
    s = re.sub(r"\\(sin|cos|tan|log|ln|exp)", r"\1", s)
    s = s.replace("ln(", "log(")
    s = s.replace("^{", "**(").replace("^", "**")
    s = s.replace("{", "(").replace("}", ")")
    s = re.sub(r"(\d)\s*(?=[a-zA-Z(])", r"\1*", s)            # 2x -> 2*x, 3( -> 3*(
    s = re.sub(r"\)\s*(?=[\w(])", ")*", s)
    s = re.sub(r"\\[a-zA-Z]+", "", s)
    return s


def _safe_for_sympy(expr: str) -> bool:
    if len(expr) > 300 or expr.count("**") > 4 or re.search(r"\*\*\s*\(?\s*\d{4,}", expr):
        return False
    names = set(re.findall(r"[a-zA-Z_]\w*", expr)) - {"sqrt", "pi", "oo", "sin", "cos", "tan", "log", "exp", "e", "E", "I"}
    return len(names) <= 3


def symbolic_equal(a: str, b: str) -> bool:
    ea, eb = latex_to_expr(a), latex_to_expr(b)
    if not (_safe_for_sympy(ea) and _safe_for_sympy(eb)):
        return False
    try:
        import sympy
        from sympy.parsing.sympy_parser import parse_expr
        xa, xb = parse_expr(ea, evaluate=True), parse_expr(eb, evaluate=True)
        if xa == xb:
            return True
        d = sympy.simplify(xa - xb)
        return d == 0
    except Exception:  # noqa: BLE001 - unparsable input is simply "not shown equal"
        return False


def _split_top_level(s: str) -> list[str]:
    parts, depth, cur = [], 0, []
    for ch in s:
        if ch in "([{":
            depth += 1
        elif ch in ")]}":
            depth -= 1
        if ch == "," and depth == 0:
            parts.append("".join(cur))
            cur = []
        else:
            cur.append(ch)
    parts.append("".join(cur))
    return [p.strip() for p in parts]


def _container(s: str):
    """(opening bracket, closing bracket, elements) of a tuple / interval / set, or None for a scalar."""
    s = s.strip()
    s = s.replace("\\{", "{").replace("\\}", "}")
    if len(s) >= 2 and s[0] in "([{" and s[-1] in ")]}":
        inner = _split_top_level(s[1:-1])
        if len(inner) > 1:
            return s[0], s[-1], inner
    return None


def _scalar_equal(a: str, b: str) -> bool:
    if a == b:
        return True
    x, y = _to_number(a), _to_number(b)
    if x is not None and y is not None:
        return abs(x - y) <= 1e-6 * max(1.0, abs(y))
    return symbolic_equal(a, b)


def grade_answer(given: str | None, truth: str | None) -> bool:
    """Is ``given`` the same mathematical object as ``truth``?"""
    a, b = normalize_answer(given), normalize_answer(truth)
    if a is None or b is None or a == "" or b == "":
        return False
    if a == b:
        return True
    ca, cb = _container(a), _container(b)
    if (ca is None) != (cb is None):
        # an unbracketed comma list against a bracketed one ("1, 2" vs "(1,2)") is still a list answer
        la, lb = _split_top_level(a) if ca is None else ca[2], _split_top_level(b) if cb is None else cb[2]
        if len(la) > 1 and len(la) == len(lb):
            return all(_scalar_equal(x, y) for x, y in zip(la, lb))
        return False
    if ca is not None:
        (oa, za, ea), (ob, zb, eb) = ca, cb
        if len(ea) != len(eb) or (oa, za) != (ob, zb):
            return False
        if oa == "{":                                         # sets: order does not matter
            left = list(eb)
            for x in ea:
                hit = next((y for y in left if _scalar_equal(x, y)), None)
                if hit is None:
                    return False
                left.remove(hit)
            return True
        return all(_scalar_equal(x, y) for x, y in zip(ea, eb))
    la, lb = _split_top_level(a), _split_top_level(b)
    if len(la) > 1 or len(lb) > 1:                            # bare comma lists: compare as multisets
        if len(la) != len(lb):
            return False
        left = list(lb)
        for x in la:
            hit = next((y for y in left if _scalar_equal(x, y)), None)
            if hit is None:
                return False
            left.remove(hit)
        return True
    return _scalar_equal(a, b)
