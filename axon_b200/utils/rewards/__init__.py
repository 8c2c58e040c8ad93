"""Reward functions: ``fn(task_info: dict, action: str) -> RewardOutput`` registered by name in
``REWARD_FN_REGISTRY`` (reference: axon/utils/rewards/__init__.py; math normalisation after
axon/utils/rewards/math_utils/utils.py). Shipped: math, code (sandboxed subprocess tests), f1, gpqa,
ifbench, remote, zero, bernoulli (synthetic benchmark reward)."""
from __future__ import annotations

import hashlib
import re
import string
import subprocess
import sys
import tempfile
from collections import Counter
from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Callable, Protocol


class RewardType(Enum):
    MATH = "math"
    CODE = "code"
    F1 = "f1"
    GPQA = "gpqa"
    IFBENCH = "ifbench"
    REMOTE = "remote"
    ZERO = "zero"
    UNK = "unk"


@dataclass
class RewardConfig:
    correct_reward: float = 1.0
    incorrect_reward: float = 0.0
    format_error_reward: float = 0.0
    unk_error_reward: float = 0.0
    apply_format_reward: bool = False
    code_timeout: float = 10.0
    remote_url: str = ""


@dataclass
class RewardInput:
    task_info: dict
    action: str


@dataclass
class RewardOutput:
    reward: float
    is_correct: bool = False
    metadata: dict = field(default_factory=dict)


class RewardFunction(Protocol):
    def __call__(self, task_info: dict, action: str) -> RewardOutput: ...


REWARD_FN_REGISTRY: dict[str, Callable] = {}


def register_reward(name: str):
    def deco(fn):
        REWARD_FN_REGISTRY[name] = fn
        return fn
    return deco


def _strip_think(text: str) -> str:
    return text.split("</think>")[-1] if "</think>" in text else text


# ------------------------------------------------------------------------------------------ math
def last_boxed(text: str) -> str | None:
    """Content of the last ``\\boxed{...}`` (balanced braces) or ``\\boxed x``."""
    i = text.rfind("\\boxed")
    if i < 0:
        i = text.rfind("\\fbox")
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


def normalize_math(ans: str) -> str:
    s = ans.strip().strip("$")
    s = re.sub(r"\\text\{(.*?)\}", r"\1", s)
    s = re.sub(r"\\(?:left|right|,|!|;|:| )", "", s)
    s = s.replace("\\dfrac", "\\frac").replace("\\tfrac", "\\frac").replace("^\\circ", "").replace("^{\\circ}", "")
    s = s.replace("\\%", "").replace("%", "").replace("\\$", "").replace("dollars", "")
    s = re.sub(r"\\frac\{([^{}]+)\}\{([^{}]+)\}", r"(\1)/(\2)", s)
    s = re.sub(r"\\sqrt\{([^{}]+)\}", r"sqrt(\1)", s)
    s = re.sub(r"(\d),(\d{3})", r"\1\2", s)
    s = s.replace(" ", "").rstrip(".").lower()
    if re.fullmatch(r"[a-z]=.+", s):
        s = s[2:]
    return s


def _as_number(s: str) -> float | None:
    try:
        if re.fullmatch(r"\(?-?[\d.]+\)?/\(?-?[\d.]+\)?", s):
            a, b = s.replace("(", "").replace(")", "").split("/")
            return float(a) / float(b)
        return float(s)
    except (ValueError, ZeroDivisionError):
        return None


def math_equal(pred: str, truth: str) -> bool:
    """Quick string / numeric comparison first, then the full grader (normalisation in the MATH checker's style, tuples /
    intervals / sets element-wise, symbolic equality with sympy): ``math_grading.grade_answer``."""
    a, b = normalize_math(pred), normalize_math(truth)
    if a == b:
        return True
    x, y = _as_number(a), _as_number(b)
    if x is not None and y is not None:
        return abs(x - y) <= 1e-6 * max(1.0, abs(y))
    from .math_grading import grade_answer
    return grade_answer(pred, truth)


@register_reward("math")
def math_reward_fn(task_info: dict, action: str, config: RewardConfig | None = None) -> RewardOutput:
    cfg = config or RewardConfig()
    truths = task_info.get("ground_truth", task_info.get("answer"))
    if truths is None:
        return RewardOutput(cfg.unk_error_reward, False, {"error": "no ground truth"})
    truths = truths if isinstance(truths, (list, tuple)) else [truths]
    from .math_grading import extract_answer
    pred = extract_answer(_strip_think(action or ""))        # the last boxed expression, else a closing "answer is ..."
    if pred is None:
        return RewardOutput(cfg.format_error_reward, False, {"error": "no boxed answer"})
    for t in truths:
        t = str(t)
        t = last_boxed(t) or t
        if math_equal(pred, t):
            return RewardOutput(cfg.correct_reward, True, {"pred": pred})
    return RewardOutput(cfg.incorrect_reward, False, {"pred": pred})


# ------------------------------------------------------------------------------------------ code
def extract_code(text: str) -> str | None:
    blocks = re.findall(r"```(?:python|py)?\n(.*?)```", _strip_think(text), re.S)
    return blocks[-1] if blocks else None


def run_python_sandboxed(code: str, stdin: str = "", timeout: float = 10.0) -> tuple[bool, str]:
    """Run code in a separate interpreter with a time limit and no inherited environment."""
    with tempfile.NamedTemporaryFile("w", suffix=".py", delete=True) as f:
        f.write(code)
        f.flush()
        try:
            r = subprocess.run([sys.executable, "-I", f.name], input=stdin, capture_output=True, text=True,
                               timeout=timeout, env={"PATH": "/usr/bin:/bin"})
            return r.returncode == 0, r.stdout if r.returncode == 0 else r.stderr[-2000:]
        except subprocess.TimeoutExpired:
            return False, "timeout"


@register_reward("code")
def code_reward_fn(task_info: dict, action: str, config: RewardConfig | None = None) -> RewardOutput:
    """``task_info['tests']``: list of {input, output} (stdin/stdout) or {assert: "..."} snippets."""
    cfg = config or RewardConfig()
    code = extract_code(action or "")
    if code is None:
        return RewardOutput(cfg.format_error_reward, False, {"error": "no code block"})
    tests = task_info.get("tests", task_info.get("ground_truth", []))
    if not tests:
        return RewardOutput(cfg.unk_error_reward, False, {"error": "no tests"})
    source = task_info.get("data_source", "")
    if source:
        # dataset formats of the reference (taco / apps / code_contests, primeintellect, livecodebench / codeforces,
        # leetcode, kodcode, humanevalplus); unknown sources raise, as there
        from .code_graders import grade
        good, details = grade(source, tests, code, timeout=cfg.code_timeout, entry_point=task_info.get("entry_point"))
        return RewardOutput(cfg.correct_reward if good else cfg.incorrect_reward, good, details)
    passed = 0
    for t in tests:
        if "assert" in t:
            ok, _ = run_python_sandboxed(code + "\n" + t["assert"], timeout=cfg.code_timeout)
        else:
            ok, out = run_python_sandboxed(code, stdin=str(t.get("input", "")), timeout=cfg.code_timeout)
            ok = ok and out.strip() == str(t.get("output", "")).strip()
        passed += int(ok)
    good = passed == len(tests)
    return RewardOutput(cfg.correct_reward if good else cfg.incorrect_reward, good, {"passed": passed, "total": len(tests)})


# ------------------------------------------------------------------------------------------ text
def _norm_text(s: str) -> list[str]:
    s = s.lower()
    s = "".join(ch for ch in s if ch not in set(string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return s.split()


def f1_score(pred: str, truth: str) -> float:
    p, t = _norm_text(pred), _norm_text(truth)
    if not p or not t:
        return float(p == t)
    common = sum((Counter(p) & Counter(t)).values())
    if common == 0:
        return 0.0
    prec, rec = common / len(p), common / len(t)
    return 2 * prec * rec / (prec + rec)


@register_reward("f1")
def f1_reward_fn(task_info: dict, action: str, config: RewardConfig | None = None) -> RewardOutput:
    truths = task_info.get("ground_truth", task_info.get("answer", ""))
    truths = truths if isinstance(truths, (list, tuple)) else [truths]
    text = _strip_think(action or "")
    m = re.findall(r"<answer>(.*?)</answer>", text, re.S)
    pred = m[-1] if m else text
    best = max((f1_score(pred, str(t)) for t in truths), default=0.0)
    return RewardOutput(best, best >= 1.0 - 1e-9, {"f1": best})


@register_reward("gpqa")
def gpqa_reward_fn(task_info: dict, action: str, config: RewardConfig | None = None) -> RewardOutput:
    cfg = config or RewardConfig()
    truth = str(task_info.get("ground_truth", task_info.get("answer", ""))).strip().upper()
    text = _strip_think(action or "")
    pred = last_boxed(text)
    if pred is None:
        m = re.findall(r"(?:answer|Answer)\s*(?:is|:)?\s*\(?([A-Da-d])\)?", text)
        pred = m[-1] if m else None
    if pred is None:
        return RewardOutput(cfg.format_error_reward, False, {"error": "no choice"})
    good = pred.strip().strip("()").upper()[:1] == truth[:1]
    return RewardOutput(cfg.correct_reward if good else cfg.incorrect_reward, good, {"pred": pred})


_IF_CHECKS = {
    "max_words": lambda text, v: len(text.split()) <= int(v),
    "min_words": lambda text, v: len(text.split()) >= int(v),
    "contains": lambda text, v: all(k.lower() in text.lower() for k in (v if isinstance(v, list) else [v])),
    "not_contains": lambda text, v: all(k.lower() not in text.lower() for k in (v if isinstance(v, list) else [v])),
    "lowercase": lambda text, v: text == text.lower(),
    "uppercase": lambda text, v: text == text.upper(),
    "ends_with": lambda text, v: text.rstrip().endswith(str(v)),
    "num_paragraphs": lambda text, v: len([p for p in text.split("\n\n") if p.strip()]) == int(v),
    "json": lambda text, v: _is_json(text),
}


def _is_json(text: str) -> bool:
    import json
    try:
        json.loads(text.strip().removeprefix("```json").removesuffix("```"))
        return True
    except ValueError:
        return False


@register_reward("ifbench")
def ifbench_reward_fn(task_info: dict, action: str, config: RewardConfig | None = None) -> RewardOutput:
    """Instruction-following: ``task_info['constraints']`` maps check names to arguments; reward is the
    fraction satisfied (1.0 only counts as correct)."""
    cons = task_info.get("constraints", {})
    text = _strip_think(action or "")
    if not cons:
        return RewardOutput(0.0, False, {"error": "no constraints"})
    ok = [bool(_IF_CHECKS[k](text, v)) for k, v in cons.items() if k in _IF_CHECKS]
    frac = sum(ok) / max(1, len(ok))
    return RewardOutput(frac, frac == 1.0, {"satisfied": sum(ok), "total": len(ok)})


@register_reward("remote")
def remote_reward_fn(task_info: dict, action: str, config: RewardConfig | None = None) -> RewardOutput:
    """POST {task_info, action} to ``task_info['reward_url']`` (or config.remote_url); expects {reward}."""
    url = task_info.get("reward_url") or (config.remote_url if config else "")
    if not url:
        return RewardOutput(0.0, False, {"error": "no reward_url"})
    try:
        import httpx
        r = httpx.post(url, json={"task_info": task_info, "action": action}, timeout=60.0)
        r.raise_for_status()
        d = r.json()
        return RewardOutput(float(d.get("reward", 0.0)), bool(d.get("is_correct", False)), d.get("metadata", {}))
    except Exception as e:  # noqa: BLE001
        return RewardOutput(0.0, False, {"error": f"{type(e).__name__}: {e}"})


@register_reward("zero")
def zero_reward_fn(task_info: dict, action: str, config: RewardConfig | None = None) -> RewardOutput:
    return RewardOutput(0.0, False, {})


@register_reward("bernoulli")
def bernoulli_reward_fn(task_info: dict, action: str, config: RewardConfig | None = None) -> RewardOutput:
    """Deterministic pseudo-random 0/1 reward with P(1) = task_info['p'] (default 0.5), seeded by the
    task seed and the response text. The synthetic reward of the throughput benchmarks."""
    p = float(task_info.get("p", 0.5))
    h = hashlib.sha256(f"{task_info.get('seed', 0)}|{action}".encode()).digest()
    u = int.from_bytes(h[:8], "big") / 2 ** 64
    return RewardOutput(float(u < p), u < p, {})
