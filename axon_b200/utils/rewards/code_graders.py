"""Dataset-aware graders for code rewards.

The reference grades model code per data source (axon/utils/rewards/code_reward.py:455-541: taco / apps /
code_contests and primeintellect as input/output lists with an optional function name, livecodebench /
codeforces as a list of cases with a test type, leetcode as a test script, kodcode as a pytest-style file
that imports ``solution``, humanevalplus as a ``check(candidate)`` body) and runs them in a firejail
sandbox. Here every format is reduced to one of three runs in a separate, isolated interpreter with a time
limit (``run_python_sandboxed``): feed stdin and compare stdout, call a function with JSON arguments and
compare its return value, or run a script that raises on failure. ``grade`` returns (all passed, details)
with one entry per test in ``details['test_results']``.
"""
from __future__ import annotations

import ast
import json
import os
import re
import subprocess
import sys
import tempfile

STDIN_SOURCES = ("taco", "apps", "code_contests", "primeintellect", "livecodebench", "codeforces")

_CALL_HARNESS = '''
import json as _json, sys as _sys
_spec = _json.loads(_sys.stdin.read())
_fn = globals().get(_spec["fn"])
if _fn is None and "Solution" in globals():
    _fn = getattr(Solution(), _spec["fn"])
_out = _fn(*_spec["args"])
if isinstance(_out, tuple):
    _out = list(_out)
print("\\n__RESULT__" + _json.dumps(_out))
'''


def clean_main_block(code: str) -> str:
    """Drop a trailing ``if __name__ == "__main__":`` block (test files import the solution)."""
    m = re.search(r'^if\s+__name__\s*==\s*[\'"]__main__[\'"]\s*:', code, re.M)
    return code[:m.start()] if m else code


def _run(code: str, stdin: str, timeout: float, extra_files: dict | None = None) -> tuple[bool, str]:
    with tempfile.TemporaryDirectory() as d:
        for name, text in (extra_files or {}).items():
            with open(os.path.join(d, name), "w") as f:
                f.write(text)
        path = os.path.join(d, "main.py")
        with open(path, "w") as f:
            if extra_files:          # isolated mode keeps the script's folder off sys.path
                f.write("import sys as _s, os as _o\n_s.path.insert(0, _o.path.dirname(_o.path.abspath(__file__)))\n")
            f.write(code)
        try:
            r = subprocess.run([sys.executable, "-I", path], input=stdin, capture_output=True, text=True, timeout=timeout,
                               cwd=d, env={"PATH": "/usr/bin:/bin", "PYTHONPATH": d})
        except subprocess.TimeoutExpired:
            return False, "timeout"
        return r.returncode == 0, r.stdout if r.returncode == 0 else (r.stderr or r.stdout)[-2000:]


def outputs_match(got: str, want: str) -> bool:
    """Whitespace-insensitive, line by line; tokens that parse as numbers compare with a small tolerance."""
    g, w = got.strip().split("\n"), str(want).strip().split("\n")
    if len(g) != len(w):
        return False
    for a, b in zip(g, w):
        ta, tb = a.split(), b.split()
        if ta == tb:
            continue
        if len(ta) != len(tb):
            return False
        for x, y in zip(ta, tb):
            if x == y:
                continue
            try:
                if abs(float(x) - float(y)) > 1e-6 * max(1.0, abs(float(y))):
                    return False
            except ValueError:
                return False
    return True


def _parse(tests):
    if isinstance(tests, str):
        try:
            return json.loads(tests)
        except json.JSONDecodeError:
            return ast.literal_eval(tests)
    return tests


def _cases(data_source: str, tests) -> list[dict]:
    """Normalise to [{input, output, fn}] (fn None = stdin / stdout)."""
    tests = _parse(tests)
    if isinstance(tests, dict):                                   # taco / apps / code_contests
        ins, outs, fn = tests.get("inputs", []), tests.get("outputs", []), tests.get("fn_name")
        n = max(len(ins), len(outs))
        pick = lambda xs, i: xs[i] if i < len(xs) else (xs[0] if xs else "")      # noqa: E731
        return [dict(input=pick(ins, i), output=pick(outs, i), fn=fn) for i in range(n)]
    out = []
    for t in tests:                                               # livecodebench / codeforces / primeintellect
        fn = t.get("fn_name") or (t.get("metadata") or {}).get("func_name") if (t.get("testtype") == "functional" or t.get("fn_name")) else None
        out.append(dict(input=t.get("input", ""), output=t.get("output", ""), fn=fn))
    return out


def _call_args(inp):
    if isinstance(inp, str):                                      # one JSON value per line
        return [json.loads(line) for line in inp.strip().split("\n") if line.strip()]
    return list(inp) if isinstance(inp, (list, tuple)) else [inp]


def _expected(out):
    if isinstance(out, str):
        try:
            return json.loads(out)
        except json.JSONDecodeError:
            return out
    return out


def grade_cases(cases: list[dict], code: str, timeout: float = 6.0, stop_on_fail: bool = True) -> tuple[bool, dict]:
    results = []
    for c in cases:
        if c["fn"]:
            ok, out = _run(code + _CALL_HARNESS, json.dumps({"fn": c["fn"], "args": _call_args(c["input"])}), timeout)
            got = None
            if ok and "__RESULT__" in out:
                got = json.loads(out.rsplit("__RESULT__", 1)[1])
                want = _expected(c["output"])
                ok = got == want or (isinstance(want, list) and len(want) == 1 and got == want[0])
            else:
                ok = False
            results.append(dict(passed=ok, input=c["input"], expected=c["output"], output=got if got is not None else out))
        else:
            stdin = c["input"] if isinstance(c["input"], str) else "\n".join(map(str, c["input"]))
            ok, out = _run(code, stdin, timeout)
            want = c["output"] if isinstance(c["output"], str) else "\n".join(map(str, c["output"]))
            ok = ok and outputs_match(out, want)
            results.append(dict(passed=ok, input=c["input"], expected=c["output"], output=out))
        if not ok and stop_on_fail:
            break
    good = bool(results) and all(r["passed"] for r in results) and len(results) == len(cases)
    return good, {"all_passed": good, "total_tests": len(cases), "test_results": results}


def grade_script(code: str, test: str, timeout: float, files: dict | None = None) -> tuple[bool, dict]:
    ok, out = _run(test if files else code + "\n" + test, "", timeout, files)
    return ok, {"all_passed": ok, "output": out, "test_results": [{"passed": ok, "output": out}]}


_KOD_RUNNER = '''
import sys as _sys
_fails = 0
for _name, _f in sorted(list(globals().items())):
    if _name.startswith("test") and callable(_f):
        try:
            _f()
        except Exception as _e:
            _fails += 1
            print(f"{_name}: {type(_e).__name__}: {_e}")
_sys.exit(1 if _fails else 0)
'''


def grade(data_source: str, tests, code: str, timeout: float = 6.0, entry_point: str | None = None) -> tuple[bool, dict]:
    if data_source in STDIN_SOURCES:
        return grade_cases(_cases(data_source, tests), code, timeout)
    if data_source == "leetcode":
        return grade_script(code, _parse(tests)["functional"] if not isinstance(tests, dict) else tests["functional"], timeout * 2)
    if data_source == "kodcode":                                  # a test file that does `from solution import ...`
        n = max(1, str(tests).count("def test"))
        return grade_script("", str(tests) + _KOD_RUNNER, timeout * n, files={"solution.py": clean_main_block(code)})
    if data_source == "humanevalplus":                            # a body defining check(candidate)
        test = str(tests)
        if entry_point and not re.search(r"^check\(", test, re.M):
            test += f"\ncheck({entry_point})\n"
        return grade_script(clean_main_block(code), test, timeout * 4)
    raise NotImplementedError(f"code grader for data source '{data_source}' is not implemented")
