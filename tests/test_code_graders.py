"""Code rewards per data source: each dataset format of the reference graded on a right and a wrong answer."""
import json

import pytest

from axon_b200.utils.rewards import code_reward_fn
from axon_b200.utils.rewards.code_graders import clean_main_block, outputs_match


def _ans(code):
    return f"thinking...\n```python\n{code}\n```"


ADD_STDIN = "a, b = map(int, input().split())\nprint(a + b)"
ADD_STDIN_BAD = "a, b = map(int, input().split())\nprint(a - b)"
ADD_FN = "def add(a, b):\n    return a + b"
ADD_FN_BAD = "def add(a, b):\n    return a * b"
ADD_CLS = "class Solution:\n    def add(self, a, b):\n        return a + b"


@pytest.mark.parametrize("source,tests,good,bad", [
    ("taco", {"inputs": ["1 2\n", "5 7\n"], "outputs": ["3\n", "12\n"]}, ADD_STDIN, ADD_STDIN_BAD),
    ("apps", {"inputs": [[1, 2], [5, 7]], "outputs": [[3], [12]], "fn_name": "add"}, ADD_FN, ADD_FN_BAD),
    ("primeintellect", str([{"input": "1 2", "output": "3"}, {"input": "2 2", "output": "4"}]), ADD_STDIN, ADD_STDIN_BAD),
    ("livecodebench", json.dumps([{"input": "1 2", "output": "3", "testtype": "stdin"}]), ADD_STDIN, ADD_STDIN_BAD),
    ("livecodebench", [{"input": "1\n2", "output": "3", "testtype": "functional", "metadata": {"func_name": "add"}}], ADD_CLS, ADD_FN_BAD),
    ("codeforces", [{"input": "3 4", "output": "7.0000001"}], "a, b = map(int, input().split())\nprint(float(a + b))", ADD_STDIN_BAD),
    ("leetcode", {"functional": "assert add(1, 2) == 3\nassert add(2, 2) == 4"}, ADD_FN, ADD_FN_BAD),
    ("kodcode", "from solution import add\n\ndef test_small():\n    assert add(1, 2) == 3\n\ndef test_big():\n    assert add(20, 22) == 42\n",
     ADD_FN + "\n\nif __name__ == '__main__':\n    raise SystemExit(1)", ADD_FN_BAD),
    ("humanevalplus", "def check(candidate):\n    assert candidate(1, 2) == 3\n    assert candidate(3, 3) == 6\n", ADD_FN, ADD_FN_BAD),
])
def test_each_data_source_separates_right_from_wrong(source, tests, good, bad):
    info = {"data_source": source, "ground_truth": tests, "entry_point": "add"}
    ok = code_reward_fn(info, _ans(good))
    assert ok.is_correct and ok.reward == 1.0, ok.metadata
    no = code_reward_fn(info, _ans(bad))
    assert not no.is_correct and no.metadata["test_results"], no.metadata


def test_helpers_and_errors():
    assert outputs_match("1  2\n3 \n", "1 2\n3") and not outputs_match("1 2", "1 3") and outputs_match("0.30000001", "0.3")
    assert clean_main_block("x = 1\nif __name__ == \"__main__\":\n    main()\n") == "x = 1\n"
    slow = code_reward_fn({"data_source": "taco", "ground_truth": {"inputs": ["1 2"], "outputs": ["3"]}},
                          _ans("while True:\n    pass"), None)
    assert not slow.is_correct
    with pytest.raises(NotImplementedError):
        code_reward_fn({"data_source": "nosuchset", "ground_truth": [1]}, _ans(ADD_FN))
    assert not code_reward_fn({"data_source": "taco", "ground_truth": {"inputs": ["1"], "outputs": ["1"]}}, "no code here").is_correct
