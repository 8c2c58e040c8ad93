"""The shipped recipes: FrozenLake dynamics and agent parsing, the math environment's scoring, the data scripts, and a
ReactProgram episode of each recipe against a scripted model."""
import asyncio
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_frozenlake_maps_are_solvable_and_deterministic():
    from recipes.frozenlake.env import FrozenLakeEnv, generate_random_map, reachable
    for seed in range(20):
        m = generate_random_map(size=6, p=0.7, seed=seed)
        assert m == generate_random_map(size=6, p=0.7, seed=seed)
        assert sum(r.count("S") for r in m) == 1 and sum(r.count("G") for r in m) == 1
        assert reachable([list(r) for r in m], 5)
    env = FrozenLakeEnv(desc=["SFF", "FHF", "FFG"], max_steps=5)
    obs, _ = env.reset()
    assert obs.splitlines()[0].split() == ["P", "_", "_"]
    _, r, done, info = env.step(4)                     # up against the border: stays
    assert (r, done, info["action_is_effective"]) == (0.0, False, False)
    _, r, done, _ = env.step(3)
    _, r, done, _ = env.step(3)
    obs, r, done, _ = env.step(2)
    assert (r, done) == (0.0, False)
    obs, r, done, _ = env.step(2)
    assert (r, done) == (1.0, True) and "√" in obs
    env.reset()
    env.step(2)
    obs, r, done, _ = env.step(3)                      # into the hole
    assert (r, done) == (0.0, True) and "X" in obs
    env.reset()
    outs = [env.step(0) for _ in range(5)]             # unparsable answers use up the turns
    assert [o[2] for o in outs] == [False] * 4 + [True]


def test_frozenlake_agent_reads_the_last_fenced_move():
    from recipes.frozenlake.agent import FrozenLakeAgent
    a = FrozenLakeAgent()
    assert a.process_action("<think>go</think> first ```Up``` then ```Right```").action == 3
    assert a.process_action("```2```").action == 2
    assert a.process_action("I move ```to the left```").action == 1
    assert a.process_action("no block here").action == 0
    assert "goal" in a.system_prompt.lower()
    first = a.process_observation(" P  _ ", 0.0, False, {})
    again = a.process_observation(" P  _ ", 0.0, False, {})
    assert "no effect" in again and "no effect" not in first


def test_data_scripts_write_rows(tmp_path):
    out = tmp_path / "fl"
    subprocess.run([sys.executable, os.path.join(ROOT, "recipes/frozenlake/data.py"), "--train_size", "7", "--test_size", "3",
                    "--out", str(out)], check=True, capture_output=True, cwd=ROOT)
    import pandas as pd
    df = pd.read_parquet(out / "train.parquet")
    assert len(df) == 7 and set(df.iloc[0]["env_args"]) >= {"seed", "size", "p"}
    src = tmp_path / "q.jsonl"
    src.write_text(json.dumps({"question": "1+1?", "answer": "so #### 2"}) + "\n")
    subprocess.run([sys.executable, os.path.join(ROOT, "recipes/math/data.py"), "--input", str(src), "--out", str(tmp_path / "m.parquet")],
                   check=True, capture_output=True, cwd=ROOT)
    row = pd.read_parquet(tmp_path / "m.parquet").iloc[0]
    assert row["ground_truth"] == "2" and row["env_name"] == "math"


class _Scripted:
    """Stands in for the engine: answers with the next scripted response."""

    def __init__(self, replies):
        self.replies, self.calls = list(replies), []

    async def __call__(self, messages, sample_params=None, **kw):
        self.calls.append(messages)
        return self.replies.pop(0), False, None


@pytest.mark.parametrize("recipe", ["frozenlake", "math"])
def test_react_program_runs_an_episode_of_each_recipe(recipe):
    from axon_b200.programs.react_program import ReactProgram
    if recipe == "frozenlake":
        prog = ReactProgram(agent_name=os.path.join(ROOT, "recipes/frozenlake/agent.py") + ":FrozenLakeAgent",
                            env_name=os.path.join(ROOT, "recipes/frozenlake/env.py") + ":FrozenLakeEnv",
                            env_args={"desc": ["SF", "FG"], "max_steps": 5})
        script = _Scripted(["```Right```", "<think>nearly</think>```Down```"])
    else:
        prog = ReactProgram(agent_name=os.path.join(ROOT, "recipes/math/agent.py") + ":MathAgent",
                            env_name=os.path.join(ROOT, "recipes/math/env.py") + ":MathEnvironment",
                            env_args={"question": "What is 6 * 7?", "ground_truth": "42"})
        script = _Scripted(["6 * 7 = 42, so \\boxed{42}"])
    prog.generate = script
    res = asyncio.run(prog.run())
    assert res.reward == 1.0 and res.done
    assert script.calls[0][-1]["role"] == "user" and not script.replies


def test_launch_files_compose_and_pass_the_configuration_check():
    """Every shell launch file hands ``axon train`` a list of overrides that composes and validates."""
    import glob
    import re
    from axon_b200.config.validate_config import validate_axon_config
    from axon_b200.utils.config import compose_config
    files = sorted(glob.glob(os.path.join(ROOT, "recipes", "*", "*.sh")))
    assert len(files) >= 4
    for f in files:
        txt = open(f).read()
        body = txt[txt.index("axon train --fg --") + len("axon train --fg --"):]
        body = body.replace("\\\n", " ").replace('"$@"', "").replace("${ROOT}", ROOT)
        overrides = [t.strip('"') for t in re.findall(r'(?:"[^"]*"|\S+)', body) if "=" in t]
        validate_axon_config(compose_config(overrides))
