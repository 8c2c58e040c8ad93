"""Verifiers and NeMo-Gym programs against in-process fakes of the external services."""
import asyncio
import json

import httpx
import pytest

from axon_b200.programs import PROGRAM_CLASS_MAPPING
from axon_b200.programs.external import NemoGymProgram, VerifiersProgram
from axon_b200.programs.external.nemo_gym_program import build_response, task_to_messages


class _FakeRubric:
    async def score_rollout(self, state, score_sem=None):
        state["rewards"] = {"exact": 1.0 if "4" in state["completion"][-1]["content"] else 0.0, "format": 0.5}


class _FakeEnv:
    dataset = [{"question": "2+2?", "answer": "4"}, {"question": "3+3?", "answer": "6"}]
    eval_dataset = []
    rubric = _FakeRubric()

    async def rollout(self, input, client, model, sampling_args):
        msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": input["prompt"]}]
        traj = []
        for _ in range(2):
            r = await client.chat.completions.create(messages=msgs, model=model, **sampling_args)
            msgs.append({"role": "assistant", "content": r.choices[0].message.content})
            traj.append(r.model_dump())
            msgs.append({"role": "user", "content": "sure?"})
        return {"completion": msgs[2:-1], "trajectory": traj, "reward": None}


def test_verifiers_program_runs_env_rollout_through_generate():
    assert PROGRAM_CLASS_MAPPING["verifiers"] is VerifiersProgram
    p = VerifiersProgram({"env_module": "fake", "task_idx": 2}, sampling_params={"temperature": 0.3, "max_tokens": 9},
                         env_loader=lambda name, **kw: _FakeEnv())
    calls = []

    async def fake_generate(messages, sample_params=None, parser_kwargs=None):
        calls.append((len(messages), dict(sample_params)))
        return "it is 4", False, len(calls) - 1
    p.generate = fake_generate
    res = asyncio.run(p.run())
    assert [c[0] for c in calls] == [2, 4] and calls[0][1]["temperature"] == 0.3 and calls[0][1]["max_tokens"] == 9
    assert res.reward == 1.5 and res.done and res.metadata["num_turns"] == 2 and res.metadata["task_idx"] == 2
    assert res.metadata["reward_components"] == {"exact": 1.0, "format": 0.5}
    with pytest.raises(ValueError):
        VerifiersProgram({"env_module": "fake"})
    assert VerifiersProgram.extract_reward({"rewards": {"total": 0.25, "x": 9}}) == 0.25


TASK = {"id": 7, "ground_truth": "sunny", "responses_create_params": {
    "instructions": "Use tools.", "input": [{"role": "user", "content": [{"type": "input_text", "text": "Weather in Oslo?"}]}],
    "tools": [{"type": "function", "name": "get_weather", "description": "d", "strict": True,
               "parameters": {"type": "object", "properties": {"city": {"type": "string"}}, "additionalProperties": False}}]}}


def _gym(log):
    def handler(req: httpx.Request) -> httpx.Response:
        body = json.loads(req.content) if req.content else None
        log.append((req.url.path, body, req.headers.get("cookie")))
        if req.url.path == "/global_config_dict_yaml":
            return httpx.Response(200, text="weather:\n  resources_servers:\n    weather:\n      host: gym.local\n      port: 9001\nsimple_agent:\n  responses_api_agents:\n    simple_agent:\n      host: gym.local\n      port: 9002\n")
        if req.url.path == "/seed_session":
            return httpx.Response(200, json={}, headers={"set-cookie": "session=abc; Path=/"})
        if req.url.path == "/get_weather":
            return httpx.Response(200, json={"weather": "sunny", "city": body["city"]})
        if req.url.path == "/verify":
            outs = [i for i in body["response"]["output"] if i["type"] == "function_call_output"]
            return httpx.Response(200, json={"reward": 1.0 if outs and "sunny" in outs[0]["output"] and body["ground_truth"] == "sunny" else 0.0})
        if req.url.path == "/run":
            return httpx.Response(200, json={"reward": 0.75, "response": {"output": []}})
        return httpx.Response(404)
    return lambda: httpx.AsyncClient(transport=httpx.MockTransport(handler))


def test_nemo_gym_builtin_loop_tools_and_verify():
    NemoGymProgram._discovered.clear()
    msgs, tools = task_to_messages(TASK)
    assert msgs[0] == {"role": "system", "content": "Use tools."} and msgs[1]["content"] == "Weather in Oslo?"
    assert tools[0]["function"]["name"] == "get_weather" and "additionalProperties" not in tools[0]["function"]["parameters"]
    log = []
    p = NemoGymProgram({"task": TASK}, mode="builtin", head_server_url="http://head:11000", resource_server_name="weather",
                       tool_call_format="qwen", http_client_factory=_gym(log))
    replies = iter(['<tool_call>\n{"name": "get_weather", "arguments": {"city": "Oslo"}}\n</tool_call>', "It is sunny in Oslo."])

    async def fake_generate(messages, sample_params=None, parser_kwargs=None):
        assert parser_kwargs == {"tools": tools}
        return next(replies), False, 0
    p.generate = fake_generate
    res = asyncio.run(p.run())
    paths = [x[0] for x in log]
    assert paths == ["/global_config_dict_yaml", "/seed_session", "/get_weather", "/verify"]
    assert log[2][1] == {"city": "Oslo"} and log[2][2] == "session=abc"            # tool call carries the session cookie
    assert res.reward == 1.0 and res.metadata["steps"] == 2 and p.resource_server_url == "http://gym.local:9001"
    kinds = [i["type"] for i in log[3][1]["response"]["output"]]
    assert kinds == ["message", "function_call", "function_call_output", "message"] and log[3][1]["id"] == 7
    assert build_response([], TASK, tools)["tools"][0]["name"] == "get_weather"


def test_nemo_gym_native_mode_posts_task_to_agent_server():
    NemoGymProgram._discovered.clear()
    log = []
    p = NemoGymProgram({"task": TASK}, mode="native", head_server_url="http://head:11000", http_client_factory=_gym(log), endpoint_url="http://me:8000")
    p.session_id = "s-1"
    res = asyncio.run(p.run())
    assert [x[0] for x in log] == ["/global_config_dict_yaml", "/run"] and res.reward == 0.75
    assert log[1][1]["responses_create_params"]["metadata"] == {"session_id": "s-1", "policy_base_url": "http://me:8000"}
