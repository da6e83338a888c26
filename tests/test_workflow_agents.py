"""Ready-made agents (``areal_b200.workflow``): in-process through the adapter, and with the ecosystems' own SDKs
(openai, anthropic, agents) over the HTTP proxy; every model call is recorded and the reward lands on the trajectory."""
import asyncio
import os

import pytest

from areal_b200.api.cli_args import GenerationHyperparameters
from areal_b200.openai.proxy import OpenAIProxyServer
from areal_b200.rollout.workflows.agent import AgentRolloutAdapter
from areal_b200.workflow import AnthropicMathAgent, LangChainMathAgent, MathAgent, MultiTurnMathAgent, OpenAIAgentsMathAgent, math_reward
from tests.test_openai_and_agents import ByteTok, ScriptedEngine

G = GenerationHyperparameters(max_new_tokens=256)
DATA = {"messages": [{"role": "user", "content": "What is 6 * 7?"}], "answer": "42"}


def test_math_reward_reads_boxed_and_plain_answers():
    assert math_reward("so the answer is \\boxed{42}", "42") == 1.0
    assert math_reward("I think 41", "42") == 0.0 and math_reward("", "42") == 0.0 and math_reward(None, "42") == 0.0


def test_one_shot_and_multi_turn_agents_in_process():
    eng = ScriptedEngine(["The answer is \\boxed{42}"])
    traj = asyncio.run(AgentRolloutAdapter(MathAgent(max_new_tokens=32, temperature=0.5), tokenizer=ByteTok(), gconfig=G).arun_episode(eng, DATA))
    assert float(traj["rewards"][0]) == 1.0 and eng.requests[0].gconfig.max_new_tokens == 32
    # wrong, wrong, right: three calls, the feedback joins the conversation, the last attempt's reward counts
    eng = ScriptedEngine(["\\boxed{40}", "\\boxed{41}", "\\boxed{42}"])
    ad = AgentRolloutAdapter(MultiTurnMathAgent(max_turns=5, max_new_tokens=32), tokenizer=ByteTok(), gconfig=G, turn_discount=0.5)
    traj = asyncio.run(ad.arun_episode(eng, DATA))
    assert len(eng.requests) == 3 and traj["rewards"].tolist() == [0.25, 0.5, 1.0]
    assert b"carefully read the original question" in bytes(eng.requests[2].input_ids)
    eng = ScriptedEngine(["\\boxed{1}"])                      # never right: stops at max_turns with reward 0
    traj = asyncio.run(AgentRolloutAdapter(MultiTurnMathAgent(max_turns=2), tokenizer=ByteTok(), gconfig=G).arun_episode(eng, DATA))
    assert len(eng.requests) == 2 and float(traj["rewards"].sum()) == 0.0


def test_anthropic_agent_in_process():
    eng = ScriptedEngine(["\\boxed{42}"])
    traj = asyncio.run(AgentRolloutAdapter(AnthropicMathAgent(max_tokens=16, system="Be brief."), tokenizer=ByteTok(), gconfig=G).arun_episode(eng, DATA))
    assert float(traj["rewards"][0]) == 1.0 and b"Be brief." in bytes(eng.requests[0].input_ids)


def _with_proxy(eng, fn):
    px = OpenAIProxyServer(eng, ByteTok(), G, admin_key="adm").start()
    try:
        return fn(px)
    finally:
        px.stop()


def test_openai_and_anthropic_sdks_over_the_http_proxy(monkeypatch):
    pytest.importorskip("openai")
    pytest.importorskip("anthropic")
    monkeypatch.setenv("AREAL_AGENT_HTTP", "1")
    eng = ScriptedEngine(["\\boxed{41}", "\\boxed{42}", "\\boxed{42}"])

    def go(px):
        ad = AgentRolloutAdapter(MultiTurnMathAgent(max_turns=4, max_new_tokens=32), tokenizer=ByteTok(), gconfig=G, proxy=px)
        t1 = asyncio.run(ad.arun_episode(eng, DATA))
        ad2 = AgentRolloutAdapter(AnthropicMathAgent(max_tokens=16), tokenizer=ByteTok(), gconfig=G, proxy=px)
        t2 = asyncio.run(ad2.arun_episode(eng, DATA))
        return t1, t2
    t1, t2 = _with_proxy(eng, go)
    assert len(eng.requests) == 3 and t1["rewards"].tolist() == [1.0, 1.0] and t2["rewards"].tolist() == [1.0]


def test_openai_agents_sdk_drives_a_tool_loop_over_the_proxy():
    pytest.importorskip("agents")
    call = '<tool_call>\n{"name": "multiply", "arguments": {"a": 6, "b": 7}}\n</tool_call>'
    eng = ScriptedEngine([call, "The product is \\boxed{42}"])

    def go(px):
        ad = AgentRolloutAdapter(OpenAIAgentsMathAgent(max_turns=4, max_new_tokens=256), tokenizer=ByteTok(), gconfig=G, proxy=px)
        return asyncio.run(ad.arun_episode(eng, DATA))
    traj = _with_proxy(eng, go)
    assert len(eng.requests) == 2 and float(traj["rewards"][-1]) == 1.0
    assert b"42" in bytes(eng.requests[1].input_ids)                   # the tool's result went back to the model
    with pytest.raises(ValueError, match="proxy mode"):
        os.environ.pop("OPENAI_BASE_URL", None)
        asyncio.run(OpenAIAgentsMathAgent().run(DATA))


def test_langchain_agent_names_its_missing_package():
    try:
        import langchain_openai  # noqa: F401
        pytest.skip("langchain-openai is installed")
    except ImportError:
        pass
    with pytest.raises(ImportError, match="langchain-openai"):
        asyncio.run(LangChainMathAgent().run(DATA, base_url="http://127.0.0.1:1/v1", api_key="k"))


def test_http_clients_are_shared_per_event_loop():
    from areal_b200.rollout import workflow_context as wctx

    async def two():
        a, b = wctx.get_httpx_client(), wctx.get_httpx_client()
        s, t = wctx.get_aiohttp_session(), wctx.get_aiohttp_session()
        return a, b, s, t

    a, b, s, t = asyncio.run(two())
    assert a is b and s is t
    a2, _, s2, _ = asyncio.run(two())                       # another loop: the old clients died with theirs
    assert a2 is not a and s2 is not s and len(wctx._HTTP._httpx) == 1 and len(wctx._HTTP._aio) == 1

    async def closing():
        c, s_ = wctx.get_httpx_client(), wctx.get_aiohttp_session()
        await wctx.close_http_clients()
        return c.is_closed, s_.closed, wctx.get_httpx_client() is not c
    assert asyncio.run(closing()) == (True, True, True)


def test_online_workflow_turns_an_outside_users_session_into_a_trajectory():
    """Online mode: the episode is whatever an outside user did between start_session and end_session on the proxy."""
    import json
    import threading
    import urllib.request

    from areal_b200.rollout.workflows.online import OnlineSessionWorkflow

    def post(url, body, key):
        req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json", "Authorization": f"Bearer {key}"})
        with urllib.request.urlopen(req, timeout=30) as r:
            return json.loads(r.read())

    eng = ScriptedEngine(["first answer", "second answer", "third"])
    px = OpenAIProxyServer(eng, ByteTok(), G, admin_key="adm").start()
    try:
        wf = OnlineSessionWorkflow(px, turn_discount=0.5, timeout=20)
        box = {}
        t = threading.Thread(target=lambda: box.setdefault("traj", asyncio.run(wf.arun_episode(eng, {}))))
        t.start()
        root = px.base_url[:-3]
        key = post(f"{root}/rl/start_session", {}, "adm")["api_key"]
        for q in ("one", "two"):
            post(f"{px.base_url}/chat/completions", {"messages": [{"role": "user", "content": q}], "max_tokens": 32}, key)
        assert t.is_alive()                                           # still waiting: the user has not closed the session
        post(f"{root}/rl/set_reward", {"reward": 2.0}, key)
        post(f"{root}/rl/end_session", {}, key)
        t.join(timeout=20)
        traj = box["traj"]
        assert traj["rewards"].tolist() == [1.0, 2.0] and traj["input_ids"].shape[0] == 2 and len(px._sessions) == 0
        # a session that ended without a reward is dropped unless a default is configured; in-process sessions never queue
        k2 = post(f"{root}/rl/start_session", {}, "adm")["api_key"]
        post(f"{px.base_url}/chat/completions", {"messages": [{"role": "user", "content": "x"}], "max_tokens": 8}, k2)
        post(f"{root}/rl/end_session", {}, k2)
        assert asyncio.run(OnlineSessionWorkflow(px, timeout=5).arun_episode(eng, {})) is None
        px.end_session(px.start_session())
        assert asyncio.run(OnlineSessionWorkflow(px, timeout=0.2, default_reward=0.0).arun_episode(eng, {})) is None      # timeout
    finally:
        px.stop()


def test_example_reward_runs_code_in_a_remote_sandbox(monkeypatch):
    """``examples/sandbox_remote``: the completion's last python block plus the record's tests decide the reward."""
    import importlib.util

    from areal_b200.infra.sandbox import SandboxServer

    srv = SandboxServer(api_key="k").start()
    try:
        monkeypatch.setenv("AREAL_SANDBOX_ADDR", srv.address)
        monkeypatch.setenv("AREAL_SANDBOX_KEY", "k")
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        spec = importlib.util.spec_from_file_location("sandbox_reward_example", os.path.join(root, "examples", "sandbox_remote", "reward_example.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        good = "Here you go:\n```python\ndef add(a, b):\n    return a + b\n```"
        bad = "```python\ndef add(a, b):\n    return a - b\n```"
        tests = "assert add(2, 3) == 5"
        assert mod.code_reward_fn("", good, [], [], tests=tests) == 1.0
        assert mod.code_reward_fn("", bad, [], [], tests=tests) == 0.0
        assert mod.code_reward_fn("", "no code here", [], [], tests=tests) == 0.0
    finally:
        srv.stop()


def test_grouped_workflow_drops_or_keeps_incomplete_groups_and_normalises_rewards():
    import torch

    from areal_b200.api.workflow_api import RolloutWorkflow
    from areal_b200.rollout import workflow_context as wctx
    from areal_b200.rollout.workflows.rlvr import GroupedRolloutWorkflow

    class Inner(RolloutWorkflow):
        def __init__(self, rewards):
            self.rewards, self.seen = rewards, []

        async def arun_episode(self, engine, data):
            i = wctx.get().sample_idx
            self.seen.append(i)
            r = self.rewards[i]
            if r is None:
                return None
            return dict(input_ids=torch.tensor([[1, 2, 3]]), attention_mask=torch.ones(1, 3, dtype=torch.bool), loss_mask=torch.tensor([[0, 1, 1]]),
                        rewards=torch.tensor([float(r)]))

    inner = Inner([1.0, None, 3.0, 0.0])
    out = asyncio.run(GroupedRolloutWorkflow(inner, 4).arun_episode(None, {}))
    assert sorted(inner.seen) == [0, 1, 2, 3] and out["rewards"].tolist() == [1.0, 3.0, 0.0]           # variable group size
    assert asyncio.run(GroupedRolloutWorkflow(Inner([1.0, None, 3.0, 0.0]), 4, drop_incomplete_group=True).arun_episode(None, {})) is None
    assert asyncio.run(GroupedRolloutWorkflow(Inner([None] * 3), 3).arun_episode(None, {})) is None
    out = asyncio.run(GroupedRolloutWorkflow(Inner([1.0, 3.0, 1.0, 3.0]), 4, reward_normalization=True).arun_episode(None, {}))
    assert torch.allclose(out["rewards"], torch.tensor([-1.0, 1.0, -1.0, 1.0]), atol=1e-5) and out["original_rewards"].tolist() == [1.0, 3.0, 1.0, 3.0]
    assert asyncio.run(GroupedRolloutWorkflow(Inner([1.0, None]), 2, reward_normalization=True).arun_episode(None, {})) is None
    g = G.new(n_samples=3, drop_incomplete_group=True)
    w = GroupedRolloutWorkflow.from_gconfig(Inner([0.0] * 3), g)
    assert (w.group_size, w.drop_incomplete_group, w.reward_normalization) == (3, True, False)
    with pytest.raises(ValueError):
        GroupedRolloutWorkflow(Inner([]), 0)
    # serial groups start their samples strictly in order
    order = []

    class Slow(RolloutWorkflow):
        async def arun_episode(self, engine, data):
            i = wctx.get().sample_idx
            order.append(("start", i))
            await asyncio.sleep(0.01 * (3 - i))
            order.append(("end", i))
            return dict(input_ids=torch.tensor([[1]]), attention_mask=torch.ones(1, 1, dtype=torch.bool), loss_mask=torch.tensor([[1]]), rewards=torch.tensor([0.0]))

    asyncio.run(GroupedRolloutWorkflow(Slow(), 3, serialize_group_samples=True).arun_episode(None, {}))
    assert order == [("start", 0), ("end", 0), ("start", 1), ("end", 1), ("start", 2), ("end", 2)]
    order.clear()
    asyncio.run(GroupedRolloutWorkflow(Slow(), 3).arun_episode(None, {}))
    assert [o for o in order if o[0] == "start"] == [("start", 0), ("start", 1), ("start", 2)] and order[3] == ("end", 2)
