"""OpenAI-compatible client, interaction cache, HTTP proxy, agent adapter, multi-turn workflow
(CPU, scripted engine)."""
import asyncio
import json
import urllib.request

import pytest
import torch

from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig
from areal_b200.api.io_struct import ModelResponse
from areal_b200.openai import ArealOpenAI
from areal_b200.openai.proxy import OpenAIProxyServer, anthropic_to_openai
from areal_b200.openai.tool_call_parser import parse_tool_calls, split_reasoning
from areal_b200.rollout.workflows.agent import AgentRolloutAdapter
from areal_b200.rollout.workflows.multi_turn import MultiTurnWorkflow


class ByteTok:
    eos_token_id = 0
    pad_token_id = 0

    def encode(self, text):
        return list(text.encode())

    def decode(self, ids):
        return bytes(int(i) for i in ids if int(i) != 0).decode(errors="replace")


class ScriptedEngine:
    """Answers with the next scripted string; records the requests it saw."""

    def __init__(self, answers, version=3):
        self.answers, self.k, self.version, self.requests = list(answers), 0, version, []

    def get_version(self):
        return self.version

    async def agenerate(self, req):
        self.requests.append(req)
        text = self.answers[min(self.k, len(self.answers) - 1)]
        self.k += 1
        out = list(text.encode())[: req.gconfig.max_new_tokens - 1] + [0]
        return ModelResponse(input_tokens=list(req.input_ids), output_tokens=out, output_logprobs=[-0.5] * len(out),
                             output_versions=[self.version] * len(out), stop_reason="stop")


def test_client_records_tokens_rewards_and_exports_individual():
    eng, tok = ScriptedEngine(["four", "five"]), ByteTok()
    cl = ArealOpenAI(eng, tok, gconfig=GenerationHyperparameters(max_new_tokens=32))

    async def go():
        m = [{"role": "user", "content": "2+2?"}]
        c1 = await cl.chat.completions.create(messages=m, temperature=0.7, max_completion_tokens=16)
        m += [{"role": "assistant", "content": c1.choices[0].message.content}, {"role": "user", "content": "again"}]
        c2 = await cl.chat.completions.create(messages=m)
        return c1, c2
    c1, c2 = asyncio.run(go())
    assert c1.choices[0].message.content == "four" and c1.usage.completion_tokens == 5
    assert eng.requests[0].gconfig.temperature == 0.7 and eng.requests[0].gconfig.max_new_tokens == 16
    cl.set_reward(c1.id, 0.5)
    cl.set_last_reward(1.0)
    cl.apply_reward_discount(0.5)
    with pytest.raises(RuntimeError):
        cl.apply_reward_discount(0.5)
    inter = cl.export_interactions("individual")
    assert list(inter) == [c1.id, c2.id]
    assert inter[c2.id].reward == 1.0 and inter[c1.id].reward == pytest.approx(0.5 + 0.5 * 1.0)
    td = inter[c1.id].to_tensor_dict()
    n_in = len(eng.requests[0].input_ids)
    assert td["input_ids"].shape == (1, n_in + 5) and td["loss_mask"][0].tolist() == [0] * n_in + [1] * 5
    assert td["versions"][0, -1] == 3 and td["versions"][0, 0] == -1 and td["logprobs"][0, -1] == -0.5
    batch = cl.to_trajectory("individual")
    assert batch["input_ids"].shape[0] == 2 and batch["rewards"].tolist() == [1.0, 1.0]
    with pytest.raises(ValueError):   # hf template type cannot be exported as a token-exact tree
        cl.export_interactions("concat")


def test_concat_export_builds_prefix_tree():
    eng, tok = ScriptedEngine(["a1", "a2", "b2"]), ByteTok()
    cl = ArealOpenAI(eng, tok, chat_template_type="concat", gconfig=GenerationHyperparameters(max_new_tokens=8))

    async def go():
        root = [{"role": "user", "content": "q"}]
        c1 = await cl.chat.completions.create(messages=root)
        h = root + [{"role": "assistant", "content": c1.choices[0].message.content}]
        c2 = await cl.chat.completions.create(messages=h + [{"role": "user", "content": "x"}])
        c3 = await cl.chat.completions.create(messages=h + [{"role": "user", "content": "y"}])
        return c1, c2, c3
    c1, c2, c3 = asyncio.run(go())
    for c in (c2, c3):
        assert cl.get_interaction(c.id).parent is cl.get_interaction(c1.id)
    cl.set_reward(c2.id, 1.0)
    cl.set_reward(c3.id, 0.0)
    leaves = cl.export_interactions("concat")
    assert set(leaves) == {c2.id, c3.id}
    td = leaves[c2.id].to_tensor_dict()
    p = cl.get_interaction(c1.id).to_tensor_dict()
    n1 = p["input_ids"].shape[1]
    assert td["input_ids"][0, :n1].tolist() == p["input_ids"][0].tolist()       # the parent's tokens are the prefix
    assert td["loss_mask"][0, :n1].tolist() == p["loss_mask"][0].tolist()       # ... and stay trainable
    assert td["loss_mask"][0].sum() == 3 + 3                                    # "a1"+eos and "a2"+eos
    # the second request was built from the parent's exact tokens
    assert eng.requests[1].input_ids[:n1] == p["input_ids"][0].tolist()


def test_tool_calls_and_reasoning_parsing():
    tools = [{"type": "function", "function": {"name": "calc", "parameters": {}}}]
    text = 'let me see <tool_call>{"name": "calc", "arguments": {"x": 1}}</tool_call>'
    rest, calls = parse_tool_calls(text, tools)
    assert rest == "let me see" and calls[0].function.name == "calc" and json.loads(calls[0].function.arguments) == {"x": 1}
    rest, calls = parse_tool_calls('<tool_call>{"name": "other", "arguments": {}}</tool_call>', tools)
    assert not calls and "tool_call" in rest
    rest, calls = parse_tool_calls("<tool_call>{broken</tool_call>", tools)
    assert not calls
    assert split_reasoning("<think>hmm</think>answer") == ("hmm", "answer")
    eng = ScriptedEngine(['<think>t</think><tool_call>{"name": "calc", "arguments": {"x": 2}}</tool_call>'])
    cl = ArealOpenAI(eng, ByteTok(), gconfig=GenerationHyperparameters(max_new_tokens=128))
    c = asyncio.run(cl.chat.completions.create(messages=[{"role": "user", "content": "?"}], tools=tools))
    assert c.choices[0].finish_reason == "tool_calls" and c.choices[0].message.tool_calls[0].function.name == "calc"
    assert c.choices[0].message.reasoning_content == "t"


def _post(url, body, key=None):
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json",
                                 **({"Authorization": f"Bearer {key}"} if key else {})})
    try:
        with urllib.request.urlopen(req, timeout=30) as r:
            return r.status, json.loads(r.read())
    except urllib.error.HTTPError as e:
        return e.code, json.loads(e.read())


def test_http_proxy_sessions_rewards_export_and_anthropic_route():
    eng = ScriptedEngine(["hello", "world"])
    px = OpenAIProxyServer(eng, ByteTok(), GenerationHyperparameters(max_new_tokens=16), admin_key="adm").start()
    try:
        root = px.base_url[:-3]
        assert _post(f"{root}/rl/start_session", {})[0] == 401
        code, s = _post(f"{root}/rl/start_session", {}, "adm")
        key = s["api_key"]
        assert _post(f"{px.base_url}/chat/completions", {"messages": [{"role": "user", "content": "hi"}]}, "sk-bad")[0] == 401
        code, c = _post(f"{px.base_url}/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 8}, key)
        assert code == 200 and c["choices"][0]["message"]["content"] == "hello" and c["usage"]["completion_tokens"] == 6
        code, a = _post(f"{root}/v1/messages", {"system": "s", "max_tokens": 8, "messages": [
            {"role": "user", "content": [{"type": "text", "text": "hi"}]}]}, key)
        assert code == 200 and a["content"][0]["text"] == "world" and a["stop_reason"] == "end_turn"
        assert _post(f"{root}/rl/set_reward", {"reward": 2.0}, key)[0] == 200
        assert _post(f"{root}/rl/end_session", {}, key)[0] == 200
        assert _post(f"{px.base_url}/chat/completions", {"messages": []}, key)[0] == 401   # ended
        code, ex = _post(f"{root}/rl/export_trajectories", {"api_key": key, "discount": 1.0}, "adm")
        assert code == 200 and len(ex["interactions"]) == 2
        assert all(v["rewards"] == [2.0] for v in ex["interactions"].values())
    finally:
        px.stop()
    o = anthropic_to_openai({"messages": [{"role": "user", "content": [{"type": "tool_result", "tool_use_id": "t1", "content": "42"}]}],
                             "tools": [{"name": "calc", "input_schema": {"type": "object"}}]})
    assert o["messages"][0] == {"role": "tool", "tool_call_id": "t1", "content": "42"} and o["tools"][0]["function"]["name"] == "calc"


def _sse(url, body, key):
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json",
                                                                                "Authorization": f"Bearer {key}"})
    with urllib.request.urlopen(req, timeout=20) as r:
        assert r.headers["Content-Type"] == "text/event-stream"
        return r.read().decode()


def test_http_proxy_streams_chat_and_anthropic_events_and_serves_responses():
    call = '<tool_call>{"name": "calc", "arguments": {"x": 1}}</tool_call>'
    eng = ScriptedEngine(["<think>hm</think>" + "a" * 150, "let me see " + call, "plain", "resp"])
    px = OpenAIProxyServer(eng, ByteTok(), GenerationHyperparameters(max_new_tokens=512)).start()
    tools = [{"type": "function", "function": {"name": "calc", "parameters": {"type": "object"}}}]
    try:
        root = px.base_url[:-3]
        key = px.start_session()
        raw = _sse(f"{px.base_url}/chat/completions", {"messages": [{"role": "user", "content": "q"}], "stream": True}, key)
        evs = [l[6:] for l in raw.split("\n") if l.startswith("data: ")]
        assert evs[-1] == "[DONE]"
        chunks = [json.loads(e) for e in evs[:-1]]
        assert all(c["object"] == "chat.completion.chunk" and c["id"] == chunks[0]["id"] for c in chunks)
        assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
        assert "".join(c["choices"][0]["delta"].get("content", "") for c in chunks) == "a" * 150
        assert "".join(c["choices"][0]["delta"].get("reasoning_content", "") for c in chunks) == "hm"
        assert sum("content" in c["choices"][0]["delta"] and c["choices"][0]["delta"]["content"] != "" for c in chunks) == 3
        assert chunks[-1]["choices"][0]["finish_reason"] == "stop" and chunks[-1]["usage"]["completion_tokens"] > 0
        raw = _sse(f"{px.base_url}/chat/completions", {"messages": [{"role": "user", "content": "q"}], "stream": True, "tools": tools}, key)
        chunks = [json.loads(l[6:]) for l in raw.split("\n") if l.startswith("data: {")]
        tc = [c["choices"][0]["delta"]["tool_calls"][0] for c in chunks if "tool_calls" in c["choices"][0]["delta"]]
        assert len(tc) == 1 and tc[0]["function"]["name"] == "calc" and json.loads(tc[0]["function"]["arguments"]) == {"x": 1}
        assert chunks[-1]["choices"][0]["finish_reason"] == "tool_calls"
        raw = _sse(f"{root}/v1/messages", {"max_tokens": 8, "stream": True, "messages": [{"role": "user", "content": "hi"}]}, key)
        names = [l[7:] for l in raw.split("\n") if l.startswith("event: ")]
        assert names[0] == "message_start" and names[-2:] == ["message_delta", "message_stop"] and "content_block_delta" in names
        text = "".join(json.loads(l[6:])["delta"]["text"] for l in raw.split("\n")
                       if l.startswith("data: ") and json.loads(l[6:]).get("type") == "content_block_delta")
        assert text == "plain"
        code, r = _post(f"{px.base_url}/responses", {"input": "hello", "instructions": "be brief", "max_output_tokens": 16}, key)
        assert code == 200 and r["object"] == "response" and r["output_text"] == "resp" and r["output"][0]["type"] == "message"
        # the four calls were all recorded for training
        assert len(px.pop_session(key).client.export_interactions("individual")) == 4
    finally:
        px.stop()


def test_tool_call_parsers_by_format():
    from areal_b200.openai.tool_call_parser import parse_tool_calls

    tools = [{"type": "function", "function": {"name": "run", "parameters": {"type": "object", "properties": {
        "code": {"type": "string"}, "n": {"type": "integer"}, "ok": {"type": "boolean"}, "xs": {"type": "array"}, "r": {"type": "number"}}}}}]
    coder = ("I will run it\n<tool_call>\n<function=run>\n<parameter=code>\nprint(1)\n</parameter>\n<parameter=n>3</parameter>\n"
             "<parameter=ok>True</parameter><parameter=xs>[1, 2]</parameter><parameter=r>0.5</parameter>\n</function>\n</tool_call>")
    rest, calls = parse_tool_calls(coder, tools, "qwen3_coder")
    assert rest == "I will run it" and len(calls) == 1 and calls[0].function.name == "run"
    assert json.loads(calls[0].function.arguments) == {"code": "print(1)", "n": 3, "ok": True, "xs": [1, 2], "r": 0.5}
    # unknown tool: left in the text; auto picks the format that matches
    assert parse_tool_calls(coder.replace("function=run", "function=zzz"), tools, "qwen3_coder") == (coder.replace("function=run", "function=zzz"), [])
    assert parse_tool_calls(coder, tools, "auto")[1][0].function.name == "run"
    assert parse_tool_calls('<tool_call>{"name": "run", "arguments": {"n": 1}}</tool_call>', tools, "auto")[1][0].function.name == "run"
    rest, calls = parse_tool_calls('```json\n[{"name": "run", "parameters": {"n": 2}}, {"name": "run", "arguments": {"n": 3}}]\n```', tools, "json")
    assert rest == "" and [json.loads(c.function.arguments)["n"] for c in calls] == [2, 3]
    assert parse_tool_calls('{"name": "other", "arguments": {}}', tools, "json")[1] == []
    assert parse_tool_calls("no call here", tools, "auto") == ("no call here", [])
    with pytest.raises(ValueError):
        parse_tool_calls("x", tools, "nope")


class EchoAgent:
    tokenizer = ByteTok()
    gconfig = GenerationHyperparameters(max_new_tokens=8)

    async def run(self, data, client):
        c1 = await client.chat.completions.create(messages=[{"role": "user", "content": data["q"]}])
        c2 = await client.chat.completions.create(messages=[{"role": "user", "content": data["q"] + "!"}])
        return {c1.id: 0.25, c2.id: 1.0} if data.get("per_call") else (None if data.get("reject") else 1.0)


def test_agent_adapter_and_executor_resolution():
    from areal_b200.rollout.executor import WorkflowExecutor

    eng = ScriptedEngine(["x", "y"])
    ad = AgentRolloutAdapter(EchoAgent(), turn_discount=0.5)
    traj = asyncio.run(ad.arun_episode(eng, {"q": "a"}))
    assert traj["input_ids"].shape[0] == 2 and traj["rewards"].tolist() == [0.5, 1.0]
    traj = asyncio.run(AgentRolloutAdapter(EchoAgent()).arun_episode(ScriptedEngine(["x"]), {"q": "a", "per_call": True}))
    assert traj["rewards"].tolist() == [1.25, 1.0]
    assert asyncio.run(AgentRolloutAdapter(EchoAgent()).arun_episode(ScriptedEngine(["x"]), {"q": "a", "reject": True})) is None
    ex = WorkflowExecutor(InferenceEngineConfig(consumer_batch_size=1, max_concurrent_rollouts=2), eng)
    assert isinstance(ex._resolve_workflow(EchoAgent(), None), AgentRolloutAdapter)


def test_multi_turn_retries_with_discount_and_masks_feedback():
    tok = ByteTok()

    def reward(prompt, completion, pids, cids, **kw):
        return 1.0 if "right" in completion else 0.0
    g = GenerationHyperparameters(max_new_tokens=16, max_tokens=512)
    wf = MultiTurnWorkflow(reward, g, tok, max_turns=3, turn_discount=0.5, reward_in_process=True)
    eng = ScriptedEngine(["wrong", "right"])
    t = asyncio.run(wf.arun_episode(eng, {"input_ids": tok.encode("q?")}))
    assert t["rewards"].item() == 0.5 and len(eng.requests) == 2
    fb = len(wf._encode_feedback())
    assert int(t["loss_mask"].sum()) == 6 + 6                    # two answers (+eos), feedback and prompt masked out
    assert t["input_ids"].shape[1] == 2 + 6 + fb + 6
    assert eng.requests[1].input_ids == t["input_ids"][0, : 2 + 6 + fb].tolist()
    t = asyncio.run(wf.arun_episode(ScriptedEngine(["no", "no", "no"]), {"input_ids": tok.encode("q?")}))
    assert t["rewards"].item() == 0.0
    t = asyncio.run(wf.arun_episode(ScriptedEngine(["right"]), {"input_ids": tok.encode("q?")}))
    assert t["rewards"].item() == 1.0


class _ByteTokenizer:
    vocab_size = 256
    eos_token_id = 0

    def encode(self, text):
        return list(text.encode())

    def decode(self, ids):
        return bytes(int(i) for i in ids).decode(errors="replace")


def test_tir_workflow_runs_code_and_masks_tool_output():
    """Tool-integrated reasoning: a scripted engine writes a python block, the sandbox runs it,
    the output block is appended with loss mask 0, and generation continues to the answer."""
    import asyncio

    from areal_b200.api.cli_args import GenerationHyperparameters
    from areal_b200.api.io_struct import ModelResponse
    from areal_b200.rollout.workflows.tir import TIRWorkflow

    tok = _ByteTokenizer()
    scripted = ["Let me compute.\n```python\nprint(6*7)\n```\n", "So the answer is 42."]
    seen_prompts = []

    class Engine:
        def get_version(self):
            return 3

        async def agenerate(self, req):
            seen_prompts.append(tok.decode(req.input_ids))
            assert req.gconfig.stop == ["```\n"]
            text = scripted[len(seen_prompts) - 1]
            ids = tok.encode(text)
            return ModelResponse(input_tokens=list(req.input_ids), output_tokens=ids, output_logprobs=[-0.5] * len(ids),
                                 output_versions=[3] * len(ids), stop_reason="stop")

    def reward(prompt, completion, prompt_ids, completion_ids, answer=None, **kw):
        return float(completion.strip().endswith(str(answer) + "."))

    wf = TIRWorkflow(reward, GenerationHyperparameters(max_new_tokens=200, max_tokens=600), tok, max_tool_calls=2)
    out = asyncio.run(wf.arun_episode(Engine(), {"input_ids": tok.encode("What is 6*7? "), "answer": 42}))
    assert len(seen_prompts) == 2 and "```output\n42\n```" in seen_prompts[1]
    ids, lm = out["input_ids"][0].tolist(), out["loss_mask"][0].tolist()
    text = tok.decode(ids)
    assert text.endswith("So the answer is 42.") and out["rewards"].item() == 1.0
    tool = "\n```output\n42\n```\n"
    a = text.index(tool)
    assert all(m == 0 for m in lm[a:a + len(tool)])                      # tool text is not trained on
    n_prompt = len(tok.encode("What is 6*7? "))
    assert all(m == 0 for m in lm[:n_prompt]) and sum(lm) == len(tok.encode(scripted[0])) + len(tok.encode(scripted[1]))
    assert out["versions"][0][a].item() == -1 and out["versions"][0][-1].item() == 3
    assert TIRWorkflow.pending_code("text ```python\nx=1\n```") == "x=1" and TIRWorkflow.pending_code("no code") is None


def test_engine_stops_on_stop_strings():
    import asyncio

    from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeInferConfig
    from areal_b200.api.io_struct import ModelRequest
    from areal_b200.engine.infer_engine import NativeInferenceEngine
    from areal_b200.models.config import preset

    tok = _ByteTokenizer()
    eng = NativeInferenceEngine(InferenceEngineConfig(), NativeInferConfig(max_running_requests=2, context_length=128),
                                model_config=preset("tiny-qwen2", vocab_size=tok.vocab_size, num_layers=1))
    eng.initialize(device="cpu", start_executor=False)
    try:
        g = GenerationHyperparameters(max_new_tokens=40, max_tokens=100, greedy=True, ignore_eos=True)
        free = asyncio.run(eng.agenerate(ModelRequest(rid="a", input_ids=tok.encode("12+3="), gconfig=g, tokenizer=tok)))
        text = tok.decode(free.output_tokens)
        assert len(free.output_tokens) == 40
        stop = text[5:7]                                   # a two-character string the greedy continuation is known to contain
        r = asyncio.run(eng.agenerate(ModelRequest(rid="b", input_ids=tok.encode("12+3="), gconfig=g.new(stop=[stop]), tokenizer=tok)))
        got = tok.decode(r.output_tokens)
        assert r.stop_reason == "stop" and got.endswith(stop) and len(r.output_tokens) == text.index(stop) + 2
    finally:
        eng.destroy()


def test_search_agent_example_calls_tool_then_answers():
    import importlib.util
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "search_agent", "train.py")
    spec = importlib.util.spec_from_file_location("search_agent_example", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.LocalSearch().query("Danube sea")[0].startswith("The Danube")
    assert mod.answer_reward("<answer>The Black Sea</answer>", "black sea") == 1.0 and mod.answer_reward("Black Sea", "black sea") == 0.0
    eng = ScriptedEngine(['<tool_call>{"name": "search", "arguments": {"query": "Danube empties sea"}}</tool_call>',
                          "<answer>Black Sea</answer>"])
    ad = AgentRolloutAdapter(mod.SearchAgent(), tokenizer=ByteTok(), gconfig=GenerationHyperparameters(max_new_tokens=200), turn_discount=0.5)
    traj = asyncio.run(ad.arun_episode(eng, mod.dataset(1)[0]))
    assert traj["input_ids"].shape[0] == 2 and traj["rewards"].tolist() == [0.5, 1.0]
    # the second request saw the retrieved passage as a tool message
    second_prompt = ByteTok().decode(eng.requests[1].input_ids)
    assert "Black Sea" in second_prompt and "Danube" in second_prompt


def test_openai_agents_example_runs_a_function_call_round_trip():
    import importlib.util
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "openai_agents", "calculator_agent.py")
    spec = importlib.util.spec_from_file_location("calculator_agent_example", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.safe_eval("(17+72)*2") == 178
    with pytest.raises(Exception):
        mod.safe_eval("__import__('os').getcwd()")
    eng = ScriptedEngine(['<tool_call>{"name": "calculate", "arguments": {"expression": "17+72"}}</tool_call>', "Answer: 89"])
    ad = AgentRolloutAdapter(mod.CalculatorAgent(), tokenizer=ByteTok(), gconfig=GenerationHyperparameters(max_new_tokens=200))
    traj = asyncio.run(ad.arun_episode(eng, {"question": "What is 17+72?", "answer": 89}))
    assert traj["input_ids"].shape[0] == 2 and traj["rewards"].tolist()[-1] == 1.0
    assert "89" in ByteTok().decode(eng.requests[1].input_ids)            # the tool result reached the second call


def test_proxy_gateway_spreads_sessions_and_relays_to_the_owner():
    """Two proxies behind one address: sessions open on the emptier proxy, later requests (streamed ones too) reach
    the proxy that owns the key, exporting closes the mapping, unknown keys and a wrong admin key are refused."""
    from areal_b200.openai.proxy_gateway import ProxyGateway

    g = GenerationHyperparameters(max_new_tokens=16)
    pa = OpenAIProxyServer(ScriptedEngine(["from-a"] * 4), ByteTok(), g, admin_key="adm").start()
    pb = OpenAIProxyServer(ScriptedEngine(["from-b"] * 4), ByteTok(), g, admin_key="adm").start()
    gw = ProxyGateway([pa.base_url, pb.base_url], admin_api_key="adm").start()
    try:
        assert _post(f"{gw.addr}/rl/start_session", {}, "nope")[0] == 401
        k1 = _post(f"{gw.addr}/rl/start_session", {}, "adm")[1]
        k2 = _post(f"{gw.addr}/rl/start_session", {}, "adm")[1]
        assert k1["base_url"] == gw.base_url and gw.sessions() == [1, 1]
        msg = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 8}
        r1 = _post(f"{gw.base_url}/chat/completions", msg, k1["api_key"])[1]["choices"][0]["message"]["content"]
        r2 = _post(f"{gw.base_url}/chat/completions", msg, k2["api_key"])[1]["choices"][0]["message"]["content"]
        assert {r1, r2} == {"from-a", "from-b"}
        raw = _sse(f"{gw.base_url}/chat/completions", {**msg, "stream": True}, k1["api_key"])
        text = "".join(json.loads(l[6:])["choices"][0]["delta"].get("content", "") for l in raw.split("\n") if l.startswith("data: {"))
        assert text == r1 and raw.rstrip().endswith("data: [DONE]")
        assert _post(f"{gw.base_url}/chat/completions", msg, "sk-unknown")[0] == 401
        assert _post(f"{gw.addr}/rl/set_reward", {"reward": 1.0}, k1["api_key"])[0] == 200
        assert _post(f"{gw.addr}/rl/end_session", {}, k1["api_key"])[0] == 200
        code, ex = _post(f"{gw.addr}/rl/export_trajectories", {"api_key": k1["api_key"], "discount": 1.0}, "adm")
        assert code == 200 and len(ex["interactions"]) == 2 and all(v["rewards"] == [1.0] for v in ex["interactions"].values())
        assert sorted(gw.sessions()) == [0, 1]
        assert _post(f"{gw.addr}/rl/export_trajectories", {"api_key": k1["api_key"]}, "adm")[0] == 401
        k3 = _post(f"{gw.addr}/rl/start_session", {}, "adm")[1]     # lands on the proxy that just emptied
        r3 = _post(f"{gw.base_url}/chat/completions", msg, k3["api_key"])[1]["choices"][0]["message"]["content"]
        assert r3 == r1
        code, h = 200, json.loads(urllib.request.urlopen(f"{gw.addr}/health", timeout=10).read())
        assert h["open_sessions"] == [1, 1]
    finally:
        gw.stop(); pa.stop(); pb.stop()


def test_anthropic_shaped_client_records_turns_with_tools():
    from areal_b200.openai.anthropic_client import ArealAnthropic

    call_text = 'sure <tool_call>{"name": "calc", "arguments": {"x": 2}}</tool_call>'
    eng = ScriptedEngine([call_text, "the answer is 4"])
    cl = ArealAnthropic(eng, ByteTok(), gconfig=GenerationHyperparameters(max_new_tokens=64))
    tools = [{"name": "calc", "description": "doubles", "input_schema": {"type": "object", "properties": {"x": {"type": "integer"}}}}]

    async def episode():
        r1 = await cl.messages.create(model="m", max_tokens=128, system="be terse", tools=tools,
                                      messages=[{"role": "user", "content": "double 2"}])
        assert r1.stop_reason == "tool_use" and r1.content[-1].type == "tool_use" and r1.content[-1].input == {"x": 2}
        r2 = await cl.messages.create(model="m", max_tokens=32, system="be terse", tools=tools, messages=[
            {"role": "user", "content": "double 2"},
            {"role": "assistant", "content": [{"type": "tool_use", "id": r1.content[-1].id, "name": "calc", "input": {"x": 2}}]},
            {"role": "user", "content": [{"type": "tool_result", "tool_use_id": r1.content[-1].id, "content": "4"}]}])
        assert r2.stop_reason == "end_turn" and r2.content[0].text == "the answer is 4" and r2.usage.output_tokens > 0
        cl.set_last_reward(1.0)
        return r1, r2
    r1, r2 = asyncio.run(episode())
    inter = cl.export_interactions("individual", reward_discount=0.5)
    assert set(inter) == {r1.id, r2.id} and inter[r2.id].reward == 1.0 and inter[r1.id].reward == 0.5
    batch = cl.to_trajectory("individual")
    assert batch["input_ids"].shape[0] == 2 and batch["loss_mask"].sum() > 0
    with pytest.raises(NotImplementedError):
        asyncio.run(cl.messages.create(messages=[], max_tokens=1, stream=True))
