"""HTTP inference server + remote client engine on CPU (tiny model)."""
import asyncio
import sys
import threading
import time

import pytest
import torch

from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeInferConfig
from areal_b200.api.io_struct import ModelRequest, SaveLoadMeta, WeightUpdateMeta
from areal_b200.engine.infer_engine import NativeInferenceEngine
from areal_b200.engine.remote_engine import RemoteInfEngine
from areal_b200.engine.server import InferenceServer, gconfig_from_sampling_params
from areal_b200.models import hf_io
from areal_b200.models.config import preset
from areal_b200.models.decoder import build_model


@pytest.fixture()
def served():
    mc = preset("tiny-qwen2", vocab_size=64, num_layers=2)
    engs, srvs = [], []
    for i in range(2):
        e = NativeInferenceEngine(InferenceEngineConfig(), NativeInferConfig(), model_config=mc)
        e.initialize(device="cpu", seed=1, start_executor=False)
        engs.append(e)
        srvs.append(InferenceServer(e).start())
    yield mc, engs, srvs
    for s in srvs:
        s.stop()
    for e in engs:
        e.destroy()


def test_sampling_params_mapping():
    g = gconfig_from_sampling_params({"temperature": 0.0, "max_new_tokens": 5, "top_k": -1, "stop_token_ids": [3]})
    assert g.greedy and g.max_new_tokens == 5 and g.top_k >= 10 ** 7 and g.stop_token_ids == [3]


def test_remote_generation_matches_local_and_round_robins(served):
    mc, engs, srvs = served
    cl = RemoteInfEngine(InferenceEngineConfig(setup_timeout=20), [s.address for s in srvs]).initialize(start_executor=False)
    g = GenerationHyperparameters(max_new_tokens=6, greedy=True, max_tokens=64)
    prompts = [[1, 2, 3, 4], [5, 6, 7], [9, 9, 1, 2, 3]]

    async def both():
        remote = await asyncio.gather(*[cl.agenerate(ModelRequest(rid=f"r{i}", input_ids=p, gconfig=g)) for i, p in enumerate(prompts)])
        local = await asyncio.gather(*[engs[0].agenerate(ModelRequest(input_ids=p, gconfig=g)) for p in prompts])
        return remote, local
    remote, local = asyncio.run(both())
    for r, l in zip(remote, local):
        assert r.output_tokens == l.output_tokens and r.stop_reason == l.stop_reason
        assert r.output_logprobs == pytest.approx(l.output_logprobs, abs=1e-5) and len(r.output_versions) == r.output_len
    assert cl.choose_server("r0") == srvs[0].address and cl.choose_server("r1") == srvs[1].address   # affinity + round robin
    cl.destroy()


def test_remote_weight_update_from_disk_pause_and_versions(served, tmp_path):
    mc, engs, srvs = served
    cl = RemoteInfEngine(InferenceEngineConfig(setup_timeout=20), [s.address for s in srvs]).initialize(start_executor=False)
    other = build_model(mc, dtype=torch.float32, device="cpu", seed=7)
    hf_io.save_model_hf(other, str(tmp_path / "ckpt"))
    cl.pause_generation()
    cl.update_weights_from_disk(WeightUpdateMeta(type="disk", path=str(tmp_path / "ckpt"), version=4)).result(timeout=60)
    cl.set_version(4)
    cl.continue_generation()
    assert cl.get_version() == 4 and all(e.get_version() == 4 for e in engs)
    k, v = next(iter(other.named_parameters()))
    assert torch.allclose(dict(engs[1].model.named_parameters())[k], v)
    g = GenerationHyperparameters(max_new_tokens=4, greedy=True, max_tokens=64)
    r = asyncio.run(cl.agenerate(ModelRequest(input_ids=[1, 2, 3], gconfig=g)))
    assert r.output_versions == [4] * r.output_len
    cl.destroy()


def test_generation_interrupted_by_pause_is_resumed_with_new_version(served):
    mc, engs, srvs = served
    cl = RemoteInfEngine(InferenceEngineConfig(setup_timeout=20), [srvs[0].address]).initialize(start_executor=False)
    g = GenerationHyperparameters(max_new_tokens=48, greedy=True, max_tokens=128, ignore_eos=True)

    def bump():
        time.sleep(0.15)
        cl.pause_generation()
        cl.set_version(9)
        cl.continue_generation()
    t = threading.Thread(target=bump)
    t.start()
    r = asyncio.run(cl.agenerate(ModelRequest(input_ids=[1, 2, 3, 4, 5], gconfig=g)))
    t.join()
    assert r.output_len == 48 and len(r.output_versions) == 48 and r.stop_reason == "length"
    assert set(r.output_versions) <= {0, 9} and r.output_versions == sorted(r.output_versions)
    cl.destroy()


def _fake_server(routes):
    """A tiny HTTP server: ``routes[path](body) -> dict``; records every (path, body)."""
    import json
    import threading
    from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

    from areal_b200.utils.network import find_free_ports

    seen = []

    class H(BaseHTTPRequestHandler):
        def log_message(self, *a):
            pass

        def _do(self):
            n = int(self.headers.get("Content-Length", "0"))
            body = json.loads(self.rfile.read(n)) if n else {}
            seen.append((self.path, body))
            fn = routes.get(self.path)
            out = json.dumps(fn(body) if fn else {"error": "no route"}).encode()
            self.send_response(200 if fn else 404)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(out)))
            self.end_headers()
            self.wfile.write(out)
        do_POST = do_GET = _do

    port = find_free_ports(1)[0]
    srv = ThreadingHTTPServer(("127.0.0.1", port), H)
    srv.daemon_threads = True
    threading.Thread(target=srv.serve_forever, daemon=True).start()
    return srv, f"127.0.0.1:{port}", seen


def test_sglang_wire_format_and_version_of_the_request_in_flight():
    """An SGLang-style server: the request carries ``sampling_params`` / ``sampling_seed`` / ``stop``, the answer's
    (logprob, token, text) triples are read back, an abort before prefill is retried, and the tokens are tagged with the
    weight version that was current when the request LEFT, although an update lands while it is in flight."""
    import asyncio

    from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig
    from areal_b200.api.io_struct import ModelRequest
    from areal_b200.engine.remote_engine import RemoteInfEngine

    state = {"calls": 0}
    box = {}

    def generate(body):
        state["calls"] += 1
        if state["calls"] == 1:
            return {"meta_info": {"finish_reason": {"type": "abort", "message": "Abort before prefill: paused"}}}
        box["eng"]._version = 11                      # the weight update lands while this request is being served
        return {"meta_info": {"finish_reason": {"type": "stop", "matched": 7},
                              "output_token_logprobs": [[-0.5, 4, "a"], [-0.25, 5, "b"], [-1.0, 7, None]]}}
    srv, addr, seen = _fake_server({"/generate": generate, "/pause_generation": lambda b: {}, "/continue_generation": lambda b: {},
                                    "/release_memory_occupation": lambda b: {}, "/update_weights_from_disk": lambda b: {"success": True}})
    try:
        eng = RemoteInfEngine(InferenceEngineConfig(request_retries=1), [addr], backend="sglang")
        box["eng"] = eng
        eng._version = 10
        g = GenerationHyperparameters(max_new_tokens=8, max_tokens=64, temperature=0.7, top_p=0.9, seed=3, stop=["\n\n"])
        r = asyncio.run(eng.agenerate(ModelRequest(rid="r0", input_ids=[1, 2], gconfig=g)))
        assert r.output_tokens == [4, 5, 7] and r.output_logprobs == [-0.5, -0.25, -1.0] and r.stop_reason == "stop"
        assert r.output_versions == [10, 10, 10] and eng.get_version() == 11
        body = [b for p, b in seen if p == "/generate"][-1]
        assert body["input_ids"] == [1, 2] and body["return_logprob"] is True and body["stream"] is False
        sp = body["sampling_params"]
        assert sp["temperature"] == 0.7 and sp["top_p"] == 0.9 and sp["sampling_seed"] == 3 and sp["stop"] == ["\n\n"] and sp["max_new_tokens"] == 8
        eng.set_version(12)                            # no such route on an SGLang server: nothing is sent
        assert not [p for p, _ in seen if p == "/set_version"] and eng.get_version() == 12
        eng.pause_generation(); eng.continue_generation(); eng.offload()
        assert [p for p, _ in seen][-3:] == ["/pause_generation", "/continue_generation", "/release_memory_occupation"]
    finally:
        srv.shutdown()


def test_vllm_wire_format_and_control_routes():
    import asyncio

    from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig
    from areal_b200.api.io_struct import ModelRequest, ParamSpec, WeightUpdateMeta
    from areal_b200.engine.remote_backends import get_backend
    from areal_b200.engine.remote_engine import RemoteInfEngine

    def completions(body):
        n = body["max_tokens"]
        toks = [40, 41, 42][:n]
        return {"choices": [{"finish_reason": "length" if n <= 3 else "stop",
                             "logprobs": {"tokens": [f"token_id:{t}" for t in toks], "token_logprobs": [-0.1 * (i + 1) for i in range(len(toks))]}}]}
    ok = lambda b: {"status": "ok"}                      # noqa: E731
    srv, addr, seen = _fake_server({"/v1/completions": completions, "/areal_pause_generation": ok, "/areal_continue_generation": ok,
                                    "/areal_update_weights": ok, "/areal_set_update_weight_meta": ok, "/areal_update_weights_xccl": ok,
                                    "/areal_init_weights_update_group": ok, "/sleep": ok, "/wake_up": ok})
    try:
        eng = RemoteInfEngine(InferenceEngineConfig(request_retries=1), [addr], backend="vllm")
        g = GenerationHyperparameters(max_new_tokens=2, max_tokens=64, greedy=True)
        r = asyncio.run(eng.agenerate(ModelRequest(rid="q", input_ids=[9, 8, 7], gconfig=g)))
        assert r.output_tokens == [40, 41] and r.stop_reason == "length" and r.output_logprobs == pytest.approx([-0.1, -0.2])
        body = seen[0][1]
        assert body["prompt"] == [9, 8, 7] and body["return_tokens_as_token_ids"] is True and body["temperature"] == 0.0 and body["max_tokens"] == 2
        eng.pause_generation(); eng.continue_generation(); eng.offload(); eng.onload()
        meta = WeightUpdateMeta(type="disk", path="/ckpt/v3", version=3)
        eng.update_weights_from_disk(meta).result(timeout=30)
        assert eng.get_version() == 3
        xm = WeightUpdateMeta(type="xccl", version=4, nccl_master_address="127.0.0.1", nccl_master_port=1234, nccl_group_name="g")
        eng.init_weights_update_group(xm).result(timeout=30)
        eng.update_weights_from_distributed(xm, [ParamSpec(name="w", shape=(2, 2), dtype="bfloat16")]).result(timeout=30)
        paths = [p for p, _ in seen]
        assert paths[1:] == ["/areal_pause_generation", "/areal_continue_generation", "/sleep", "/wake_up", "/areal_update_weights",
                             "/areal_init_weights_update_group", "/areal_set_update_weight_meta", "/areal_update_weights_xccl"]
        init = [b for p, b in seen if p == "/areal_init_weights_update_group"][0]
        assert init["rank_offset"] == 1 and init["world_size"] == 2 and init["group_name"] == "g"
        with pytest.raises(ValueError, match="return_tokens_as_token_ids"):
            get_backend("vllm").parse_generation({"choices": [{"finish_reason": "stop", "logprobs": {"tokens": ["hello"], "token_logprobs": [0.0]}}]})
        with pytest.raises(ValueError, match="unknown generation-server backend"):
            get_backend("tgi")
    finally:
        srv.shutdown()


def test_server_command_builders_and_external_launch(tmp_path):
    """Flag lists for SGLang / vLLM servers from their config sections, and the launch of an external server process
    (a stand-in that answers the health route) that the engine waits for and tears down."""
    import textwrap

    from areal_b200.api.cli_args import InferenceEngineConfig, SGLangConfig, server_cmd, vLLMConfig
    from areal_b200.engine.remote_engine import RemoteInfEngine
    from areal_b200.utils.network import find_free_ports

    c = SGLangConfig.build_cmd(SGLangConfig(model_path="/m", attention_backend=None, extra={"enable_deterministic_inference": True}), 2, 4,
                               host="127.0.0.1", port=3000, dist_init_addr="10.0.0.1:99", n_nodes=2, node_rank=1)
    assert c[1:3] == ["-m", "sglang.launch_server"] and c[c.index("--tp-size") + 1] == "2" and c[c.index("--base-gpu-id") + 1] == "4"
    assert "--disable-radix-cache" in c and "--enable-deterministic-inference" in c and "--disable-cuda-graph" not in c and "--attention-backend" not in c
    assert c[c.index("--dist-init-addr") + 1] == "10.0.0.1:99" and c[c.index("--node-rank") + 1] == "1"
    v = vLLMConfig.build_cmd(vLLMConfig(model="/m"), 2, 1, port=8000, n_nodes=2, node_rank=1, dist_init_addr="10.0.0.1:555")
    assert v[v.index("--tensor-parallel-size") + 1] == "2" and "--headless" in v and v[v.index("--master-port") + 1] == "555" and "--enforce-eager" not in v
    assert server_cmd("m", {"a_b": [1, 2], "c": {"k": 1}, "d": None, "e": False, "f": True})[3:] == ["--a-b", "1", "2", "--c", '{"k": 1}', "--f"]
    fake = tmp_path / "fake_server.py"
    fake.write_text(textwrap.dedent("""
        import sys
        from http.server import BaseHTTPRequestHandler, HTTPServer
        port = int(sys.argv[sys.argv.index("--port") + 1])
        class H(BaseHTTPRequestHandler):
            def log_message(self, *a): pass
            def do_GET(self):
                self.send_response(200 if self.path == "/health" else 404); self.send_header("Content-Length", "0"); self.end_headers()
        HTTPServer(("127.0.0.1", port), H).serve_forever()
    """))
    port = find_free_ports(1)[0]
    eng = RemoteInfEngine(InferenceEngineConfig(setup_timeout=30), [], backend="sglang")
    addr = eng.launch_server({"cmd": [sys.executable, str(fake), "--port", port], "host": "127.0.0.1", "port": port})
    try:
        assert addr == f"127.0.0.1:{port}" and eng.addresses == [addr] and eng._server_procs[0].poll() is None
    finally:
        proc = eng._server_procs[0]
        eng.teardown_server()
    assert proc.poll() is not None
    bad = RemoteInfEngine(InferenceEngineConfig(setup_timeout=10), [], backend="vllm")
    with pytest.raises(RuntimeError, match="exited with code"):
        bad.launch_server({"cmd": [sys.executable, "-c", "raise SystemExit(3)"], "port": find_free_ports(1)[0]})


def test_least_requests_policy_prefers_the_idle_server():
    from areal_b200.api.cli_args import InferenceEngineConfig
    from areal_b200.engine.remote_engine import RemoteInfEngine

    eng = RemoteInfEngine(InferenceEngineConfig(schedule_policy="least_requests"), ["a:1", "b:1", "c:1"])
    eng._inflight.update({"a:1": 3, "b:1": 0, "c:1": 2})
    assert eng.choose_server("r1") == "b:1" and eng.choose_server("r1") == "b:1"          # and a request id stays where it went
    eng._inflight["b:1"] = 5
    assert eng.choose_server("r2") == "c:1"
    rr = RemoteInfEngine(InferenceEngineConfig(), ["a:1", "b:1"])
    assert [rr.choose_server() for _ in range(4)] == ["a:1", "b:1", "a:1", "b:1"]
