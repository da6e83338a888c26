"""v2 microservices with in-process servers: gateway / router / data proxies, training
service with a fake engine, weight-update gateway, CLI state."""
import json
import os
import time

import pytest
import torch

from areal_b200.api.cli_args import GenerationHyperparameters
from areal_b200.v2 import cli
from areal_b200.v2.common import HTTPError, JsonService, call
from areal_b200.v2.inference_service.controller import InferenceServiceController
from areal_b200.v2.training_service.controller import TrainingServiceClient
from areal_b200.v2.training_service.worker import TrainingWorker
from areal_b200.v2.weight_update.gateway import WeightUpdateGateway
from tests.test_openai_and_agents import ByteTok, ScriptedEngine


class CtlEngine(ScriptedEngine):
    def __init__(self, answers):
        super().__init__(answers, version=0)
        self.events = []

    def pause_generation(self):
        self.events.append("pause")

    def continue_generation(self):
        self.events.append("continue")

    def set_version(self, v):
        self.version = v
        self.events.append(("version", v))


def test_json_service_routing_and_errors():
    svc = JsonService("t")

    @svc.route("POST", "/a/{x}/b")
    def h(body, ctx):
        if body.get("boom"):
            raise HTTPError(418, "teapot")
        return {"x": ctx.params["x"], "key": ctx.api_key, "n": body.get("n", 0) + 1}
    svc.start()
    try:
        assert call(f"{svc.url}/a/7/b", {"n": 1}, api_key="k") == {"x": "7", "key": "k", "n": 2}
        with pytest.raises(HTTPError) as e:
            call(f"{svc.url}/a/7/b", {"boom": True})
        assert e.value.status == 418 and e.value.message == "teapot"
        with pytest.raises(HTTPError) as e:
            call(f"{svc.url}/nope", {})
        assert e.value.status == 404
    finally:
        svc.stop()
    with pytest.raises(HTTPError) as e:
        call(f"{svc.url}/a/7/b", {}, timeout=1)
    assert e.value.status == 503


def test_inference_service_sessions_affinity_export_and_control():
    engines = [CtlEngine(["alpha", "beta"]), CtlEngine(["gamma", "delta"])]
    ctl = InferenceServiceController(admin_key="adm").start(engines, ByteTok(), GenerationHyperparameters(max_new_tokens=16))
    try:
        with pytest.raises(HTTPError) as e:
            call(f"{ctl.gateway.svc.url}/rl/start_session", {}, api_key="wrong")
        assert e.value.status == 401
        s1, s2 = ctl.start_session("t1"), ctl.start_session("t2")
        assert s1["base_url"] == ctl.base_url
        owners = {call(f"http://{ctl.router.address}/route/lookup", {"session_id": s["api_key"]})["address"] for s in (s1, s2)}
        assert len(owners) == 2                                         # least-loaded placement spreads the two sessions
        for s in (s1, s2):
            for turn in range(2):                                        # both turns of a session hit the same engine
                c = call(f"{ctl.base_url}/chat/completions", {"messages": [{"role": "user", "content": f"q{turn}"}]}, api_key=s["api_key"])
                assert c["choices"][0]["message"]["content"] in ("alpha", "beta", "gamma", "delta")
            call(f"{ctl.gateway.svc.url}/rl/set_reward", {"reward": 1.5}, api_key=s["api_key"])
            call(f"{ctl.gateway.svc.url}/rl/end_session", {}, api_key=s["api_key"])
        assert [len(e.requests) for e in engines] == [2, 2]
        with pytest.raises(HTTPError):                                   # ended sessions are gone
            call(f"{ctl.base_url}/chat/completions", {"messages": []}, api_key=s1["api_key"])
        batch = ctl.export_batch(style="individual", discount=0.5)
        assert batch["input_ids"].shape[0] == 4 and sorted(batch["rewards"].tolist()) == [0.75, 0.75, 1.5, 1.5]
        assert ctl.export_batch() is None
        ctl.pause_generation()
        ctl.set_version(3)
        ctl.continue_generation()
        assert all(e.events == ["pause", ("version", 3), "continue"] for e in engines)
        assert call(f"http://{ctl.router.address}/health_check", {})["workers"][ctl.proxies[0].address]["healthy"]
    finally:
        ctl.stop()


def test_inference_service_streams_completions_through_the_gateway():
    """``stream: true`` at the gateway: the worker's server-sent events are relayed as they are; the concatenated deltas
    equal the non-streamed answer and the turn is recorded for training like any other."""
    import json

    from areal_b200.v2.common import sse_lines

    engines = [CtlEngine(["x" * 150, "plain"])]
    ctl = InferenceServiceController(admin_key="adm").start(engines, ByteTok(), GenerationHyperparameters(max_new_tokens=256))
    try:
        s = ctl.start_session("t1")
        evs = list(sse_lines(f"{ctl.base_url}/chat/completions", {"messages": [{"role": "user", "content": "q"}], "stream": True},
                             api_key=s["api_key"]))
        assert evs[-1] == (None, "[DONE]")
        chunks = [json.loads(d) for _, d in evs[:-1]]
        assert all(c["object"] == "chat.completion.chunk" for c in chunks) and len(chunks) >= 5
        assert "".join(c["choices"][0]["delta"].get("content", "") for c in chunks) == "x" * 150
        assert chunks[-1]["choices"][0]["finish_reason"] == "stop" and chunks[-1]["usage"]["completion_tokens"] > 0
        c = call(f"{ctl.base_url}/chat/completions", {"messages": [{"role": "user", "content": "q"}]}, api_key=s["api_key"])
        assert c["choices"][0]["message"]["content"] == "plain"
        with pytest.raises(HTTPError) as e:
            list(sse_lines(f"{ctl.base_url}/chat/completions", {"messages": [], "stream": True}, api_key="sk-unknown"))
        assert e.value.status in (401, 404)
        call(f"{ctl.gateway.svc.url}/rl/set_reward", {"reward": 1.0}, api_key=s["api_key"])
        call(f"{ctl.gateway.svc.url}/rl/end_session", {}, api_key=s["api_key"])
        batch = ctl.export_batch(style="individual", discount=1.0)
        assert batch["input_ids"].shape[0] == 2
    finally:
        ctl.stop()


class FakeTrainEngine:
    """CPU stand-in for a train engine: deterministic functions of the batch."""

    def __init__(self):
        self.version, self.saved, self.lr_steps = 0, [], 0

    def get_version(self):
        return self.version

    def set_version(self, v):
        self.version = v

    def step_lr_scheduler(self):
        self.lr_steps += 1

    def compute_logp(self, batch):
        return batch["input_ids"].float() * -0.5

    def compute_advantages(self, batch, group_sizes=None):
        batch["advantages"] = batch["rewards"][:, None].expand_as(batch["input_ids"]).float() * batch["attention_mask"]
        return batch

    def ppo_update(self, batch):
        return [{"n_seqs": float(batch["input_ids"].shape[0])}]

    def train_lm(self, batch):
        return {"nll": 1.0}

    def save(self, meta):
        os.makedirs(meta.path, exist_ok=True)
        open(os.path.join(meta.path, "model.safetensors"), "w").write("x")
        self.saved.append(meta.path)

    def export_stats(self):
        return {"k": 1.0}


def test_training_service_dispatch_and_merge():
    engs = [FakeTrainEngine(), FakeTrainEngine()]
    workers = [TrainingWorker(e).start() for e in engs]
    try:
        cl = TrainingServiceClient([w.address for w in workers], group_size=2)
        lens = torch.tensor([9, 3, 5, 7, 2, 8, 6, 4])
        am = torch.arange(9)[None] < lens[:, None]
        batch = {"attention_mask": am, "input_ids": torch.randint(1, 9, (8, 9)) * am, "rewards": torch.arange(8).float()}
        lp = cl.compute_logp(batch)
        assert torch.equal(lp, batch["input_ids"].float() * -0.5)
        out = cl.compute_advantages(batch)
        assert out is batch and torch.equal(batch["advantages"], batch["rewards"][:, None].expand(8, 9) * am)
        assert cl.ppo_update(batch) == [{"n_seqs": 4.0}]
        assert cl.train_lm(batch) == {"nll": 1.0}
        cl.set_version(5)
        cl.step_lr_scheduler()
        assert [e.version for e in engs] == [5, 5] and [e.lr_steps for e in engs] == [1, 1]
        assert cl.export_stats() == {"k": 1.0} and all(h["status"] == "ok" for h in cl.health())
        with pytest.raises(HTTPError) as e:
            cl._batch_call("/rw/train", batch)
        assert e.value.status == 404
    finally:
        for w in workers:
            w.stop()


def test_weight_update_gateway_disk_flow(tmp_path):
    eng = FakeTrainEngine()
    tw = TrainingWorker(eng).start()
    infer = JsonService("fake_infer")
    log = []
    for name in ("pause_generation", "continue_generation", "update_weights_from_disk"):
        infer.route("POST", f"/{name}")(lambda body, ctx, name=name: log.append((name, body.get("model_path"), body.get("version"))) or {"success": True})
    infer.start()
    gw = WeightUpdateGateway().start()
    try:
        with pytest.raises(HTTPError):
            call(f"{gw.svc.url}/connect", {"pair": "p", "train_workers": [], "infer_workers": [], "mode": "disk"})
        call(f"{gw.svc.url}/connect", {"pair": "p", "train_workers": [tw.address], "infer_workers": [infer.address], "mode": "disk",
                                       "path": str(tmp_path)})
        r = call(f"{gw.svc.url}/update_weights", {"pair": "p", "version": 2})
        assert r["ok"] and r["version"] == 2
        ck = os.path.join(str(tmp_path), "v2")
        assert eng.saved == [ck] and eng.version == 2
        assert log == [("pause_generation", None, None), ("update_weights_from_disk", ck, 2), ("continue_generation", None, None)]
        assert call(f"{gw.svc.url}/weight_meta/p/version") == {"version": 2}
        assert call(f"{gw.svc.url}/weight_meta/p/last_checkpoint") == {"last_checkpoint": ck}
        call(f"{gw.svc.url}/disconnect", {"pair": "p"})
        with pytest.raises(HTTPError) as e:
            call(f"{gw.svc.url}/update_weights", {"pair": "p", "version": 3})
        assert e.value.status == 404
    finally:
        gw.stop(); infer.stop(); tw.stop()


def test_weight_update_gateway_http_flow_moves_real_weights():
    """``mode: http``: the inference worker pulls the trainer's weight dictionary over HTTP and its engine swaps it in;
    a real train engine and a real inference engine (tiny model, CPU) end up with identical parameters and versions."""
    import torch

    from areal_b200.api.cli_args import InferenceEngineConfig, MicroBatchSpec, NativeInferConfig, OptimizerConfig, TrainEngineConfig
    from areal_b200.engine.infer_engine import NativeInferenceEngine
    from areal_b200.engine.train_engine import B200TrainEngine
    from areal_b200.models.config import preset
    from areal_b200.v2.inference_service.data_proxy import DataProxy

    mc = preset("tiny-qwen2", vocab_size=64, num_layers=2)
    tr = B200TrainEngine(TrainEngineConfig(init_from_scratch=True, dtype="float32", optimizer=OptimizerConfig(lr=1e-2),
                                           mb_spec=MicroBatchSpec(max_tokens_per_mb=128)))
    tr.create_process_group()
    tr.initialize(model_config=mc, seed=1)
    inf = NativeInferenceEngine(InferenceEngineConfig(), NativeInferConfig(max_running_requests=4, page_size=16, context_length=64, num_pages=32),
                                model_config=mc).initialize(seed=2, start_executor=False)
    name = "layers.0.mlp.down_proj"
    assert not torch.equal(dict(inf.model.named_parameters())[name], dict(tr.model.named_parameters())[name])
    tw = TrainingWorker(tr).start()
    dp = DataProxy(inf, ByteTok(), GenerationHyperparameters(max_new_tokens=4)).start()
    gw = WeightUpdateGateway().start()
    try:
        call(f"{gw.svc.url}/connect", {"pair": "p", "train_workers": [tw.address], "infer_workers": [dp.address], "mode": "http"})
        r = call(f"{gw.svc.url}/update_weights", {"pair": "p", "version": 5})
        assert r["ok"] and r["version"] == 5
        for (n, a), (_, b) in zip(tr.model.named_parameters(), inf.model.named_parameters()):
            assert torch.equal(a.detach(), b.detach()), n
        assert tr.get_version() == 5 and inf.get_version() == 5
        assert call(f"{gw.svc.url}/weight_meta/p/tensors")["tensors"] == len(list(tr.model.named_parameters()))
    finally:
        gw.stop(); dp.stop(); tw.stop(); inf.destroy(); tr.destroy()


def test_cli_state_roundtrip(tmp_path, monkeypatch, capsys):
    monkeypatch.setattr(cli, "STATE", str(tmp_path / "st.json"))
    svc = JsonService("x")
    svc.route("GET", "/health")(lambda b, c: {"status": "ok"})
    svc.start()
    try:
        cli.record("inference", svc.address, preset="tiny")
        cli.record("inference", "127.0.0.1:9", preset="dead")
        assert cli.main(["inference", "status"]) == 1
        out = capsys.readouterr().out
        assert "ok" in out and "DOWN" in out
        assert len(json.load(open(tmp_path / "st.json"))["services"]) == 2
        assert cli.main(["inference", "ps"]) == 0 and "PID" in capsys.readouterr().out
        assert cli.main(["inference", "models"]) == 1                  # the stub has no /v1/models route
        log = tmp_path / "svc.log"
        log.write_text("a\nb\nc\n")
        cli.record("sandbox", "127.0.0.1:7", log=str(log), name="sbx0")
        capsys.readouterr()
        assert cli.main(["logs", "sbx0", "-n", "2"]) == 0 and capsys.readouterr().out == "b\nc\n"
        assert cli.main(["logs", "nobody"]) == 1
        assert cli.main(["sandbox", "stop", "--address", "127.0.0.1:7"]) == 0      # recorded by this very process: only forgotten
        assert cli.main(["sandbox", "stop"]) == 1
        assert [s_["kind"] for s_ in cli.load_state()["services"]] == ["inference", "inference"]
        assert cli.main(["state", "clear"]) == 0 and cli.load_state() == {"services": []}
    finally:
        svc.stop()


def test_cli_serves_a_sandbox_and_a_data_worker(tmp_path):
    """``python -m areal_b200.v2.cli sandbox serve`` / ``data serve worker`` as real child processes: they print their
    address, answer, are listed in the state file, and ``stop`` ends them by their recorded pid."""
    import os
    import subprocess
    import sys
    import time

    from areal_b200.infra.sandbox import RemoteSandbox

    env = dict(os.environ, AREAL_V2_STATE=str(tmp_path / "st.json"), PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    procs = []
    try:
        addrs = {}
        for args, tag in ((["sandbox", "serve", "--api-key", "k"], "SANDBOX_READY"), (["data", "serve", "worker"], "DATA_WORKER_READY")):
            p = subprocess.Popen([sys.executable, "-m", "areal_b200.v2.cli"] + args, env=env, stdout=subprocess.PIPE, text=True)
            procs.append(p)
            line = p.stdout.readline()
            assert line.startswith(tag), line
            addrs[tag] = line.split()[1]
        assert RemoteSandbox(addrs["SANDBOX_READY"], api_key="k").run("print(1+1)").stdout.strip() == "2"
        assert call(f"http://{addrs['DATA_WORKER_READY']}/health")["status"] == "ok"
        st = json.load(open(tmp_path / "st.json"))["services"]
        assert sorted(s_["kind"] for s_ in st) == ["data", "sandbox"] and {s_["pid"] for s_ in st} == {p.pid for p in procs}
        r = subprocess.run([sys.executable, "-m", "areal_b200.v2.cli", "sandbox", "stop"], env=env, capture_output=True, text=True)
        assert r.returncode == 0 and "stopped 1" in r.stdout
        for _ in range(100):
            if procs[0].poll() is not None:
                break
            time.sleep(0.05)
        assert procs[0].poll() is not None and procs[1].poll() is None
    finally:
        for p in procs:
            if p.poll() is None:
                p.terminate()
            p.wait(timeout=10)


def test_agent_service_runs_queues_and_ends_sessions():
    import threading
    import time

    from areal_b200.v2.agent_service import AgentController
    from areal_b200.v2.common import call

    gate = threading.Event()
    seen = []

    def agent(message, session):
        seen.append((session.session_key, message, len(session.history)))
        if message == "slow":
            gate.wait(5)
        return {"text": f"echo:{message}", "n_history": len(session.history)}

    ctl = AgentController(agent, n_workers=2)
    try:
        r = ctl.run("s1", "hello")
        assert r["status"] == "ok" and r["result"]["text"] == "echo:hello"
        r2 = ctl.run("s1", "again")
        assert r2["result"]["n_history"] == 2                       # the session's history reached the agent
        # while a run is active, messages queue; collect mode folds them into one follow-up turn
        first = ctl.run("s2", "slow", wait=False)
        q1 = ctl.run("s2", "a", wait=False)
        q2 = ctl.run("s2", "b", wait=False)
        assert q1["status"] == "queued" and q2["queued"] == 2 and q2["active_run_id"] == first["run_id"]
        gate.set()
        done = ctl.gateway.wait_run(first["run_id"])
        follow = ctl.gateway.wait_run(done["followup_run_id"])
        assert follow["message"] == "a\nb" and follow["result"]["text"] == "echo:a\nb"
        # followup mode replays them one by one
        gate.clear()
        f0 = ctl.run("s3", "slow", wait=False)
        ctl.run("s3", "x", queue_mode="followup", wait=False)
        ctl.run("s3", "y", queue_mode="followup", wait=False)
        gate.set()
        d0 = ctl.gateway.wait_run(f0["run_id"])
        d1 = ctl.gateway.wait_run(d0["followup_run_id"])
        d2 = ctl.gateway.wait_run(d1["followup_run_id"])
        assert (d1["message"], d2["message"]) == ("x", "y")
        polled = call(f"http://{ctl.gateway.address}/agent/runs/{d2['run_id']}")
        assert polled["status"] == "ok" and polled["result"]["text"] == "echo:y"
        ended = call(f"http://{ctl.gateway.address}/agent/sessions/s1/end", {})
        assert ended["turns"] == 2
        try:
            ctl.run("s1", "late")
            raise AssertionError("an ended session accepted a run")
        except Exception as e:
            assert "409" in repr(e) or "ended" in repr(e)
        # sessions stick to one worker; two workers share the sessions
        assert sum(w.turns for w in ctl.workers) == len(seen) and all(w.turns > 0 for w in ctl.workers)
    finally:
        gate.set()
        ctl.close()


def test_control_plane_fault_injection_5xx_drop_and_delay():
    """HTTP faults on the control plane: 5xx answers and refused connections are retried with
    back-off, 4xx answers are final, a slow answer beyond the caller's time-out counts as a fault."""
    import asyncio
    import time

    import aiohttp

    from areal_b200.engine.remote_engine import arequest_with_retry
    from areal_b200.utils.network import find_free_ports
    from areal_b200.v2.common import HTTPError, JsonService, call

    hits = {"flaky": 0, "bad": 0, "slow": 0}
    svc = JsonService("faulty")

    @svc.route("POST", "/flaky")
    def flaky(body, ctx):
        hits["flaky"] += 1
        if hits["flaky"] % 3:                       # two 5xx answers, then success
            raise RuntimeError("injected failure")
        return {"ok": True, "attempts": hits["flaky"]}

    @svc.route("POST", "/bad")
    def bad(body, ctx):
        hits["bad"] += 1
        raise HTTPError(422, "malformed")

    @svc.route("POST", "/slow")
    def slow(body, ctx):
        hits["slow"] += 1
        if hits["slow"] == 1:
            time.sleep(1.0)                         # first answer comes too late for the caller
        return {"ok": True}

    svc.start()
    try:
        assert call(f"{svc.url}/flaky", {}, retries=3)["attempts"] == 3
        try:
            call(f"{svc.url}/flaky", {}, retries=2)                        # 5xx twice: gives up
            raise AssertionError("expected a failure")
        except HTTPError as e:
            assert e.status == 500
        try:
            call(f"{svc.url}/bad", {}, retries=5)
            raise AssertionError("expected a failure")
        except HTTPError as e:
            assert e.status == 422 and hits["bad"] == 1                     # client errors are not retried
        dead = f"http://127.0.0.1:{find_free_ports(1)[0]}/x"
        t0 = time.time()
        try:
            call(dead, {}, retries=2, timeout=1.0)
            raise AssertionError("expected a failure")
        except HTTPError as e:
            assert e.status == 503 and time.time() - t0 < 5

        async def go():
            async with aiohttp.ClientSession() as s:
                hits["flaky"] = 0
                r = await arequest_with_retry(s, svc.address, "/flaky", {}, max_retries=3, retry_delay=0.01)
                assert r["attempts"] == 3
                r = await arequest_with_retry(s, svc.address, "/slow", {}, max_retries=2, timeout=0.3, retry_delay=0.01)
                assert r["ok"] and hits["slow"] == 2                          # timed out once, then served
                try:
                    await arequest_with_retry(s, dead[7:].split("/")[0], "/x", {}, max_retries=2, retry_delay=0.01)
                    raise AssertionError("expected a failure")
                except RuntimeError as e:
                    assert "failed after 2 attempts" in str(e)
        asyncio.run(go())
    finally:
        svc.stop()


def test_training_gateway_dispatches_by_topology_and_heads_answer(tmp_path):
    """Two data-parallel groups of two model-parallel ranks each: every rank of a group receives the group's share of the
    batch, the head's answer is merged; control calls reach all four workers; a group with a missing rank degrades the
    gateway instead of dispatching to half a group."""
    from areal_b200.api.io_struct import SaveLoadMeta
    from areal_b200.v2.training_service.gateway import GatewayTrainingClient, TrainingGateway, TrainingRouter

    class Eng(FakeTrainEngine):
        def __init__(self, rank, dp_rank, head):
            super().__init__()
            self.rank, self.dp_rank, self.dp_size, self._head, self.seen = rank, dp_rank, 2, head, []

        def is_data_parallel_head(self):
            return self._head

        def compute_logp(self, batch):
            self.seen.append(batch["input_ids"].shape[0])
            return batch["input_ids"].float() * (-0.5 if self._head else 99.0)      # only the head's answer may come back

    engs = [Eng(0, 0, True), Eng(1, 0, False), Eng(2, 1, True), Eng(3, 1, False)]
    workers = [TrainingWorker(e).start() for e in engs]
    router = TrainingRouter(heartbeat_timeout=1.0).start()
    gw = TrainingGateway(router, admin_key="adm", group_size=2).start()
    try:
        with pytest.raises(HTTPError) as e:                     # nobody registered yet: the gateway says so with a 503
            call(f"{gw.svc.url}/health", method="GET")
        assert e.value.status == 503
        for w in workers[:3]:
            w.register(router.svc.address, heartbeat_s=0.2)
        cl = GatewayTrainingClient(gw.svc.address, "adm")
        lens = torch.tensor([9, 3, 5, 7, 2, 8, 6, 4])
        am = torch.arange(9)[None] < lens[:, None]
        batch = {"attention_mask": am, "input_ids": torch.randint(1, 9, (8, 9)) * am, "rewards": torch.arange(8).float()}
        with pytest.raises(HTTPError) as e:                     # rank 3 has not registered: group 1 is incomplete
            cl.compute_logp(batch)
        assert e.value.status == 503
        workers[3].register(router.svc.address, heartbeat_s=0.2)
        with pytest.raises(HTTPError) as e:
            GatewayTrainingClient(gw.svc.address, "wrong").compute_logp(batch)
        assert e.value.status == 401
        topo = cl.topology()
        assert [[w["rank"] for w in g] for g in topo] == [[0, 1], [2, 3]] and all(g[0]["is_dp_head"] and not g[1]["is_dp_head"] for g in topo)
        lp = cl.compute_logp(batch)
        assert torch.equal(lp, batch["input_ids"].float() * -0.5)
        assert engs[0].seen == engs[1].seen == [4] and engs[2].seen == engs[3].seen == [4]      # peers saw their head's share
        out = cl.compute_advantages(batch)
        assert out is batch and torch.equal(batch["advantages"], batch["rewards"][:, None].expand(8, 9) * am)
        cl.set_version(7)
        cl.step_lr_scheduler()
        cl.save(SaveLoadMeta(path=str(tmp_path / "ck"), weight_format="hf", with_optim=False))
        assert [e_.version for e_ in engs] == [7] * 4 and [e_.lr_steps for e_ in engs] == [1] * 4 and all(e_.saved for e_ in engs)
        # a worker that stops beating drops out of the live set after the timeout
        workers[1].stop()
        time.sleep(1.5)
        assert call(f"{router.svc.url}/workers")["workers"].__len__() == 3
        with pytest.raises(HTTPError):
            cl.compute_logp(batch)
    finally:
        gw.stop(); router.stop()
        for w in workers:
            try:
                w.stop()
            except Exception:
                pass


def test_inference_service_serves_messages_responses_and_the_tokenizer():
    """Anthropic Messages and Responses shapes through the gateway land in the same recorded session as chat
    completions; the tokenizer routes answer with the policy's own tokenizer."""
    from areal_b200.v2.common import sse_lines

    engines = [CtlEngine(["alpha", "beta", "gamma"])]
    ctl = InferenceServiceController(admin_key="adm").start(engines, ByteTok(), GenerationHyperparameters(max_new_tokens=16))
    try:
        s = ctl.start_session("t")
        root = ctl.gateway.svc.url
        m = call(f"{root}/v1/messages", {"system": "be brief", "max_tokens": 8, "messages": [{"role": "user", "content": [{"type": "text", "text": "hi"}]}]},
                 api_key=s["api_key"])
        assert m["type"] == "message" and m["content"][0]["text"] == "alpha" and m["stop_reason"] == "end_turn"
        r = call(f"{root}/v1/responses", {"input": "and again", "max_output_tokens": 8}, api_key=s["api_key"])
        assert r["object"] == "response" and r["output_text"] == "beta" and r["usage"]["output_tokens"] > 0
        evs = list(sse_lines(f"{root}/v1/messages", {"max_tokens": 8, "stream": True, "messages": [{"role": "user", "content": "more"}]}, api_key=s["api_key"]))
        kinds = [e for e, _ in evs]
        assert kinds[0] == "message_start" and kinds[-1] == "message_stop" and "content_block_delta" in kinds
        t = call(f"{root}/tokenize", {"text": "abc"})
        assert t == {"input_ids": [97, 98, 99], "count": 3} and call(f"{root}/detokenize", {"input_ids": [97, 98]}) == {"text": "ab"}
        call(f"{root}/rl/set_reward", {"reward": 1.0}, api_key=s["api_key"])
        call(f"{root}/rl/end_session", {}, api_key=s["api_key"])
        assert ctl.export_batch(style="individual", discount=1.0)["input_ids"].shape[0] == 3          # three recorded model calls
    finally:
        ctl.stop()
