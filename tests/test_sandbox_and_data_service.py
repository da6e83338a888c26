import torch
from torch.utils.data import DataLoader, SequentialSampler

from areal_b200.dataset import ArithmeticDataset
from areal_b200.infra.data_service.rdataset import DatasetWorker, PrefetchAwareSampler, RDataset
from areal_b200.infra.sandbox import LocalSandbox, SandboxConfig, extract_code_blocks, run_python_tool
from areal_b200.infra.sandbox.local import code_exec_reward_fn


def test_sandbox_runs_limits_and_reports():
    sb = LocalSandbox(SandboxConfig(timeout_s=3.0, memory_mb=512))
    r = sb.run("import sys\nprint(int(sys.stdin.read()) * 2)", stdin="21")
    assert r.ok and r.stdout.strip() == "42"
    r = sb.run("raise SystemExit(3)")
    assert not r.ok and r.returncode == 3 and not r.timed_out
    r = LocalSandbox(SandboxConfig(timeout_s=0.5)).run("while True: pass")
    assert r.timed_out and not r.ok
    r = sb.run("x = bytearray(2 * 1024 ** 3)\nprint('big')")             # over the address-space limit
    assert not r.ok and "big" not in r.stdout
    r = sb.run("print(open('data.txt').read())", files={"data.txt": "hello"})
    assert r.stdout.strip() == "hello"
    assert "exit code 1" in run_python_tool({"code": "1/0"}) and "ZeroDivisionError" in run_python_tool({"code": "1/0"})
    text = "think\n```python\nprint(input()[::-1])\n```\ndone"
    assert extract_code_blocks(text) == ["print(input()[::-1])"]
    assert code_exec_reward_fn("", text, [], [], tests=[{"stdin": "abc", "expected": "cba"}, {"stdin": "xy", "expected": "nope"}]) == 0.5
    assert code_exec_reward_fn("", "no code", [], [], tests=[{"stdin": "", "expected": ""}]) == 0.0


def test_remote_dataset_with_prefetch():
    ds = ArithmeticDataset(size=40, seed=3)
    w = DatasetWorker(ds).start()
    try:
        rd = RDataset(w.address, prefetch=16)
        assert len(rd) == 40 and rd[7] == ds[7]
        sampler = PrefetchAwareSampler(SequentialSampler(rd), rd, lookahead=16)
        got = [b for b in DataLoader(rd, batch_size=8, sampler=sampler, collate_fn=list)]
        assert len(got) == 5 and got[0][3] == ds[3] and got[4][7] == ds[39]
        try:
            rd[100]
            raise AssertionError("expected IndexError")
        except IndexError:
            pass
    finally:
        w.stop()


def test_data_service_registers_fans_out_and_keeps_state(tmp_path):
    """Three workers behind one gateway: a dataset registered once is loaded everywhere, a fetch is served by the
    owners of its indices and comes back in request order, epoch / state travel to every worker, tokens and the admin
    key are enforced, and a DataLoader over the remote dataset sees the same samples as the local one."""
    import pytest

    from areal_b200.infra.data_service.service import DataController
    from areal_b200.v2.common import HTTPError, call

    ctl = DataController(n_workers=3).start()
    try:
        ds = ArithmeticDataset(size=50, seed=9)
        rd = ctl.register_dataset(factory="areal_b200.dataset.ArithmeticDataset", kwargs={"size": 50, "seed": 9}, prefetch=16)
        assert len(rd) == 50 and rd.token.startswith("sk-data-")
        order = [49, 0, 7, 7, 23, 1, 2]
        got = call(f"http://{ctl.gateway.address}/v1/samples/fetch", {"indices": order}, api_key=rd.token)["samples"]
        from areal_b200.infra.rpc.serialization import deserialize_value

        assert [deserialize_value(g) for g in got] == [ds[i] for i in order]
        served = [h["datasets"] for h in (call(f"http://{w.address}/health") for w in ctl.workers)]
        assert all(list(s.values()) == [50] for s in served)            # every worker loaded the whole set
        sampler = PrefetchAwareSampler(SequentialSampler(rd), rd, lookahead=16)
        batches = [b for b in DataLoader(rd, batch_size=10, sampler=sampler, collate_fn=list)]
        assert [x for b in batches for x in b] == [ds[i] for i in range(50)]
        assert rd.advance_epoch() == 1 and rd.advance_epoch(5) == 5
        files = rd.save_state(str(tmp_path / "state"))
        assert len(files) == 3
        rd.advance_epoch(9)
        st = rd.load_state(str(tmp_path / "state"))
        assert st["epoch"] == 5 and st["served"] >= 50 + len(order)
        with pytest.raises(HTTPError) as e:
            call(f"http://{ctl.gateway.address}/v1/samples/fetch", {"indices": [0]}, api_key="sk-data-wrong")
        assert e.value.status == 401
        with pytest.raises(HTTPError) as e:
            call(f"http://{ctl.gateway.address}/v1/datasets/register", {"factory": "x.y"}, api_key="nope")
        assert e.value.status == 401
        with pytest.raises(HTTPError) as e:
            call(f"http://{ctl.gateway.address}/v1/samples/fetch", {"indices": [50]}, api_key=rd.token)
        assert e.value.status == 400
        stat = ctl.status()
        assert stat["datasets"][rd.dataset_id]["len"] == 50 and len(stat["workers"]) == 3
        # a worker that went away is marked unhealthy and no longer routed to
        ctl.workers[2].stop()
        ctl.router.check_health()
        assert [w["healthy"] for w in call(f"http://{ctl.router.address}/workers", api_key=ctl.admin_key)["workers"]] == [True, True, False]
        assert call(f"http://{ctl.router.address}/route", {}, api_key=ctl.admin_key)["address"] in (ctl.workers[0].address, ctl.workers[1].address)
    finally:
        ctl.stop()


def test_remote_sandbox_runs_code_on_a_server_with_its_limits():
    import pytest

    from areal_b200.infra.sandbox import DaytonaRunner, RemoteSandbox, SandboxConfig, SandboxServer
    from areal_b200.infra.sandbox.local import run_python_tool
    from areal_b200.v2.common import HTTPError

    srv = SandboxServer(SandboxConfig(timeout_s=2.0), api_key="k", max_concurrent=2).start()
    try:
        sb = RemoteSandbox(srv.address, api_key="k")
        r = sb.run("import sys; print(sys.stdin.read().upper() + open('d.txt').read())", stdin="ab", files={"d.txt": "!"})
        assert r.ok and r.stdout.strip() == "AB!"
        r = sb.run("raise SystemExit(3)")
        assert not r.ok and r.returncode == 3
        slow = RemoteSandbox(srv.address, api_key="k", timeout_s=50.0).run("import time; time.sleep(30)")
        assert slow.timed_out and slow.seconds < 10                 # the server's own limit (2 s) wins over the request's 50 s
        assert "exit code" not in run_python_tool({"code": "print(6*7)"}, sandbox=sb) and "42" in run_python_tool({"code": "print(6*7)"}, sandbox=sb)
        with pytest.raises(HTTPError) as e:
            RemoteSandbox(srv.address, api_key="wrong", retries=1).run("print(1)")
        assert e.value.status == 401
    finally:
        srv.stop()
    with pytest.raises(ImportError, match="daytona"):
        DaytonaRunner()
