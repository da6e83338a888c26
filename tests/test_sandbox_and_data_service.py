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
