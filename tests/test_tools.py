import json
import os

from areal_b200.tools import perf_trace_converter as ptc
from areal_b200.tools import validate_installation as vi


def test_trace_converter_merges_ranks_and_sessions(tmp_path):
    d = tmp_path / "perf_tracer"
    d.mkdir()
    for r in range(2):
        with open(d / f"traces-r{r}.jsonl", "w") as f:
            f.write(json.dumps(dict(name="train.ppo_update", cat="compute", ph="X", ts=1000.0 + r, dur=500.0, pid=r, tid=1, args={})) + "\n")
            f.write("not json\n")
            f.write(json.dumps(dict(name="mark", cat="misc", ph="i", ts=1700.0, pid=r, tid=1, args={})) + "\n")
    with open(d / "sessions.jsonl", "w") as f:
        f.write(json.dumps(dict(session_id=3, task_id=7, rank=0, submit_ts=10.0, status="accepted", end_ts=11.0,
                                phases=[dict(name="generate", start=10.1, end=10.6), dict(name="reward", start=10.6, end=10.7)])) + "\n")
    out = tmp_path / "trace.json"
    ptc.main([str(tmp_path), "-o", str(out), "--summary"])
    tr = json.load(open(out))
    ev = tr["traceEvents"]
    assert tr["otherData"] == {"ranks": [0, 1], "sessions": 1, "source_files": 3}
    assert sum(e.get("ph") == "M" for e in ev) == 3
    x = [e for e in ev if e.get("ph") == "X" and e["name"] == "train.ppo_update"]
    assert len(x) == 2 and min(e["ts"] for e in x) == 0.0
    gen = next(e for e in ev if e["name"] == "generate")
    assert abs(gen["dur"] - 0.5e6) < 1 and gen["pid"] == 2 and gen["tid"] == 3 and gen["args"]["task_id"] == 7
    s = ptc.summarize(tr)
    assert s["train.ppo_update"]["count"] == 2 and abs(s["train.ppo_update"]["total_ms"] - 1.0) < 1e-9


def test_validate_installation_cpu_mode(capsys):
    rc = vi.main(["--no-gpu"])
    outp = capsys.readouterr().out
    assert rc == 0 and "import torch" in outp and "import areal_b200" in outp
    r = vi.Report()
    r.run("bad", lambda: 1 / 0, required=True)
    r.run("opt", lambda: 1 / 0, required=False)
    assert not r.ok and [s for _, s, _ in r.rows] == ["FAIL", "missing"]


def test_local_launcher_restarts_failed_job(tmp_path):
    """The trainer script fails on its first run and succeeds on the recover run."""
    import sys

    from areal_b200.api.cli_args import BaseExperimentConfig, ClusterSpecConfig, RecoverConfig
    from areal_b200.infra.launcher.local import JobFailed, LocalLauncher, launch

    script = tmp_path / "train.py"
    marker = tmp_path / "ran_once"
    script.write_text(
        "import os, sys\n"
        f"m = {str(marker)!r}\n"
        "if os.environ.get('RANK') == '0' and not os.path.exists(m):\n"
        "    open(m, 'w').write(os.environ['AREAL_RECOVER_RUN']); sys.exit(3)\n"
        "assert os.environ['WORLD_SIZE'] == '2'\n"
        f"open(os.path.join({str(tmp_path)!r}, 'done_' + os.environ['RANK']), 'w').write(os.environ['AREAL_RECOVER_RUN'])\n")
    cfg = BaseExperimentConfig(experiment_name="l", trial_name="t", cluster=ClusterSpecConfig(fileroot=str(tmp_path)),
                               allocation_mode="d2", recover=RecoverConfig(mode="auto", retries=2))
    assert launch(str(script), [], cfg, n_gpus=0) == 0
    assert marker.read_text() == "0" and (tmp_path / "done_0").read_text() == "1" and (tmp_path / "done_1").exists()
    # with recovery disabled the failure is final
    marker.unlink()
    cfg.recover.mode = "disabled"
    assert launch(str(script), [], cfg, n_gpus=0) != 0
    la = LocalLauncher("l", "t", str(tmp_path), n_gpus=0)
    la.submit("bad", [sys.executable, "-c", "import sys; sys.exit(5)"])
    try:
        la.wait()
        raise AssertionError("expected JobFailed")
    except JobFailed as e:
        assert e.code == 5 and e.name == "bad"
    la.stop_all()


KILLED_RANK_SCRIPT = r'''
import faulthandler, json, os, signal, sys
faulthandler.dump_traceback_later(240, exit=True)
sys.path.insert(0, %(root)r)
os.environ["AREAL_FORCE_CPU"] = "1"
import torch.distributed as dist
from tests.test_e2e_cpu import _cfg, digit_reward
from areal_b200.dataset import ArithmeticDataset
from areal_b200.models.config import preset
from areal_b200.rollout.workflows.rlvr import RLVRWorkflow
from areal_b200.trainer.rl_trainer import PPOTrainer
dist.init_process_group("gloo")
rank = dist.get_rank()
first_run = os.environ["AREAL_RECOVER_RUN"] == "0"
cfg = _cfg(%(tmp)r, steps=6, recover="auto")
cfg.actor.backend = "d2"
mc = preset("tiny-qwen2", vocab_size=64, num_layers=2)
with PPOTrainer(cfg, ArithmeticDataset(size=128), tokenizer=None, model_config=mc) as tr:
    wf = RLVRWorkflow(digit_reward, cfg.gconfig, reward_in_process=True)
    start = tr.start_step
    if first_run:
        hist = tr.train(workflow=wf, max_steps=3)
        dist.barrier()
        if rank == 1:
            os.kill(os.getpid(), signal.SIGKILL)          # dies between steps, nothing of it in flight
        hist += tr.train(workflow=wf)                      # the survivor walks into a collective with a dead peer
    else:
        hist = tr.train(workflow=wf)
    json.dump({"start": start, "steps": len(hist), "version": tr.actor.get_version()}, open(os.path.join(%(tmp)r, f"result_{rank}.json"), "w"))
dist.barrier()
'''


def test_killed_rank_restarts_job_which_resumes_from_recover_checkpoint(tmp_path):
    """SIGKILL of one gloo trainer rank between steps: torchrun ends the job, the launcher starts it
    again as a recover run, and training continues from the last recover checkpoint (step 3 of 6)."""
    import json

    from areal_b200.api.cli_args import BaseExperimentConfig, ClusterSpecConfig, RecoverConfig
    from areal_b200.infra.launcher.local import launch

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "train.py"
    script.write_text(KILLED_RANK_SCRIPT % dict(root=root, tmp=str(tmp_path)))
    cfg = BaseExperimentConfig(experiment_name="e2e", trial_name="t0", cluster=ClusterSpecConfig(fileroot=str(tmp_path)),
                               allocation_mode="d2", recover=RecoverConfig(mode="auto", retries=1))
    assert launch(str(script), [], cfg, n_gpus=0) == 0
    res = [json.load(open(tmp_path / f"result_{r}.json")) for r in range(2)]
    assert all(r["start"] == 3 and r["steps"] == 3 and r["version"] == 6 for r in res), res


def test_plot_session_trace(tmp_path, capsys):
    from areal_b200.tools import plot_session_trace as pst

    d = tmp_path / "rank0"
    d.mkdir()
    rows = [dict(session_id=i, task_id=i, rank=0, submit_ts=100.0 + i, end_ts=103.0 + i, status="accepted" if i % 3 else "rejected",
                 phases=[dict(name="generate", start=100.2 + i, end=102.0 + i), dict(name="reward", start=102.0 + i, end=102.5 + i)]) for i in range(5)]
    (d / "sessions.jsonl").write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    out = tmp_path / "s.html"
    assert pst.main([str(tmp_path), "-o", str(out)]) == 0
    summ = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert summ["n_sessions"] == 5 and abs(summ["phase_seconds"]["generate"] - 9.0) < 1e-6 and summ["status"] == {"rejected": 2, "accepted": 3}
    assert abs(summ["unattributed_seconds"] - 5 * 0.7) < 1e-6 and abs(summ["session_seconds"]["max"] - 3.0) < 1e-9
    text = out.read_text()
    assert text.count("<rect") >= 5 * 3 and "generate" in text and "<svg" in text
    assert "no sessions" in pst.render_svg([])
