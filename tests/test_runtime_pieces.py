"""Small runtime pieces the trainers lean on: the asyncio task runner behind the rollout executor, the reward
wrapper (time-outs, failures, pool rebuild), the learning-rate schedule, the statistics tracker (masked moments, scopes,
reduction over ranks) and the parameter count of a model configuration."""
import asyncio
import math
import os
import subprocess
import sys
import time

import pytest
import torch

from areal_b200.api.reward_api import AsyncRewardWrapper
from areal_b200.engine.optimizer import lr_lambda
from areal_b200.models.config import preset
from areal_b200.models.decoder import build_model
from areal_b200.rollout.task_runner import AsyncTaskRunner, TaskQueueFullError
from areal_b200.utils import stats_tracker
from areal_b200.utils.stats_tracker import DistributedStatsTracker, ReduceType

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ---------------------------------------------------------------- task runner
def _drain(r: AsyncTaskRunner, n: int, timeout: float = 10.0):
    out, t0 = [], time.monotonic()
    while len(out) < n and time.monotonic() - t0 < timeout:
        res = r.poll(0.05)
        if res is not None:
            out.append(res)
    return out


def test_task_runner_runs_concurrently_reports_errors_and_pauses():
    r = AsyncTaskRunner(max_queue_size=8)
    r.initialize()
    try:
        started = []

        def job(i, delay, fail=False):
            async def run():
                started.append(i)
                await asyncio.sleep(delay)
                if fail:
                    raise ValueError(f"boom {i}")
                return i * 10
            return run
        t0 = time.monotonic()
        ids = [r.submit(job(i, 0.3)) for i in range(4)] + [r.submit(job(9, 0.0, fail=True))]
        res = _drain(r, 5)
        assert time.monotonic() - t0 < 1.0                       # four 0.3 s jobs overlapped on one loop
        by_id = {x.task_id: x for x in res}
        assert sorted(by_id) == sorted(ids) and isinstance(by_id[ids[-1]].error, ValueError)
        assert sorted(x.data for x in res if x.error is None) == [0, 10, 20, 30]
        r.check_health()                                         # a failing task does not take the runner down
        r.pause()
        tid = r.submit(job(5, 0.0))
        time.sleep(0.2)
        assert r.is_paused() and 5 not in started and r.input_queue_size() == 1 and r.poll(0.05) is None
        r.resume()
        (late,) = _drain(r, 1)
        assert late.task_id == tid and late.data == 50 and r.running == 0
        assert r.submit(job(6, 0.0), task_id=777) == 777 and _drain(r, 1)[0].task_id == 777
    finally:
        r.destroy()


def test_task_runner_queue_bound_and_shutdown_hook():
    r = AsyncTaskRunner(max_queue_size=2)
    closed = []

    async def hook():
        closed.append(True)
    r.register_shutdown_hook(hook)
    r.pause()
    r.initialize()

    async def noop():
        return 1
    r.submit(lambda: noop())
    r.submit(lambda: noop())
    with pytest.raises(TaskQueueFullError):
        r.submit(lambda: noop())
    r.destroy()
    assert closed == [True]


# ---------------------------------------------------------------- reward wrapper
def _slow_reward(*a, **k):
    time.sleep(5)
    return 1.0


def _flaky_reward(*a, **k):
    raise RuntimeError("bad parse")


def _good_reward(prompt, completion, prompt_ids, completion_ids, bonus=0.0, **k):
    return len(completion) + bonus


def test_reward_wrapper_timeout_failure_and_keyword_passthrough():
    AsyncRewardWrapper.shutdown()

    async def main():
        good = AsyncRewardWrapper(_good_reward, use_threads=True)
        assert await good("p", "abc", [1], [2, 3], bonus=0.5) == 3.5
        slow = AsyncRewardWrapper(_slow_reward, timeout_seconds=0.2, use_threads=True)
        t0 = time.monotonic()
        assert await slow("p", "c", [], []) == 0.0 and time.monotonic() - t0 < 2.0
        bad = AsyncRewardWrapper(_flaky_reward, max_retries=2, use_threads=True)
        assert await bad("p", "c", [], []) == 0.0
        # many evaluations share the one pool
        vals = await asyncio.gather(*[good("p", "x" * i, [], []) for i in range(20)])
        assert vals == [float(i) for i in range(20)]
    asyncio.run(main())
    AsyncRewardWrapper.shutdown()


# ---------------------------------------------------------------- learning-rate schedule
@pytest.mark.parametrize("kind", ["constant", "linear", "cosine"])
def test_lr_schedule_warms_up_then_decays_to_the_floor(kind):
    total, warm, floor = 100, 10, 0.1
    v = [lr_lambda(s, total, warm, kind, floor) for s in range(total + 5)]
    assert v[0] == pytest.approx(0.0 if warm else 1.0, abs=0.11) and v[warm] == pytest.approx(1.0)
    assert all(b >= a - 1e-12 for a, b in zip(v[:warm], v[1:warm + 1]))          # monotone warm-up
    if kind == "constant":
        assert all(x == pytest.approx(1.0) for x in v[warm:])
    else:
        assert all(b <= a + 1e-12 for a, b in zip(v[warm:], v[warm + 1:]))      # monotone decay
        assert v[total] == pytest.approx(floor) and min(v[warm:]) >= floor - 1e-9 and v[-1] == pytest.approx(floor)
        mid = v[warm + (total - warm) // 2]
        want = floor + (1 - floor) * (0.5 if kind == "linear" else 0.5 * (1 + math.cos(math.pi * 0.5)))
        assert mid == pytest.approx(want, abs=0.02)
    assert lr_lambda(5, 100, 0, kind, floor) <= 1.0


# ---------------------------------------------------------------- statistics tracker
def test_stats_tracker_masked_moments_scopes_scalars_and_reset():
    t = DistributedStatsTracker("run")
    m = torch.tensor([True, True, False, True])
    x = torch.tensor([1.0, 3.0, 100.0, 5.0])
    with t.scope("actor"):
        t.denominator(tok=m)
        t.stat(denominator="tok", x=x)
        t.stat(denominator="tok", reduce_type=ReduceType.SUM, s=x)
        t.scalar(lr=0.5)
        t.scalar(lr=1.5)
        with pytest.raises(ValueError, match="bool"):
            t.denominator(bad=x)
        with pytest.raises(ValueError, match="not recorded"):
            t.stat(denominator="nope", y=x)
        with pytest.raises(ValueError, match="shape"):
            t.stat(denominator="tok", y=x[:2])
    out = t.export()
    assert out["run/actor/tok"] == 3.0
    assert out["run/actor/x/avg"] == pytest.approx(3.0) and out["run/actor/x/min"] == 1.0 and out["run/actor/x/max"] == 5.0
    assert out["run/actor/s"] == pytest.approx(9.0) and out["run/actor/lr"] == pytest.approx(1.0)
    assert t.export() == {}                                      # exporting resets
    with t.record_timing("step"):
        time.sleep(0.01)
    assert t.export()["timeperf/step"] >= 0.01
    # the module-level tracker is a named singleton
    assert stats_tracker.get("a") is stats_tracker.get("a") and stats_tracker.get("a") is not stats_tracker.get("b")


REDUCE_SCRIPT = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, %(root)r)
from areal_b200.utils.stats_tracker import DistributedStatsTracker
dist.init_process_group("gloo")
r = dist.get_rank()
t = DistributedStatsTracker()
m = torch.tensor([True, True, r == 0])
t.denominator(tok=m)
t.stat(denominator="tok", x=torch.tensor([1.0, 2.0, 30.0]) * (r + 1))
t.scalar(step_time=float(r + 1))
if r == 1:
    t.scalar(only_on_one=7.0)          # keys need not exist on every rank
sub = dist.new_group([0, 1])
out = t.export(reduce_group=sub if r < 2 else None) if r < 2 else t.export(distributed=False)
if r == 0:
    # tokens: 3 on rank 0 + 2 on rank 1; x: (1 + 2 + 30) + (2 + 4) over 5 tokens
    assert out["tok"] == 5.0 and abs(out["x/avg"] - 39.0 / 5) < 1e-6 and out["x/max"] == 30.0 and out["x/min"] == 1.0, out
    assert abs(out["step_time"] - 1.5) < 1e-9 and out["only_on_one"] == 7.0, out
if r == 2:
    assert out["tok"] == 2.0 and out["step_time"] == 3.0, out
print("STATS_OK", r, flush=True)
dist.barrier()
'''


def test_stats_tracker_reduces_over_a_subgroup(tmp_path):
    script = tmp_path / "stats.py"
    script.write_text(REDUCE_SCRIPT % dict(root=ROOT))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
                        "--master-port", "29951", str(script)], cwd=ROOT, capture_output=True, text=True, timeout=200,
                       env=dict(os.environ, OMP_NUM_THREADS="1"))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert r.stdout.count("STATS_OK") == 3


# ---------------------------------------------------------------- parameter counts
@pytest.mark.parametrize("name", ["tiny-qwen2", "tiny-qwen3", "tiny-qwen3-moe"])
def test_num_params_matches_the_built_model(name):
    cfg = preset(name)
    model = build_model(cfg, dtype=torch.float32, device="meta")
    n = sum(p.numel() for p in model.parameters())
    assert cfg.num_params() == n


def test_published_sizes_are_in_the_right_ballpark():
    assert 7.5e9 < preset("qwen3-8b").num_params() < 8.5e9
    assert 1.4e9 < preset("qwen2.5-1.5b").num_params() < 1.9e9


def test_small_config_switches_take_effect(tmp_path):
    """Fields that used to be accepted and ignored: evaluation before training, extra arguments of a custom lambda
    schedule, the session tracer's flush threshold, the pause grace period."""
    import json
    import os
    import time
    import types

    import torch

    from areal_b200.api.cli_args import EvaluatorConfig, InferenceEngineConfig, PPOActorConfig, SessionTracerConfig
    from areal_b200.algo.advantages import AdvantageComputer
    from areal_b200.engine.remote_engine import RemoteInfEngine
    from areal_b200.utils.evaluator import Evaluator
    from areal_b200.utils.perf_tracer import SessionTracer

    calls = []
    ev = Evaluator(EvaluatorConfig(freq_steps=100, eval_before_train=True))
    assert ev.evaluate(lambda: calls.append("pre") or 1, 0, -1, -1) == 1 and calls == ["pre"]
    assert Evaluator(EvaluatorConfig(freq_steps=100)).evaluate(lambda: calls.append("no"), 0, -1, -1) is None and calls == ["pre"]
    # a custom lambda schedule gets its configured keyword arguments
    mod = types.ModuleType("my_lambda_mod")
    mod.fn = lambda lengths, floor=0.0, scale=1.0: torch.full((lengths.numel(),), floor + scale)
    import sys

    sys.modules["my_lambda_mod"] = mod
    cfg = PPOActorConfig(gae_lambda="my_lambda_mod.fn", gae_lambda_kwargs={"floor": 0.5, "scale": 0.25})
    pipe = AdvantageComputer(cfg)
    lam = pipe._lambda(torch.ones(3, 4, dtype=torch.bool), torch.zeros(3, 4, dtype=torch.long))
    assert torch.allclose(lam, torch.full((3,), 0.75))
    # finished sessions reach the file as soon as the threshold is met
    st = SessionTracer(SessionTracerConfig(enabled=True, flush_threshold=2), rank=0, out_dir=str(tmp_path))
    a, b, c = st.register(1), st.register(2), st.register(3)
    st.finish(a, "accepted")
    assert not os.path.exists(tmp_path / "sessions.jsonl")
    st.finish(b, "rejected")
    rows = [json.loads(l) for l in open(tmp_path / "sessions.jsonl")]
    assert [r["status"] for r in rows] == ["accepted", "rejected"] and st._done == []
    st.finish(c, "accepted")
    assert len(st._done) == 1
    # the grace period after pausing
    eng = RemoteInfEngine(InferenceEngineConfig(pause_grace_period=0.3), [])
    t0 = time.time()
    eng.pause_generation()
    assert time.time() - t0 >= 0.3
    eng.continue_generation()
