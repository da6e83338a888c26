"""Rollout runtime on CPU: executor ordering / accept filter / staleness gating, interruptible
generation with per-token versions, trajectory format check."""
import asyncio
import threading
import time

import pytest
import torch

from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeInferConfig
from areal_b200.api.io_struct import ModelRequest, ModelResponse
from areal_b200.api.workflow_api import RolloutWorkflow
from areal_b200.engine.infer_engine import NativeInferenceEngine
from areal_b200.models.config import preset
from areal_b200.rollout.executor import WorkflowExecutor, check_trajectory_format
from areal_b200.rollout.workflows.rlvr import RLVRWorkflow


class FakeEngine:
    """Minimal engine: echoes tokens after a delay; version is settable."""

    def __init__(self):
        self.v = 0

    def get_version(self):
        return self.v

    async def agenerate(self, req):
        await asyncio.sleep(req.metadata.get("delay", 0.01))
        return ModelResponse(input_tokens=req.input_ids, output_tokens=[1, 2], output_logprobs=[-0.1, -0.2],
                             output_versions=[self.v, self.v], stop_reason="stop")


class EchoWorkflow(RolloutWorkflow):
    async def arun_episode(self, engine, data):
        r = await engine.agenerate(ModelRequest(input_ids=data["input_ids"], metadata={"delay": data.get("delay", 0.01)}))
        if data.get("reject"):
            return None
        n = len(r.input_tokens) + 2
        return dict(input_ids=torch.tensor([r.input_tokens + r.output_tokens]), attention_mask=torch.ones(1, n, dtype=torch.bool),
                    rewards=torch.tensor([float(data.get("tag", 0))]), versions=torch.tensor([[-1] * len(r.input_tokens) + r.output_versions]))


def _executor(**kw):
    cfg = InferenceEngineConfig(max_concurrent_rollouts=kw.pop("mc", 8), consumer_batch_size=kw.pop("bs", 2),
                                max_head_offpolicyness=kw.pop("stale", 0), **kw)
    eng = FakeEngine()
    return WorkflowExecutor(cfg, eng).initialize(), eng


def test_submit_wait_and_rejects():
    ex, _ = _executor(stale=10)
    try:
        for i in range(4):
            ex.submit(dict(input_ids=[i], tag=i, reject=(i == 2)), EchoWorkflow())
        res = ex.wait(3, timeout=10)
        assert sorted(int(r["rewards"][0]) for r in res) == [0, 1, 3]
        assert ex.staleness.get_stats().rejected == 1
        with pytest.raises(TimeoutError):
            ex.wait(1, timeout=0.2)
    finally:
        ex.destroy()


def test_staleness_gates_admission_until_version_bumps():
    ex, eng = _executor(bs=2, stale=0, mc=16)
    try:
        for i in range(6):
            ex.submit(dict(input_ids=[i], tag=i), EchoWorkflow())
        first = ex.wait(2, timeout=10)
        time.sleep(0.3)
        assert ex.staleness.get_stats().accepted == 2          # budget (0+0+1)*2 exhausted
        assert ex.wait(1, timeout=0.2, raise_timeout=False) == []
        eng.v = 1
        second = ex.wait(2, timeout=10)
        assert len(first) == 2 and len(second) == 2
    finally:
        ex.destroy()


def test_pause_blocks_new_episodes_only():
    ex, _ = _executor(stale=10)
    try:
        ex.pause()
        ex.submit(dict(input_ids=[1]), EchoWorkflow())
        assert ex.wait(1, timeout=0.3, raise_timeout=False) == []
        ex.resume()
        assert len(ex.wait(1, timeout=10)) == 1
    finally:
        ex.destroy()


def test_failing_workflow_surfaces_in_caller():
    class Boom(RolloutWorkflow):
        async def arun_episode(self, engine, data):
            raise ValueError("boom")

    ex, _ = _executor(stale=10)
    try:
        ex.submit(dict(input_ids=[1]), Boom())
        with pytest.raises(RuntimeError):
            ex.wait(1, timeout=5)
    finally:
        ex.destroy()


def test_trajectory_format_check():
    good = dict(input_ids=torch.zeros(2, 5, dtype=torch.long), attention_mask=torch.ones(2, 5, dtype=torch.bool), rewards=torch.zeros(2))
    assert check_trajectory_format(good)
    with pytest.raises(ValueError):
        check_trajectory_format(dict(input_ids=torch.zeros(2, 5)))
    with pytest.raises(ValueError):
        check_trajectory_format(dict(good, logprobs=torch.zeros(2, 4)))
    with pytest.raises(ValueError):
        check_trajectory_format(good, expected_keys={"input_ids"})


def _cpu_engine(**kw):
    e = NativeInferenceEngine(InferenceEngineConfig(max_concurrent_rollouts=8, consumer_batch_size=4, max_head_offpolicyness=4),
                              NativeInferConfig(max_running_requests=8), model_config=preset("tiny-qwen2"), eos_token_id=kw.get("eos"))
    return e.initialize(device="cpu", start_executor=kw.get("executor", False))


def test_generation_budget_greedy_determinism_and_stop_ids():
    e = _cpu_engine()
    try:
        g = GenerationHyperparameters(max_new_tokens=5, max_tokens=64, greedy=True)

        async def run():
            a = await e.agenerate(ModelRequest(input_ids=[3, 4, 5], gconfig=g))
            b = await e.agenerate(ModelRequest(input_ids=[3, 4, 5], gconfig=g))
            c = await e.agenerate(ModelRequest(input_ids=[3, 4, 5], gconfig=g.new(stop_token_ids=[a.output_tokens[1]])))
            return a, b, c

        a, b, c = asyncio.run(run())
        assert a.output_tokens == b.output_tokens and len(a.output_tokens) == 5 and a.stop_reason == "length"
        first = a.output_tokens.index(a.output_tokens[1])
        assert c.stop_reason == "stop" and c.output_tokens == a.output_tokens[:first + 1]
        assert all(lp <= 0 for lp in a.output_logprobs)
        with pytest.raises(ValueError):
            asyncio.run(e.agenerate(ModelRequest(input_ids=list(range(70)), gconfig=g)))
    finally:
        e.destroy()


def test_interrupted_generation_carries_both_versions():
    e = _cpu_engine()
    try:
        g = GenerationHyperparameters(max_new_tokens=40, max_tokens=128)

        def interrupter():
            time.sleep(0.15)
            e.pause_generation()
            e.set_version(7)
            e.continue_generation()

        th = threading.Thread(target=interrupter)
        th.start()
        r = asyncio.run(e.agenerate(ModelRequest(input_ids=[1, 2, 3], gconfig=g)))
        th.join()
        assert len(r.output_tokens) == 40 == len(r.output_versions) == len(r.output_logprobs)
        assert set(r.output_versions) <= {0, 7} and r.output_versions == sorted(r.output_versions)
        assert e.stats["aborted"] >= 0
    finally:
        e.destroy()


def test_rlvr_workflow_through_engine_executor():
    e = _cpu_engine(executor=True)
    try:
        wf = RLVRWorkflow(lambda p, c, pi, ci, **kw: float(len(ci)), GenerationHyperparameters(n_samples=2, max_new_tokens=4, max_tokens=64),
                          reward_in_process=True)
        b = e.rollout_batch([dict(input_ids=[5, 6, 7]), dict(input_ids=[8, 9])], workflow=wf)
        assert b["input_ids"].shape[0] == 4 and b["rewards"].tolist() == [4.0] * 4
        lm, ver = b["loss_mask"], b["versions"]
        assert bool(((ver >= 0) == (lm == 1))[b["attention_mask"]].all())
        assert bool((b["logprobs"][lm == 0] == 0).all()) and bool((b["logprobs"][lm == 1] < 0).all())
    finally:
        e.destroy()
