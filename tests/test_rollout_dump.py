"""Trajectory dump records: version summaries, prompt / completion split, multi-turn segments, the files written."""
import json
import os

import pytest
import torch

from areal_b200.rollout import dump as D


class _Tok:
    def decode(self, ids, **kw):
        return f"[{len(ids)} tokens]"


def test_mask_runs_and_version_summary():
    assert D.mask_runs([0, 0, 1, 1, 0, 1]) == [(0, 0, 2), (1, 2, 4), (0, 4, 5), (1, 5, 6)]
    assert D.mask_runs([]) == [] and D.mask_runs([1]) == [(1, 0, 1)]
    assert D.version_summary([-1, -1, 3, 3, 4, 4, 4], [0, 0, 1, 1, 1, 1, 1]) == (3, 4, [[3, 2], [4, 3]])
    assert D.version_summary([5, 5], [0, 0]) == (-1, -1, [])
    # versions of masked-out (context) tokens never count, and equal versions separated by context merge into one run
    assert D.version_summary([0, 2, 9, 2, 3], [0, 1, 0, 1, 1]) == (2, 3, [[2, 2], [3, 1]])


def test_single_turn_split_decodes_twice_and_has_no_segments():
    r = D.split_for_dump([1, 2, 3, 4, 5, 6], [0, 0, 0, 1, 1, 1], _Tok())
    assert r == {"prompt_end": 3, "prompt_text": "[3 tokens]", "completion_text": "[3 tokens]", "segments": None}
    r = D.split_for_dump([1, 2], [0, 0], _Tok())                # nothing generated: everything is prompt
    assert r["prompt_end"] == 2 and r["completion_text"] == "[0 tokens]"
    with pytest.raises(ValueError, match="mask length"):
        D.split_for_dump([1, 2, 3], [0, 1], _Tok())


def test_multi_turn_split_lists_prompt_gen_context_segments():
    r = D.split_for_dump(list(range(8)), [0, 0, 1, 1, 0, 0, 1, 1], _Tok())
    assert r["prompt_end"] == 2 and [s["role"] for s in r["segments"]] == ["prompt", "gen", "context", "gen"]
    assert [s["len"] for s in r["segments"]] == [2, 2, 2, 2]
    r = D.split_for_dump(list(range(5)), [1, 1, 0, 1, 1], _Tok())   # starts with generated tokens: no prompt segment at all
    assert r["prompt_end"] == 0 and [s["role"] for s in r["segments"]] == ["gen", "context", "gen"]


def test_dump_trajectory_writes_one_line_per_generated_sample(tmp_path):
    ids = torch.tensor([[5, 6, 7, 8, 0, 0], [1, 2, 3, 4, 5, 6], [9, 9, 9, 0, 0, 0]])
    am = torch.tensor([[1, 1, 1, 1, 0, 0], [1, 1, 1, 1, 1, 1], [1, 1, 1, 0, 0, 0]])
    lm = torch.tensor([[0, 0, 1, 1, 0, 0], [0, 1, 1, 0, 1, 1], [0, 0, 0, 0, 0, 0]])
    ver = torch.tensor([[-1, -1, 4, 5, -1, -1], [-1, 3, 3, -1, 5, 5], [-1, -1, -1, -1, -1, -1]])
    traj = dict(input_ids=ids, attention_mask=am, loss_mask=lm, versions=ver, rewards=torch.tensor([1.0, 0.5, 0.0]),
                original_rewards=torch.tensor([2.0, 1.0, 0.0]))
    path = D.dump_trajectory(traj, 17, str(tmp_path), _Tok())
    assert path == os.path.join(str(tmp_path), "5", "17.jsonl")           # the directory is named for the newest version in the batch
    recs = [json.loads(l) for l in open(path)]
    assert [r["sample_idx"] for r in recs] == [0, 1]                       # the third sample generated nothing
    a, b = recs
    assert (a["seqlen"], a["prompt_len"], a["head_version"], a["tail_version"], a["version_rle"]) == (4, 2, 4, 5, [[4, 1], [5, 1]])
    assert a["reward"] == 1.0 and a["original_reward"] == 2.0 and a["prompt"] == "[2 tokens]" and "segments" not in a
    assert (b["head_version"], b["tail_version"], b["version_rle"]) == (3, 5, [[3, 2], [5, 2]]) and len(b["segments"]) == 4
    # no tokenizer: token ids instead of text; no versions: the engine's current version for every generated token
    del traj["versions"]
    p2 = D.dump_trajectory(traj, 18, str(tmp_path), None, default_version=7)
    r2 = [json.loads(l) for l in open(p2)]
    assert p2.endswith(os.path.join("7", "18.jsonl")) and r2[0]["input_ids"] == [5, 6, 7, 8] and r2[0]["version_rle"] == [[7, 2]]
    with pytest.raises(KeyError):
        D.trajectory_records({"input_ids": ids}, 1)


def test_executor_dumps_accepted_trajectories(tmp_path):
    """``dump_to_file`` end to end through the workflow executor with a stub engine and workflow."""
    import asyncio  # noqa: F401

    from areal_b200.api.cli_args import InferenceEngineConfig
    from areal_b200.api.workflow_api import RolloutWorkflow
    from areal_b200.rollout.executor import WorkflowExecutor

    class Eng:
        def get_version(self):
            return 2

    class WF(RolloutWorkflow):
        async def arun_episode(self, engine, data):
            return dict(input_ids=torch.tensor([[1, 2, 3, 4]]), attention_mask=torch.ones(1, 4, dtype=torch.long),
                        loss_mask=torch.tensor([[0, 0, 1, 1]]), versions=torch.tensor([[-1, -1, 2, 2]]), rewards=torch.tensor([1.0]))

    cfg = InferenceEngineConfig(dump_to_file=True, fileroot=str(tmp_path), experiment_name="e", trial_name="t", consumer_batch_size=1,
                                max_concurrent_rollouts=2)
    ex = WorkflowExecutor(cfg, Eng())
    ex.initialize()
    try:
        ex.submit({"x": 1}, workflow=WF())
        out = ex.wait(1, timeout=30)
        assert out is not None
    finally:
        ex.destroy()
    files = [os.path.join(dp, f) for dp, _, fs in os.walk(str(tmp_path)) for f in fs if f.endswith(".jsonl")]
    assert len(files) == 1 and os.sep + "rollout" + os.sep + "2" + os.sep in files[0]
    rec = json.loads(open(files[0]).read().strip())
    assert rec["prompt_len"] == 2 and rec["tail_version"] == 2 and rec["input_ids"] == [1, 2, 3, 4]


def test_stats_logger_feeds_trackio_and_swanlab_when_importable(tmp_path, monkeypatch):
    """Both trackers are driven through the wandb-shaped calls (init / log / finish); a missing package only warns."""
    import sys
    import types

    from areal_b200.api.cli_args import StatsLoggerConfig, TrackioConfig
    from areal_b200.utils.stats_logger import StatsLogger

    calls = []
    fake = types.ModuleType("trackio")
    fake.init = lambda **kw: calls.append(("init", kw))
    fake.log = lambda d, step=None: calls.append(("log", dict(d), step))
    fake.finish = lambda: calls.append(("finish",))
    monkeypatch.setitem(sys.modules, "trackio", fake)
    monkeypatch.setitem(sys.modules, "swanlab", None)                      # import fails: logged, not raised
    cfg = StatsLoggerConfig(experiment_name="exp", trial_name="t1", fileroot=str(tmp_path))
    cfg.trackio = TrackioConfig(mode="local", space_id="me/space")
    cfg.swanlab.mode = "local"
    lg = StatsLogger(cfg, None)
    lg.commit(0, 0, 0, {"loss": 1.5})
    lg.commit(0, 1, 1, [{"loss": 1.25}, {"lr": 0.1}])
    lg.close()
    assert calls[0] == ("init", {"project": "exp", "name": "t1", "space_id": "me/space"})
    assert calls[1] == ("log", {"loss": 1.5}, 0) and calls[2] == ("log", {"loss": 1.25, "lr": 0.1}, 1) and calls[3] == ("finish",)
    with pytest.raises(ValueError, match="trackio.mode"):
        TrackioConfig(mode="cloud")


def test_stats_logger_passes_the_wandb_section_through(tmp_path, monkeypatch):
    import sys
    import types

    from areal_b200.api.cli_args import StatsLoggerConfig
    from areal_b200.utils.stats_logger import StatsLogger

    calls = {}
    fake = types.ModuleType("wandb")
    fake.init = lambda **kw: calls.update(init=kw)
    fake.log = lambda d, step=None: calls.setdefault("log", []).append((dict(d), step))
    fake.finish = lambda: calls.update(finished=True)
    monkeypatch.setitem(sys.modules, "wandb", fake)
    monkeypatch.delenv("WANDB_BASE_URL", raising=False)
    cfg = StatsLoggerConfig(experiment_name="exp", trial_name="t1", fileroot=str(tmp_path))
    cfg.wandb.mode, cfg.wandb.wandb_base_url, cfg.wandb.job_type, cfg.wandb.tags, cfg.wandb.config = "offline", "http://wb.local", "rl", ["a"], {"k": 1}
    lg = StatsLogger(cfg, None, exp_config={"lr": 0.1})
    lg.commit(0, 0, 0, {"loss": 1.0})
    lg.close()
    i = calls["init"]
    assert i["id"] == "exp_t1_train" and i["resume"] == "allow" and i["job_type"] == "rl" and i["tags"] == ["a"] and i["config"] == {"k": 1, "lr": 0.1}
    assert i["group"] == "exp_t1" and os.environ["WANDB_BASE_URL"] == "http://wb.local" and calls["log"] == [({"loss": 1.0}, 0)] and calls["finished"]
