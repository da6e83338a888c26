"""Readable records of finished trajectories (``rollout.dump_to_file``).

One JSON line per sample under ``<log dir>/rollout/<newest weight version in the batch>/<task id>.jsonl`` (``eval-rollout``
for evaluation episodes): lengths, reward, the oldest and newest weight version among the generated tokens with a
run-length list of versions (how stale each part of the answer is), and, when a tokenizer is configured, the decoded
prompt and completion; multi-turn samples also list their alternating prompt / generated / context segments.

Reference: ``areal/infra/workflow_executor.py:844-1030`` (``_get_dump_dir``, ``_compute_output_versions``,
``_split_trajectory_for_dump``, ``_dump_trajectory``).
"""
from __future__ import annotations

import json
import os
from typing import Any, Optional


def mask_runs(mask: list[int]) -> list[tuple[int, int, int]]:
    """Maximal runs of equal values: ``(value, start, end)``."""
    runs, start = [], 0
    for i in range(1, len(mask) + 1):
        if i == len(mask) or mask[i] != mask[start]:
            runs.append((int(mask[start]), start, i))
            start = i
    return runs


def version_summary(versions: list[int], mask: list[int]) -> tuple[int, int, list[list[int]]]:
    """(oldest, newest, run-length list ``[version, count]``) over the generated tokens (``mask == 1``); ``-1`` when
    nothing was generated."""
    gen = [int(v) for v, m in zip(versions, mask) if m == 1]
    if not gen:
        return -1, -1, []
    rle: list[list[int]] = []
    for v in gen:
        if rle and rle[-1][0] == v:
            rle[-1][1] += 1
        else:
            rle.append([v, 1])
    return min(gen), max(gen), rle


def split_for_dump(ids: list[int], mask: list[int], tokenizer) -> dict[str, Any]:
    """Prompt / completion text of one sample; ``segments`` (role ``prompt`` | ``gen`` | ``context``, length, text) only
    when the sample has more than one generated run (multi-turn), so the common case decodes twice."""
    if len(ids) != len(mask):
        raise ValueError(f"ids length {len(ids)} != mask length {len(mask)}")
    runs = mask_runs(mask)
    first_gen = next((a for v, a, _ in runs if v == 1), len(ids))
    dec = lambda a, b: tokenizer.decode(ids[a:b], skip_special_tokens=False)      # noqa: E731
    out = {"prompt_end": first_gen, "prompt_text": dec(0, first_gen), "completion_text": dec(first_gen, len(ids)), "segments": None}
    if sum(1 for v, _, _ in runs if v == 1) > 1:
        segs = []
        for k, (v, a, b) in enumerate(runs):
            role = "gen" if v == 1 else ("prompt" if not any(s["role"] == "prompt" for s in segs) and k == 0 else "context")
            segs.append({"role": role, "len": b - a, "text": dec(a, b)})
        out["segments"] = segs
    return out


def trajectory_records(traj: dict[str, Any], task_id: int, tokenizer=None, default_version: int = 0) -> tuple[int, list[dict]]:
    """(newest version in the batch, one record per sample that generated something)."""
    ids, am, lm, rewards = (traj.get(k) for k in ("input_ids", "attention_mask", "loss_mask", "rewards"))
    if ids is None or am is None or lm is None or rewards is None:
        raise KeyError("a trajectory needs input_ids, attention_mask, loss_mask and rewards to be dumped")
    versions = traj.get("versions")
    newest = int(versions.max()) if versions is not None and versions.numel() else int(default_version)
    orig = traj.get("original_rewards")
    recs = []
    for i in range(ids.shape[0]):
        n = int(am[i].sum())
        if n == 0:
            continue
        row, mask = ids[i, :n].tolist(), [int(x) for x in lm[i, :n].tolist()]
        if mask[-1] != 1:                    # nothing generated at the end: an empty completion
            continue
        if versions is not None:
            head, tail, rle = version_summary(versions[i, :n].tolist(), mask)
        else:
            head = tail = int(default_version)
            rle = [[int(default_version), sum(mask)]]
        rec = {"task_id": task_id, "sample_idx": i, "seqlen": n, "prompt_len": mask.index(1), "head_version": head, "tail_version": tail,
               "version_rle": rle, "reward": float(rewards[i])}
        if tokenizer is not None:
            sp = split_for_dump(row, mask, tokenizer)
            rec.update(prompt=sp["prompt_text"], completion=sp["completion_text"])
            if sp["segments"] is not None:
                rec["segments"] = sp["segments"]
        else:
            rec["input_ids"] = row
        if orig is not None:
            rec["original_reward"] = float(orig[i])
        recs.append(rec)
    return newest, recs


def dump_dir(config, is_eval: bool) -> Optional[str]:
    from ..utils.stats_logger import StatsLogger

    if not getattr(config, "fileroot", None):
        return None
    return os.path.join(StatsLogger.get_log_path(config), "eval-rollout" if is_eval else "rollout")


def dump_trajectory(traj: dict[str, Any], task_id: int, root: str, tokenizer=None, default_version: int = 0) -> str:
    newest, recs = trajectory_records(traj, task_id, tokenizer, default_version)
    d = os.path.join(root, str(newest))
    os.makedirs(d, exist_ok=True)
    path = os.path.join(d, f"{task_id}.jsonl")
    with open(path, "a") as f:
        for r in recs:
            f.write(json.dumps(r) + "\n")
    return path
