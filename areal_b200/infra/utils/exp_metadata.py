"""``version.json`` beside a trial's logs: which source state produced the run (commit, branch, dirty flag), the
experiment / trial names and whatever the caller adds (the resolved allocation string, the world size ...).

Reference: ``areal/infra/utils/exp_metadata.py``.
"""
from __future__ import annotations

import getpass
import json
import os
import time
from typing import Optional

from ...version import version_info


def metadata_dir(fileroot: str, experiment_name: str, trial_name: str) -> str:
    path = os.path.join(fileroot, "logs", getpass.getuser(), experiment_name, trial_name)
    os.makedirs(path, exist_ok=True)
    return path


def save_experiment_metadata(fileroot: str, experiment_name: str, trial_name: str, additional: Optional[dict] = None) -> str:
    meta = {"commit_id": version_info.commit, "branch": version_info.branch, "is_dirty": version_info.is_dirty,
            "version": version_info.full_version_with_dirty_description, "experiment_name": experiment_name, "trial_name": trial_name,
            "saved_at": time.strftime("%Y-%m-%dT%H:%M:%S")}
    meta.update(additional or {})
    path = os.path.join(metadata_dir(fileroot, experiment_name, trial_name), "version.json")
    with open(path, "w") as f:
        json.dump(meta, f, indent=2, default=str)
    return path


def load_experiment_metadata(fileroot: str, experiment_name: str, trial_name: str) -> Optional[dict]:
    path = os.path.join(metadata_dir(fileroot, experiment_name, trial_name), "version.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        return json.load(f)
