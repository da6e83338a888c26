"""A reward that runs the model's code in a remote sandbox (``areal_b200/infra/sandbox/remote.py``): start a sandbox
server on a machine where untrusted code may run (``python -m areal_b200.v2.cli sandbox serve --port 8191``), point
``AREAL_SANDBOX_ADDR`` at it, and use ``code_reward_fn`` as the reward of an RLVR workflow. Reference:
``examples/sandbox_daytona/reward_example.py`` of the reference project."""
import os
import re

from areal_b200.infra.sandbox.remote import RemoteSandbox


def code_reward_fn(prompt, completions, prompt_ids, completion_ids, tests: str = "", timeout_s: float = 10.0, **kwargs) -> float:
    """1.0 when the last ```python block of the completion, followed by the record's ``tests``, exits with code 0."""
    blocks = re.findall(r"```python\n(.*?)```", completions or "", re.S)
    if not blocks:
        return 0.0
    box = RemoteSandbox(os.environ.get("AREAL_SANDBOX_ADDR", "127.0.0.1:8191"), api_key=os.environ.get("AREAL_SANDBOX_KEY"), timeout_s=timeout_s)
    res = box.run(blocks[-1] + "\n\n" + (tests or ""))
    return 1.0 if res.returncode == 0 and not res.timed_out else 0.0
