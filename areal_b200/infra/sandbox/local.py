"""Code-execution sandbox for tool-use rollouts and code rewards: runs untrusted Python in a
child process with wall-clock, CPU-time, memory and output limits, no network-facing
environment, and a scratch working directory that is removed afterwards. Reference:
``areal/infra/sandbox/*`` (local backend; the hosted Daytona backend needs a network service
and is represented by the same interface)."""
from __future__ import annotations

import asyncio
import os
import re
import resource
import shutil
import subprocess
import sys
import tempfile
import time
from dataclasses import dataclass, field
from typing import Optional


@dataclass
class SandboxConfig:
    timeout_s: float = 10.0
    cpu_time_s: int = 10
    memory_mb: int = 1024
    max_output_bytes: int = 64 * 1024
    python: str = sys.executable
    env: dict = field(default_factory=dict)
    allow_network_env: bool = False


@dataclass
class ExecResult:
    stdout: str
    stderr: str
    returncode: int
    timed_out: bool
    seconds: float

    @property
    def ok(self) -> bool:
        return self.returncode == 0 and not self.timed_out


_CODE_RE = re.compile(r"```(?:python|py)?\s*\n(.*?)```", re.S)


def extract_code_blocks(text: str) -> list[str]:
    return [m.group(1).strip() for m in _CODE_RE.finditer(text)]


class LocalSandbox:
    def __init__(self, config: Optional[SandboxConfig] = None):
        self.cfg = config or SandboxConfig()

    def _limits(self):
        c = self.cfg

        def fn():
            os.setsid()
            resource.setrlimit(resource.RLIMIT_CPU, (c.cpu_time_s, c.cpu_time_s))
            mem = c.memory_mb * 1024 * 1024
            resource.setrlimit(resource.RLIMIT_AS, (mem, mem))
            resource.setrlimit(resource.RLIMIT_FSIZE, (16 * 1024 * 1024, 16 * 1024 * 1024))
            resource.setrlimit(resource.RLIMIT_NPROC, (64, 64)) if os.getuid() != 0 else None
        return fn

    def run(self, code: str, stdin: str = "", files: Optional[dict[str, str]] = None) -> ExecResult:
        c = self.cfg
        work = tempfile.mkdtemp(prefix="areal_sbx_")
        try:
            for name, content in (files or {}).items():
                p = os.path.join(work, os.path.basename(name))
                with open(p, "w") as f:
                    f.write(content)
            with open(os.path.join(work, "main.py"), "w") as f:
                f.write(code)
            env = {"PATH": os.environ.get("PATH", "/usr/bin:/bin"), "HOME": work, "PYTHONDONTWRITEBYTECODE": "1", "PYTHONHASHSEED": "0",
                   "OMP_NUM_THREADS": "1"}
            if not c.allow_network_env:
                env.update({"http_proxy": "http://127.0.0.1:9", "https_proxy": "http://127.0.0.1:9", "no_proxy": ""})
            env.update(c.env)
            t0 = time.monotonic()
            p = subprocess.Popen([c.python, "-I", "main.py"], cwd=work, env=env, stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                                 stderr=subprocess.PIPE, preexec_fn=self._limits())
            try:
                out, err = p.communicate(stdin.encode(), timeout=c.timeout_s)
                timed_out = False
            except subprocess.TimeoutExpired:
                try:
                    os.killpg(p.pid, 9)             # the child is its own session leader
                except ProcessLookupError:
                    pass
                out, err = p.communicate()
                timed_out = True
            dt = time.monotonic() - t0
            cut = c.max_output_bytes
            return ExecResult(out[:cut].decode(errors="replace"), err[:cut].decode(errors="replace"), p.returncode if p.returncode is not None else -9,
                              timed_out, dt)
        finally:
            shutil.rmtree(work, ignore_errors=True)

    async def arun(self, code: str, stdin: str = "", files: Optional[dict[str, str]] = None) -> ExecResult:
        return await asyncio.get_running_loop().run_in_executor(None, self.run, code, stdin, files)


def run_python_tool(arguments: dict, sandbox: Optional[LocalSandbox] = None) -> str:
    """Tool implementation for agents: ``{"code": "..."}`` -> text the model sees."""
    r = (sandbox or LocalSandbox()).run(arguments.get("code", ""), arguments.get("stdin", ""))
    if r.timed_out:
        return f"[timed out after {r.seconds:.1f}s]\n{r.stdout}"
    if r.returncode != 0:
        return f"[exit code {r.returncode}]\n{r.stdout}{r.stderr[-2000:]}"
    return r.stdout


def code_exec_reward_fn(prompt, completion, prompt_ids, completion_ids, tests: Optional[list[dict]] = None, **kwargs) -> float:
    """Fraction of ``tests`` (``{"stdin": ..., "expected": ...}``) the last code block of the
    completion passes."""
    blocks = extract_code_blocks(completion or "")
    if not blocks or not tests:
        return 0.0
    sbx = LocalSandbox(SandboxConfig(timeout_s=float(kwargs.get("timeout_s", 5.0))))
    ok = 0
    for t in tests:
        r = sbx.run(blocks[-1], t.get("stdin", ""))
        ok += int(r.ok and r.stdout.strip() == str(t.get("expected", "")).strip())
    return ok / len(tests)
