from .local import ExecResult, LocalSandbox, SandboxConfig, extract_code_blocks, run_python_tool

from .remote import DaytonaRunner, RemoteSandbox, SandboxServer  # noqa: E402

__all__ = ["LocalSandbox", "SandboxConfig", "ExecResult", "extract_code_blocks", "run_python_tool", "SandboxServer", "RemoteSandbox",
           "DaytonaRunner"]
