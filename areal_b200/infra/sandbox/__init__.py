from .local import ExecResult, LocalSandbox, SandboxConfig, extract_code_blocks, run_python_tool

__all__ = ["LocalSandbox", "SandboxConfig", "ExecResult", "extract_code_blocks", "run_python_tool"]
