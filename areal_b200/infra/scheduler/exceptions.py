"""Exception taxonomy of worker scheduling (reference: ``areal/infra/scheduler/exceptions.py``)."""


class SchedulerError(RuntimeError):
    pass


class WorkerCreationError(SchedulerError):
    def __init__(self, role: str, reason: str, detail: str = ""):
        super().__init__(f"failed to create worker(s) for role '{role}': {reason}. {detail}")
        self.role, self.reason, self.detail = role, reason, detail


class WorkerFailedError(SchedulerError):
    def __init__(self, worker_id: str, exit_code, stderr: str = ""):
        super().__init__(f"worker '{worker_id}' failed with exit code {exit_code}. {stderr[-2000:]}")
        self.worker_id, self.exit_code = worker_id, exit_code


class WorkerNotFoundError(SchedulerError):
    def __init__(self, worker_id: str):
        super().__init__(f"worker '{worker_id}' not found")
        self.worker_id = worker_id


class WorkerTimeoutError(SchedulerError):
    def __init__(self, role: str, timeout: float):
        super().__init__(f"workers of role '{role}' not ready after {timeout:.0f}s")


class EngineCreationError(SchedulerError):
    def __init__(self, worker_id: str, reason: str, status: int = 0):
        super().__init__(f"engine creation failed on '{worker_id}' (HTTP {status}): {reason}")


class EngineCallError(SchedulerError):
    def __init__(self, worker_id: str, method: str, reason: str, attempt: int = 1):
        super().__init__(f"call '{method}' failed on '{worker_id}' (attempt {attempt}): {reason}")
        self.worker_id, self.method, self.reason = worker_id, method, reason


class RPCConnectionError(SchedulerError):
    pass


class GPUAllocationError(SchedulerError):
    pass
