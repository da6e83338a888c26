"""Worker scheduling contract (reference: ``areal/api/scheduler_api.py:13-329``)."""
from __future__ import annotations

import abc
from dataclasses import dataclass, field
from typing import Any, Optional

from .cli_args import SchedulingSpec, SchedulingStrategy


@dataclass
class Worker:
    id: str
    ip: str
    worker_ports: list[str] = field(default_factory=list)
    engine_ports: list[str] = field(default_factory=list)
    gpu_ids: list[int] = field(default_factory=list)

    @property
    def address(self) -> str:
        return f"{self.ip}:{self.worker_ports[0]}" if self.worker_ports else self.ip


@dataclass
class Job:
    replicas: int = 1
    tasks: list[SchedulingSpec] = field(default_factory=list)
    scheduling_strategy: SchedulingStrategy = field(default_factory=SchedulingStrategy)
    role: str = "worker"


class Scheduler(abc.ABC):
    @abc.abstractmethod
    def create_workers(self, job: Job, *args, **kwargs) -> list[str]:
        ...

    @abc.abstractmethod
    def get_workers(self, role: str, timeout: Optional[float] = None) -> list[Worker]:
        ...

    @abc.abstractmethod
    def delete_workers(self, role: Optional[str] = None):
        ...

    def fork_workers(self, role: str, target_role: str, command: Optional[str] = None) -> list[str]:
        raise NotImplementedError

    @abc.abstractmethod
    def create_engine(self, worker_id: str, engine: str, *args, **kwargs) -> Any:
        ...

    def set_worker_env(self, worker_id: str, env: dict[str, str]) -> None:
        raise NotImplementedError

    @abc.abstractmethod
    def call_engine(self, worker_id: str, method: str, *args, **kwargs) -> Any:
        ...

    @abc.abstractmethod
    async def async_call_engine(self, worker_id: str, method: str, *args, **kwargs) -> Any:
        ...
