"""Public contracts: engines, workflows, configs, allocation strings, io records."""
from .alloc_mode import (AllocationMode, AllocationType, FSDPParallelStrategy, MegatronParallelStrategy,
                         ModelAllocation, ParallelStrategy)
from .engine_api import InferenceEngine, TrainEngine
from .io_struct import (FinetuneSpec, LocalInfServerInfo, ModelRequest, ModelResponse, ParamSpec, RolloutStat,
                        SaveLoadMeta, StepInfo, WeightUpdateMeta)
from .scheduler_api import Job, Scheduler, Worker
from .workflow_api import AgentWorkflow, RolloutWorkflow, WorkflowLike


def __getattr__(name):
    if name == "AsyncRewardWrapper":
        from .reward_api import AsyncRewardWrapper

        return AsyncRewardWrapper
    raise AttributeError(name)
