"""Abstract contracts of training and inference engines.

Method names and call semantics mirror the reference's ``areal/api/engine_api.py``
(``TrainEngine`` :32-548, ``InferenceEngine`` :551-1027) so trainers, workflows and user
scripts written against it run on this framework's engines.
"""
from __future__ import annotations

import abc
from concurrent.futures import Future
from typing import TYPE_CHECKING, Any, Callable, Optional

import torch

from .io_struct import (DeviceRuntimeInfo, FinetuneSpec, ModelRequest, ModelResponse, ParamSpec, SaveLoadMeta,
                        WeightUpdateMeta)

if TYPE_CHECKING:  # pragma: no cover
    from .alloc_mode import ParallelStrategy
    from .workflow_api import RolloutWorkflow


class TrainEngine(abc.ABC):
    """A model + optimizer that can run forward/backward over packed micro-batches."""

    # ---- lifecycle
    def create_process_group(self, parallel_strategy: "Optional[ParallelStrategy]" = None):
        raise NotImplementedError

    def initialize(self, addr: Optional[str] = None, ft_spec: Optional[FinetuneSpec] = None, **kwargs):
        raise NotImplementedError

    def destroy(self):
        pass

    # ---- topology
    @property
    def data_parallel_group(self):
        raise NotImplementedError

    @property
    def data_parallel_rank(self) -> int:
        raise NotImplementedError

    @property
    def data_parallel_world_size(self) -> int:
        raise NotImplementedError

    def current_data_parallel_head(self) -> int:
        raise NotImplementedError

    def is_data_parallel_head(self) -> bool:
        raise NotImplementedError

    @property
    def context_and_model_parallel_group(self):
        raise NotImplementedError

    @property
    def cpu_group(self):
        raise NotImplementedError

    # ---- modes
    def train(self, mode: bool = True):
        raise NotImplementedError

    def eval(self):
        return self.train(False)

    # ---- weights / versions
    def update_weights(self, meta: WeightUpdateMeta):
        raise NotImplementedError

    def connect_engine(self, engine: "InferenceEngine", meta: WeightUpdateMeta):
        raise NotImplementedError

    def rollout_batch(self, data: list[dict[str, Any]], workflow=None, workflow_kwargs=None,
                      should_accept_fn=None) -> dict[str, Any]:
        raise NotImplementedError

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None,
                      dynamic_bs: bool = False) -> dict[str, Any]:
        raise NotImplementedError

    def set_version(self, version: int):
        raise NotImplementedError

    def get_version(self) -> int:
        raise NotImplementedError

    def save(self, meta: SaveLoadMeta):
        raise NotImplementedError

    def load(self, meta: SaveLoadMeta):
        raise NotImplementedError

    # ---- optimisation
    def optimizer_zero_grad(self):
        raise NotImplementedError

    def optimizer_step(self) -> dict[str, float]:
        raise NotImplementedError

    def lr_scheduler_step(self):
        raise NotImplementedError

    def step_lr_scheduler(self):
        return self.lr_scheduler_step()

    def forward_backward_batch(self, mb_list, process_output_fn: Callable, forward_only: bool = False):
        raise NotImplementedError

    def train_batch(self, input_: dict[str, Any], loss_fn: Callable[..., torch.Tensor],
                    loss_weight_fn: Callable[[dict[str, Any]], torch.Tensor]) -> dict[str, float]:
        """One optimizer step over ``input_`` split into micro-batches; the loss of each
        micro-batch is weighted by ``loss_weight_fn`` so the result is a global mean."""
        raise NotImplementedError

    @torch.no_grad()
    def eval_batch(self, input_: dict[str, Any], loss_fn: Callable, loss_weight_fn: Callable) -> Optional[torch.Tensor]:
        raise NotImplementedError

    @torch.no_grad()
    def forward_batch(self, input_: dict[str, Any], output_seqlens: Optional[list[int]] = None,
                      aggregate_fn: Callable = torch.cat) -> Any:
        raise NotImplementedError

    def forward(self, *args, **kwargs):
        return self.forward_batch(*args, **kwargs)

    # ---- stats / memory
    def export_stats(self) -> dict[str, float]:
        from ..utils import stats_tracker

        return stats_tracker.export_all(reduce_group=getattr(self, "_stats_group", None))

    def onload(self):
        raise NotImplementedError

    def offload(self):
        raise NotImplementedError

    def get_device_stats(self) -> DeviceRuntimeInfo:
        return DeviceRuntimeInfo.get_current()

    def clear_batches(self, *args, **kwargs):
        pass

    def config_perf_tracer(self, config, rank: int, role: str) -> None:
        from ..utils import perf_tracer

        perf_tracer.configure(config, rank=rank, role=role)

    def save_perf_tracer(self, step: Optional[int] = None, force: bool = False) -> None:
        from ..utils import perf_tracer

        perf_tracer.save(step=step, force=force)


class InferenceEngine(abc.ABC):
    """A generation service with asynchronous request handling and weight hot-swap."""

    def initialize(self, *args, **kwargs):
        raise NotImplementedError

    def destroy(self):
        pass

    @property
    def initialized(self) -> bool:
        return True

    def launch_server(self, server_args: dict[str, Any]):
        raise NotImplementedError

    def teardown_server(self):
        pass

    async def agenerate(self, req: ModelRequest) -> ModelResponse:
        raise NotImplementedError

    def init_weights_update_group(self, meta: WeightUpdateMeta) -> Future:
        raise NotImplementedError

    def update_weights_from_distributed(self, meta: WeightUpdateMeta, param_specs: list[ParamSpec]) -> Future:
        raise NotImplementedError

    def update_weights_from_disk(self, meta: WeightUpdateMeta) -> Future:
        raise NotImplementedError

    def update_weights_from_tensors(self, named_tensors, meta: Optional[WeightUpdateMeta] = None) -> Future:
        raise NotImplementedError

    def set_version(self, version: int) -> None:
        raise NotImplementedError

    def get_version(self) -> int:
        raise NotImplementedError

    def compute_logp(self, *args, **kwargs):
        raise NotImplementedError

    def submit(self, data: dict[str, Any], workflow=None, workflow_kwargs=None, should_accept_fn=None,
               task_id: Optional[int] = None, is_eval: bool = False) -> int:
        raise NotImplementedError

    def wait(self, count: int, timeout: Optional[float] = None, raise_timeout: bool = True) -> list:
        raise NotImplementedError

    def wait_for_task(self, task_id: int, timeout: Optional[float] = None, raise_timeout: bool = True):
        raise NotImplementedError

    def rollout_batch(self, data: list[dict[str, Any]], workflow=None, workflow_kwargs=None,
                      should_accept_fn=None) -> dict[str, Any]:
        raise NotImplementedError

    def prepare_batch(self, dataloader, workflow=None, workflow_kwargs=None, should_accept_fn=None,
                      dynamic_bs: bool = False) -> dict[str, Any]:
        raise NotImplementedError

    def pause_generation(self):
        raise NotImplementedError

    def continue_generation(self):
        raise NotImplementedError

    def pause(self):
        raise NotImplementedError

    def resume(self):
        raise NotImplementedError

    def offload(self, tags: Optional[list[str]] = None):
        raise NotImplementedError

    def onload(self, tags: Optional[list[str]] = None):
        raise NotImplementedError

    def export_stats(self) -> dict[str, float]:
        from ..utils import stats_tracker

        return stats_tracker.export_all(distributed=False)
