"""Request / response / metadata records exchanged between trainers, engines, workflows
and the weight-update service.

Field names and semantics follow the reference's ``areal/api/io_struct.py`` (ModelRequest
:28, ModelResponse :63, FinetuneSpec :134, ParamSpec :150, WeightUpdateMeta :183,
HttpRequest :311, HttpGenerationResult :323, SaveLoadMeta :362, RolloutStat :373,
StepInfo :381) so user workflows written against it keep working.
"""
from __future__ import annotations

import math
import os
import uuid
from dataclasses import dataclass, field
from typing import TYPE_CHECKING, Any, Literal, Optional

if TYPE_CHECKING:  # pragma: no cover
    from .cli_args import GenerationHyperparameters


@dataclass
class ModelRequest:
    rid: str = field(default_factory=lambda: str(uuid.uuid4()))
    input_ids: list[int] = field(default_factory=list)
    gconfig: "GenerationHyperparameters" = None  # type: ignore[assignment]
    metadata: dict[str, Any] = field(default_factory=dict)
    tokenizer: Any = None
    image_data: Optional[list] = None
    processor: Any = None
    vision_msg_vllm: Optional[list] = None

    def __post_init__(self):
        if self.gconfig is None:
            from .cli_args import GenerationHyperparameters

            self.gconfig = GenerationHyperparameters()

    def copy(self) -> "ModelRequest":
        return ModelRequest(
            rid=self.rid, input_ids=list(self.input_ids), gconfig=self.gconfig.new(),
            metadata=dict(self.metadata), tokenizer=self.tokenizer,
            image_data=None if self.image_data is None else list(self.image_data),
            processor=self.processor, vision_msg_vllm=self.vision_msg_vllm,
        )


@dataclass
class ModelResponse:
    """Result of one (possibly interrupted and resumed) generation.

    ``output_versions[i]`` is the weight version that produced ``output_tokens[i]``; a
    response that straddled a weight update carries several versions."""

    input_tokens: list[int] = field(default_factory=list)
    output_tokens: list[int] = field(default_factory=list)
    output_logprobs: list[float] = field(default_factory=list)
    output_versions: list[int] = field(default_factory=list)
    stop_reason: Literal["length", "stop", "tool_calls", "abort", "interrupt"] = "stop"
    input_images: Optional[list] = None
    tokenizer: Any = None
    processor: Any = None
    latency: float = float("inf")
    ttft: float = float("inf")
    itl: list[float] = field(default_factory=list)
    routed_experts: Any = None
    metadata: dict[str, Any] = field(default_factory=dict)

    @property
    def input_len(self) -> int:
        return len(self.input_tokens)

    @property
    def output_len(self) -> int:
        return len(self.output_tokens)


@dataclass
class FinetuneSpec:
    total_train_epochs: int
    dataset_size: int
    train_batch_size: int

    @property
    def total_train_steps(self) -> int:
        return self.total_train_epochs * self.steps_per_epoch

    @property
    def steps_per_epoch(self) -> int:
        return max(1, self.dataset_size // self.train_batch_size)


@dataclass
class ParamSpec:
    name: str
    shape: tuple
    dtype: str

    @property
    def size(self) -> int:
        """Bytes occupied by the parameter."""
        width = {"bfloat16": 2, "float16": 2, "float32": 4, "float8_e4m3fn": 1, "float8_e5m2": 1,
                 "int8": 1, "uint8": 1, "int32": 4, "int64": 8}.get(self.dtype.replace("torch.", ""), 2)
        return int(math.prod(self.shape)) * width


@dataclass
class WeightUpdateMeta:
    """How new weights travel from the trainer to the rollout engines.

    ``type``:
      * ``disk``  - HF safetensors written to ``path`` and loaded by the servers;
      * ``xccl``  - collective broadcast (kept as the measured baseline);
      * ``p2p``   - shard-direct push over NVLink peer memory with in-kernel reshard/cast
                    (the native path of this framework; takes the role of ``awex``).
    """

    type: Literal["disk", "xccl", "p2p", "awex", "shared"] = "p2p"
    path: Optional[str] = None
    alloc_mode: Any = None
    nccl_master_address: str = "127.0.0.1"
    nccl_master_port: int = 29500
    nccl_param_specs: list[list[ParamSpec]] = field(default_factory=list)
    nccl_group_name: str = "update_weight_group"
    weight_chunked_mem_mb: int = 1024
    use_lora: bool = False
    lora_name: str = ""
    lora_int_id: int = 0
    base_model_name: str = ""
    peft_config: dict = field(default_factory=dict)
    version: Optional[int] = None
    cast_dtype: Optional[str] = None  # e.g. "float8_e4m3fn" for block-scaled rollout weights
    clear_checkpoint_after_load: bool = True

    @classmethod
    def from_disk(cls, experiment_name: str, trial_name: str, file_root: str, name: str = "default",
                  use_lora: bool = False, **kw) -> "WeightUpdateMeta":
        from ..utils.saver import Saver

        path = os.path.join(Saver.get_model_save_root(experiment_name, trial_name, file_root, name), "weight_update")
        return cls(type="disk", path=path, use_lora=use_lora, **kw)

    @classmethod
    def from_fsdp_xccl(cls, alloc_mode=None, nccl_group_name: str = "update_weight_group",
                       weight_chunked_mem_mb: int = 1024, **kw) -> "WeightUpdateMeta":
        return cls(type="xccl", alloc_mode=alloc_mode, nccl_group_name=nccl_group_name,
                   weight_chunked_mem_mb=weight_chunked_mem_mb, **kw)

    @classmethod
    def from_p2p(cls, alloc_mode=None, cast_dtype: Optional[str] = None, **kw) -> "WeightUpdateMeta":
        return cls(type="p2p", alloc_mode=alloc_mode, cast_dtype=cast_dtype, **kw)

    def with_version(self, version: int) -> "WeightUpdateMeta":
        """Copy of the meta bound to ``version``; disk updates go to ``weight_update_v{N}``."""
        import copy

        m = copy.copy(self)
        m.version = version
        if self.type == "disk" and self.path is not None:
            base = self.path
            # strip a previous version suffix
            if "weight_update_v" in os.path.basename(base):
                base = os.path.join(os.path.dirname(base), "weight_update")
            m.path = f"{base}_v{version}"
        return m


@dataclass
class HttpRequest:
    endpoint: str
    payload: dict[str, Any] = field(default_factory=dict)
    method: str = "POST"


@dataclass
class HttpGenerationResult:
    output_tokens: list[int]
    output_logprobs: list[float]
    stop_reason: str
    routed_experts: Any = None

    def __post_init__(self):
        for lp in self.output_logprobs:
            if lp is None or not math.isfinite(lp):
                raise ValueError(f"non-finite logprob in generation result: {lp}")


@dataclass
class WeightUpdateRequests:
    requests: list[HttpRequest] = field(default_factory=list)


@dataclass
class SaveLoadMeta:
    path: str
    weight_format: Literal["hf", "dcp", "sharded"] = "hf"
    with_optim: bool = False
    tokenizer: Any = None
    processor: Any = None
    base_model_path: Optional[str] = None
    naive_distributed: bool = False


@dataclass
class RolloutStat:
    enqueued: int = 0
    accepted: int = 0
    running: int = 0
    rejected: int = 0


@dataclass
class StepInfo:
    epoch: int
    epoch_step: int
    global_step: int
    steps_per_epoch: int

    def next(self) -> "StepInfo":
        last = self.epoch_step == self.steps_per_epoch - 1
        return StepInfo(
            epoch=self.epoch + int(last), epoch_step=0 if last else self.epoch_step + 1,
            global_step=self.global_step + 1, steps_per_epoch=self.steps_per_epoch,
        )


@dataclass
class LocalInfServerInfo:
    host: str
    port: int
    process: Any = None
    gpu_ids: list[int] = field(default_factory=list)


@dataclass
class DeviceRuntimeInfo:
    mem_allocated: float = 0.0
    mem_reserved: float = 0.0
    mem_used: float = 0.0
    mem_total: float = 0.0

    @classmethod
    def get_current(cls) -> "DeviceRuntimeInfo":
        import torch

        if not torch.cuda.is_available():
            return cls()
        free, total = torch.cuda.mem_get_info()
        gb = 1024 ** 3
        return cls(torch.cuda.memory_allocated() / gb, torch.cuda.memory_reserved() / gb, (total - free) / gb,
                   total / gb)

    def log(self, msg: str = "") -> str:
        return (f"{msg} mem allocated {self.mem_allocated:.2f} GB reserved {self.mem_reserved:.2f} GB "
                f"device used {self.mem_used:.2f}/{self.mem_total:.2f} GB")
