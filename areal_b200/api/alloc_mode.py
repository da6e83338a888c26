"""Allocation-mode strings: which backend runs a model and how it is parallelised.

Grammar (same surface as the reference's ``areal/api/alloc_mode.py:594-639``):

    expr        := component ( '+' component )* | legacy
    component   := [ name ':' ] backend ':' strategy        e.g.  sglang:d4t2   actor:fsdp:d8
                 | backend ':' '(' 'attn' ':' dims '|' 'ffn' ':' dims ')'   (hybrid MoE layout)
                 | backend '[' name ']' ':' strategy
    strategy    := dims
    dims        := ( letter int )+      letters d=data p=pipeline t=tensor c=context e=expert
                                        (et<k> = expert-tensor)
    legacy      := dims                  (a bare strategy means an FSDP/SPMD trainer)

``ParallelStrategy.world_size = dp * cp * tp * pp`` (alloc_mode.py:32-200). FSDP rejects
pipeline and expert parallelism (:249-379); the hybrid form requires the attention and FFN
foldings to cover the same number of GPUs and the same pipeline depth (:957-1054).

The parser is a small hand-written recursive-descent parser (the reference uses Lark).
"""
from __future__ import annotations

import enum
import re
from dataclasses import dataclass, field
from typing import Optional


class AllocationValidationError(ValueError):
    pass


class InvalidAllocationModeError(ValueError):
    pass


class AllocationType(enum.Enum):
    COLOCATE = 0
    DECOUPLED_TRAIN = 1
    LLM_SERVER_ONLY = 2
    DECOUPLED_EVAL = 3


TRAIN_BACKENDS = ("fsdp", "megatron", "archon", "b200")
INFER_BACKENDS = ("sglang", "vllm", "native")


@dataclass
class ParallelStrategy:
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    data_parallel_size: int = 1
    context_parallel_size: int = 1
    expert_parallel_size: int = 1
    expert_tensor_parallel_size: int = 1

    def __post_init__(self):
        for k, v in self.__dict__.items():
            if not isinstance(v, int) or v < 1:
                raise AllocationValidationError(f"{k} must be a positive integer, got {v}")
        if self.expert_parallel_size > 1:
            total = self.world_size
            etp = self.expert_tensor_parallel_size
            if total % (self.expert_parallel_size * etp * self.pipeline_parallel_size) != 0:
                raise AllocationValidationError(
                    f"world size {total} not divisible by ep*etp*pp = "
                    f"{self.expert_parallel_size * etp * self.pipeline_parallel_size}")

    # short aliases used throughout the code base
    @property
    def tp_size(self): return self.tensor_parallel_size
    @property
    def pp_size(self): return self.pipeline_parallel_size
    @property
    def dp_size(self): return self.data_parallel_size
    @property
    def cp_size(self): return self.context_parallel_size
    @property
    def ep_size(self): return self.expert_parallel_size
    @property
    def etp_size(self): return self.expert_tensor_parallel_size

    @property
    def edp_size(self) -> int:
        """Data-parallel degree of the expert (FFN) part."""
        return self.world_size // (self.ep_size * self.etp_size * self.pp_size)

    @property
    def world_size(self) -> int:
        return (self.data_parallel_size * self.context_parallel_size * self.tensor_parallel_size
                * self.pipeline_parallel_size)

    def __str__(self) -> str:
        s = f"d{self.dp_size}p{self.pp_size}t{self.tp_size}"
        if self.cp_size > 1:
            s += f"c{self.cp_size}"
        if self.ep_size > 1:
            s += f"e{self.ep_size}"
        if self.etp_size > 1:
            s += f"et{self.etp_size}"
        return s

    @staticmethod
    def parallelism_eq(a: "ParallelStrategy", b: "ParallelStrategy") -> bool:
        return (a.tp_size, a.pp_size, a.dp_size, a.cp_size, a.ep_size, a.etp_size) == (
            b.tp_size, b.pp_size, b.dp_size, b.cp_size, b.ep_size, b.etp_size)


@dataclass
class FSDPParallelStrategy(ParallelStrategy):
    """FSDP-style layout; ``cp`` is Ulysses sequence parallelism."""

    @staticmethod
    def parallelism_eq(a, b):
        return ParallelStrategy.parallelism_eq(a, b)


@dataclass
class MegatronParallelStrategy(ParallelStrategy):
    virtual_pipeline_parallel_size: int = 1
    use_sequence_parallel: bool = False

    def __post_init__(self):
        vpp = self.virtual_pipeline_parallel_size
        usp = self.use_sequence_parallel
        # validate the int fields only
        object.__setattr__(self, "use_sequence_parallel", 1)
        try:
            super().__post_init__()
        finally:
            object.__setattr__(self, "use_sequence_parallel", usp)
        if vpp < 1:
            raise AllocationValidationError("virtual pipeline size must be >= 1")


@dataclass
class ModelAllocation:
    backend: str
    parallel: ParallelStrategy
    name: Optional[str] = None
    ffn_parallel: Optional[ParallelStrategy] = None  # hybrid (attn|ffn) layouts

    @property
    def is_train(self) -> bool:
        return self.backend in TRAIN_BACKENDS

    @property
    def is_inference(self) -> bool:
        return self.backend in INFER_BACKENDS

    @property
    def world_size(self) -> int:
        return self.parallel.world_size

    def __post_init__(self):
        if self.backend not in TRAIN_BACKENDS + INFER_BACKENDS:
            raise InvalidAllocationModeError(f"unknown backend '{self.backend}'")
        p = self.parallel
        if self.backend == "fsdp":
            if p.pp_size > 1:
                raise AllocationValidationError("the fsdp backend does not support pipeline parallelism")
            if p.ep_size > 1:
                raise AllocationValidationError("the fsdp backend does not support expert parallelism")
        if self.is_inference:
            if p.cp_size > 1 or p.ep_size > 1 and self.backend != "native":
                raise AllocationValidationError("inference backends take only d/t/p dimensions")

    @classmethod
    def from_str(cls, text: str, name: Optional[str] = None) -> "ModelAllocation":
        allocs = _Parser(text).parse()
        if len(allocs) != 1:
            raise InvalidAllocationModeError(f"expected a single component in '{text}'")
        a = allocs[0]
        if name is not None and a.name is None:
            a.name = name
        return a

    def __str__(self) -> str:
        head = f"{self.backend}:"
        if self.ffn_parallel is not None:
            return f"{head}(attn:{self.parallel}|ffn:{self.ffn_parallel})"
        return head + str(self.parallel)


_DIM = re.compile(r"(et|[dptce])(\d+)")


def _parse_dims(text: str) -> dict:
    pos = 0
    out: dict = {}
    text = text.strip()
    if not text:
        raise InvalidAllocationModeError("empty parallel strategy")
    while pos < len(text):
        m = _DIM.match(text, pos)
        if not m:
            raise InvalidAllocationModeError(f"cannot parse parallel strategy '{text}' at '{text[pos:]}'")
        key, val = m.group(1), int(m.group(2))
        if key in out:
            raise InvalidAllocationModeError(f"dimension '{key}' given twice in '{text}'")
        if val < 1:
            raise AllocationValidationError(f"dimension '{key}' must be >= 1")
        out[key] = val
        pos = m.end()
    return out


def _strategy_from_dims(d: dict, backend: str) -> ParallelStrategy:
    kw = dict(
        data_parallel_size=d.get("d", 1), pipeline_parallel_size=d.get("p", 1), tensor_parallel_size=d.get("t", 1),
        context_parallel_size=d.get("c", 1), expert_parallel_size=d.get("e", 1),
        expert_tensor_parallel_size=d.get("et", 1),
    )
    if backend == "megatron":
        return MegatronParallelStrategy(**kw)
    if backend in ("fsdp", "b200"):
        return FSDPParallelStrategy(**kw)
    return ParallelStrategy(**kw)


class _Parser:
    def __init__(self, text: str):
        self.text = text.strip()

    def parse(self) -> list[ModelAllocation]:
        if not self.text:
            raise InvalidAllocationModeError("empty allocation mode")
        comps = self._split_top(self.text, "+")
        return [self._component(c.strip()) for c in comps]

    @staticmethod
    def _split_top(s: str, sep: str) -> list[str]:
        parts, depth, cur = [], 0, []
        for ch in s:
            if ch in "([":
                depth += 1
            elif ch in ")]":
                depth -= 1
            if ch == sep and depth == 0:
                parts.append("".join(cur))
                cur = []
            else:
                cur.append(ch)
        parts.append("".join(cur))
        if any(not p.strip() for p in parts):
            raise InvalidAllocationModeError(f"empty component in '{s}'")
        return parts

    def _component(self, comp: str) -> ModelAllocation:
        name = None
        m = re.match(r"^([A-Za-z_][\w-]*)\[([\w-]+)\]\s*:(.*)$", comp)
        if m:  # backend[name]:strategy
            backend, name, rest = m.group(1), m.group(2), m.group(3).strip()
        else:
            head, sep, rest = comp.partition(":")
            if not sep:
                # bare strategy => trainer on this framework's FSDP-style engine
                return ModelAllocation("fsdp", _strategy_from_dims(_parse_dims(comp), "fsdp"))
            head, rest = head.strip(), rest.strip()
            if head in TRAIN_BACKENDS + INFER_BACKENDS:
                backend = head
            else:
                name = head
                backend, sep2, rest = rest.partition(":")
                backend, rest = backend.strip(), rest.strip()
                if not sep2:
                    raise InvalidAllocationModeError(f"missing strategy in '{comp}'")
        if backend not in TRAIN_BACKENDS + INFER_BACKENDS:
            raise InvalidAllocationModeError(f"unknown backend '{backend}' in '{comp}'")
        if rest.startswith("("):
            if not rest.endswith(")"):
                raise InvalidAllocationModeError(f"unbalanced parentheses in '{comp}'")
            inner = rest[1:-1]
            halves = inner.split("|")
            if len(halves) != 2:
                raise InvalidAllocationModeError("hybrid layout must be (attn:...|ffn:...)")
            parts = {}
            for h in halves:
                k, sep, v = h.partition(":")
                if not sep or k.strip() not in ("attn", "ffn"):
                    raise InvalidAllocationModeError("hybrid layout must be (attn:...|ffn:...)")
                parts[k.strip()] = _parse_dims(v)
            if set(parts) != {"attn", "ffn"}:
                raise InvalidAllocationModeError("hybrid layout needs both attn and ffn parts")
            attn, ffn = parts["attn"], parts["ffn"]
            if "e" in attn or "et" in attn:
                raise AllocationValidationError("the attention part cannot carry expert dimensions")
            if "c" in ffn:
                raise AllocationValidationError("the ffn part cannot carry a context dimension")
            a_world = attn.get("d", 1) * attn.get("c", 1) * attn.get("t", 1) * attn.get("p", 1)
            f_world = ffn.get("d", 1) * ffn.get("e", 1) * ffn.get("t", ffn.get("et", 1)) * ffn.get("p", 1)
            if a_world != f_world:
                raise AllocationValidationError(
                    f"attention ({a_world} GPUs) and ffn ({f_world} GPUs) foldings must cover the same world")
            if attn.get("p", 1) != ffn.get("p", 1):
                raise AllocationValidationError("attention and ffn parts must share the pipeline depth")
            merged = dict(attn)
            merged["e"] = ffn.get("e", 1)
            merged["et"] = ffn.get("et", ffn.get("t", 1))
            par = _strategy_from_dims(merged, backend)
            ffn_dims = dict(ffn)
            ffn_par = ParallelStrategy(
                data_parallel_size=ffn_dims.get("d", 1) * ffn_dims.get("e", 1),
                tensor_parallel_size=ffn_dims.get("t", ffn_dims.get("et", 1)),
                pipeline_parallel_size=ffn_dims.get("p", 1),
            )
            object.__setattr__(ffn_par, "expert_parallel_size", ffn_dims.get("e", 1))
            return ModelAllocation(backend, par, name, ffn_par)
        return ModelAllocation(backend, _strategy_from_dims(_parse_dims(rest), backend), name)


@dataclass
class AllocationMode:
    """A full experiment allocation: any number of named components."""

    allocations: list[ModelAllocation] = field(default_factory=list)

    @classmethod
    def from_str(cls, text: str) -> "AllocationMode":
        return cls(_Parser(text).parse())

    @property
    def gen(self) -> Optional[ModelAllocation]:
        return next((a for a in self.allocations if a.is_inference), None)

    @property
    def train(self) -> Optional[ModelAllocation]:
        return next((a for a in self.allocations if a.is_train), None)

    @property
    def gen_backend(self) -> Optional[str]:
        return self.gen.backend if self.gen else None

    @property
    def train_backend(self) -> Optional[str]:
        return self.train.backend if self.train else None

    @property
    def gen_instance_size(self) -> int:
        g = self.gen
        return g.parallel.tp_size * g.parallel.pp_size if g else 0

    @property
    def type_(self) -> AllocationType:
        if self.gen and self.train:
            return AllocationType.DECOUPLED_TRAIN
        if self.gen:
            return AllocationType.LLM_SERVER_ONLY
        return AllocationType.COLOCATE

    @property
    def world_size(self) -> int:
        return sum(a.world_size for a in self.allocations)

    def __getitem__(self, name: str) -> ModelAllocation:
        for a in self.allocations:
            if a.name == name:
                return a
        raise KeyError(name)
