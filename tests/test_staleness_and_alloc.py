"""Admission control formula and allocation-mode grammar."""
import pytest

from areal_b200.api.alloc_mode import (AllocationMode, AllocationType, AllocationValidationError,
                                       InvalidAllocationModeError, ModelAllocation, ParallelStrategy)
from areal_b200.rollout.staleness import StalenessManager


class _Version:
    def __init__(self, v=0):
        self.v = v

    def get_version(self):
        return self.v


def test_capacity_formula_concurrency_and_staleness():
    ver = _Version(0)
    m = StalenessManager(ver, max_concurrent_rollouts=10, consumer_batch_size=4, max_staleness=1)
    # (1 + 0 + 1) * 4 = 8 samples may exist before version 1
    assert m.get_capacity() == 8
    for _ in range(8):
        m.on_rollout_enqueued()
        m.on_rollout_submitted()
    assert m.get_capacity() == 0
    for _ in range(4):
        m.on_rollout_accepted()
    assert m.get_capacity() == 0            # accepted still counts against the staleness budget
    ver.v = 1
    assert m.get_capacity() == 4            # (1 + 1 + 1) * 4 - (4 + 4)
    for _ in range(2):
        m.on_rollout_rejected()
    assert m.get_capacity() == 6            # rejected samples give their budget back
    s = m.get_stats()
    assert (s.accepted, s.running, s.rejected) == (4, 2, 2)


def test_capacity_concurrency_bound_and_recovery():
    ver = _Version(5)
    m = StalenessManager(ver, max_concurrent_rollouts=3, consumer_batch_size=2, max_staleness=100)
    assert m.get_capacity() == 3
    m.on_rollout_enqueued(); m.on_rollout_submitted()
    assert m.get_capacity() == 2
    m.on_version_recovered(5)
    assert m.get_stats().accepted == 10 and m.get_stats().running == 0
    assert m.get_pending_limit() == 202


@pytest.mark.parametrize("text,backend,dims", [
    ("sglang:d4p1t1", "sglang", (4, 1, 1)), ("fsdp:d4", "fsdp", (4, 1, 1)), ("d2t2", "fsdp", (2, 1, 2)),
    ("vllm:d2t4", "vllm", (2, 1, 4)), ("native:d2t2", "native", (2, 1, 2)), ("megatron:d2p2t2", "megatron", (2, 2, 2)),
])
def test_alloc_mode_single(text, backend, dims):
    a = ModelAllocation.from_str(text)
    assert a.backend == backend
    p = a.parallel
    assert (p.dp_size, p.pp_size, p.tp_size) == dims
    assert p.world_size == dims[0] * dims[1] * dims[2]


def test_alloc_mode_compound_and_hybrid():
    m = AllocationMode.from_str("sglang:d4t2+fsdp:d8")
    assert m.type_ == AllocationType.DECOUPLED_TRAIN
    assert m.gen.world_size == 8 and m.train.world_size == 8 and m.gen_instance_size == 2
    h = ModelAllocation.from_str("megatron:(attn:d2c4|ffn:d1e8)")
    assert h.parallel.cp_size == 4 and h.parallel.ep_size == 8 and h.parallel.world_size == 8
    named = AllocationMode.from_str("actor:fsdp:d4+critic:fsdp:d2")
    assert named["actor"].world_size == 4 and named["critic"].world_size == 2


@pytest.mark.parametrize("bad", ["", "fsdp:", "fsdp:d0", "fsdp:x4", "nope:d2", "fsdp:d2d2", "megatron:(attn:d2c4|ffn:d1e4)",
                                 "megatron:(attn:d2p2|ffn:d2e2)"])
def test_alloc_mode_rejects(bad):
    with pytest.raises((InvalidAllocationModeError, AllocationValidationError)):
        AllocationMode.from_str(bad)


def test_fsdp_rejects_pipeline_and_expert():
    with pytest.raises(AllocationValidationError):
        ModelAllocation.from_str("fsdp:d2p2")
    with pytest.raises(AllocationValidationError):
        ModelAllocation.from_str("fsdp:d2e2")
    assert ParallelStrategy(data_parallel_size=2, context_parallel_size=2, tensor_parallel_size=2).world_size == 8
