"""Batch containers, packing, micro-batching, sequence bin-packing, stats tracker."""
import pytest
import torch

from areal_b200.api.cli_args import MicroBatchSpec
from areal_b200.utils import data as D
from areal_b200.utils import seqpack, stats_tracker


def _seqs(lens):
    return [dict(input_ids=torch.arange(n), loss_mask=torch.ones(n, dtype=torch.int32), rewards=torch.tensor(float(n)))
            for n in lens]


def test_pad_pack_roundtrip():
    lens = [5, 3, 9, 1]
    b = D.pad_sequences_to_tensors(_seqs(lens))
    assert b["input_ids"].shape == (4, 9) and b["rewards"].shape == (4,)
    assert b["attention_mask"].sum(1).tolist() == lens
    p = D.pack_tensor_dict(b)
    assert p["cu_seqlens"].tolist() == [0, 5, 8, 17, 18] and p["max_seqlen"] == 9
    assert p["input_ids"].tolist() == [x for n in lens for x in range(n)]
    back = D.unpack_to_padded(p["input_ids"], lens)
    assert torch.equal(back, b["input_ids"])
    assert D.positions_from_cu_seqlens(p["cu_seqlens"]).tolist() == [x for n in lens for x in range(n)]


def test_concat_padded_and_select():
    a = D.pad_sequences_to_tensors(_seqs([4, 2]))
    b = D.pad_sequences_to_tensors(_seqs([7]))
    c = D.concat_padded_tensors([a, b])
    assert c["input_ids"].shape == (3, 7) and c["attention_mask"].sum(1).tolist() == [4, 2, 7]
    s = D.select_batch(c, [1, 0])
    assert s["input_ids"].shape == (2, 4) and s["rewards"].tolist() == [2.0, 4.0]


def test_micro_batch_split_respects_budget_and_order():
    lens = [50, 10, 40, 30, 20, 60]
    b = D.pad_sequences_to_tensors(_seqs(lens))
    mbl = D.split_padded_tensor_dict_into_mb_list(b, MicroBatchSpec(max_tokens_per_mb=70))
    assert sorted(i for g in mbl.groups for i in g) == list(range(6))
    assert all(t <= 70 for t in mbl.group_lens)
    assert [mbl.forward_indices[mbl.backward_indices[i]] for i in range(6)] == list(range(6))
    D.pad_mb_list(mbl, align=64)
    for mb, pad, old in zip(mbl.padded_mbs, mbl.padding_lengths, mbl.old_cu_seqlens_list):
        T = int(mb["cu_seqlens"][-1])
        assert T % 64 == 0 and T - pad == int(old[-1]) and mb["input_ids"].shape[0] == T
        assert mb["loss_mask"][T - pad:].sum() == 0
    mbl2 = D.split_padded_tensor_dict_into_mb_list(b, MicroBatchSpec(n_mbs=4, max_tokens_per_mb=1000))
    assert len(mbl2) >= 4


@pytest.mark.parametrize("fn", ["ffd", "kk"])
def test_allocators(fn):
    sizes = [9, 8, 7, 6, 5, 4, 3, 2, 1, 10]
    groups = seqpack.get_allocate_fn(fn)(sizes, 15, 1)
    assert sorted(i for g in groups for i in g) == list(range(10))
    assert all(sum(sizes[i] for i in g) <= 15 for g in groups)


def test_kk_balance_and_greedy_counts():
    sizes = [100, 90, 80, 70, 60, 50, 40, 30]
    g = seqpack.kk_allocate(sizes, 2)
    sums = sorted(sum(sizes[i] for i in x) for x in g)
    assert sums[1] - sums[0] <= 20
    eq = seqpack.kk_allocate(sizes, 4, equal_size=True)
    assert all(len(x) == 2 for x in eq)
    bg = seqpack.balanced_greedy_partition(sizes, 3)
    assert sorted(len(x) for x in bg) == [2, 3, 3]
    with pytest.raises(ValueError):
        seqpack.kk_allocate([1, 2, 3], 2, equal_size=True)


def test_ffd_min_groups():
    groups = seqpack.ffd_allocate([1, 1, 1, 1], 100, min_groups=3)
    assert len(groups) == 3


def test_stats_tracker_scopes_and_reduce_types():
    t = stats_tracker.DistributedStatsTracker()
    mask = torch.tensor([True, False, True, True])
    with t.scope("a"):
        t.denominator(n=mask)
        t.stat(x=torch.tensor([1.0, 100.0, 3.0, 5.0]), denominator="n")
        t.stat(y=torch.tensor([1.0, 1.0, 1.0, 1.0]), denominator="n", reduce_type=stats_tracker.ReduceType.SUM)
        t.scalar(lr=0.5)
        t.scalar(lr=1.5)
        with t.record_timing("step"):
            pass
    out = t.export()
    assert out["a/n"] == 3 and out["a/x/avg"] == pytest.approx(3.0) and out["a/x/min"] == 1 and out["a/x/max"] == 5
    assert out["a/y"] == 3 and out["a/lr"] == 1.0 and "timeperf/step" in out
    assert t.export() == {}
    with pytest.raises(ValueError):
        t.denominator(bad=torch.tensor([1.0]))
    with pytest.raises(ValueError):
        t.stat(x=torch.tensor([1.0]), denominator="missing")
