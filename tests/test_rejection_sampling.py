"""Rejection sampling between the proximal and the behaviour policy: configuration rules, token- and sequence-level
filtering with every metric and aggregation, truncation, packed and padded layouts, degenerate inputs."""
import math

import pytest
import torch

from areal_b200.algo.functional import apply_rejection_sampling
from areal_b200.api.cli_args import RejectionSamplingConfig as RS


def _run(prox, old, mask=None, cu=None, **kw):
    prox, old = torch.as_tensor(prox, dtype=torch.float32), torch.as_tensor(old, dtype=torch.float32)
    mask = torch.ones_like(prox) if mask is None else torch.as_tensor(mask, dtype=torch.float32)
    return apply_rejection_sampling(prox, old, mask, None if cu is None else torch.tensor(cu, dtype=torch.int32), RS(**kw))


# ---------------------------------------------------------------- configuration
@pytest.mark.parametrize("kw,msg", [
    (dict(metric="ratio", upper=1.0), "upper must be > 1.0"),
    (dict(metric="ratio", lower=-0.1, upper=5.0), "lower must be positive"),
    (dict(metric="kl_k2", upper=0.0), "upper must be positive"),
    (dict(metric="kl_k3", upper=-1.0), "upper must be positive"),
    (dict(action="clamp", metric="kl_k2", upper=1.0), "only supports metric='ratio'"),
    (dict(metric="ratio", lower=3.0, upper=2.0), "lower must not exceed upper"),
    (dict(level="group"), "level"), (dict(action="drop"), "action"), (dict(metric="tv"), "metric"), (dict(agg="median"), "agg"),
    (dict(upper=None, lower=None), "at least one bound"),
])
def test_config_rules(kw, msg):
    with pytest.raises(ValueError, match=msg):
        RS(**kw)


def test_config_defaults_and_warnings():
    assert RS(action="clamp", metric="ratio", upper=5.0).lower == 0.0
    assert RS(metric="kl_k1", lower=-0.5, upper=0.5).lower == -0.5          # k1 is signed: a negative bound is fine
    with pytest.warns(UserWarning, match="is ignored at token level"):
        RS(level="token", agg="max", metric="ratio", upper=5.0)


# ---------------------------------------------------------------- token level, mask
def test_token_ratio_bounds_filter_both_sides_and_keep_the_boundary():
    up = math.log(2.0)
    r = _run([[0.0, 1.0, up, -2.0]], [[0.0] * 4], metric="ratio", upper=2.0, lower=0.5)
    assert r.loss_mask.tolist() == [[1, 0, 1, 0]]                            # exp(1) > 2 and exp(-2) < 0.5 leave; ratio == upper stays
    assert r.filtered_fraction == 0.5
    assert torch.allclose(r.behave_imp_weight, torch.tensor([[1.0, 0.0, 2.0, 0.0]]))


def test_padding_and_prompt_tokens_are_not_counted():
    r = _run([[0.0, 3.0, 3.0, 0.0]], [[0.0] * 4], mask=[[1, 1, 0, 0]], metric="ratio", upper=2.0)
    assert r.loss_mask.tolist() == [[1, 0, 0, 0]] and r.filtered_fraction == 0.5   # one of the TWO valid tokens


@pytest.mark.parametrize("metric,lr,upper,kept", [
    ("kl_k1", [0.0, -3.0, 0.4, 0.6], 0.5, [1, 1, 1, 0]),                     # k1 = log ratio, signed: -3 passes an upper bound
    ("kl_k2", [0.0, -1.2, 0.9, 1.1], 0.5, [1, 0, 1, 0]),                     # k2 = lr^2 / 2
    ("kl_k3", [0.0, 0.5, -0.5, 2.0], 0.2, [1, 1, 1, 0]),                     # k3 = exp(-lr) - 1 + lr >= 0
])
def test_token_kl_metrics(metric, lr, upper, kept):
    r = _run([lr], [[0.0] * 4], metric=metric, upper=upper)
    assert r.loss_mask.tolist() == [kept]
    if metric == "kl_k3":
        k3 = torch.exp(-torch.tensor(lr)) - 1 + torch.tensor(lr)
        assert (k3 >= 0).all()


def test_binary_kl_is_symmetric_and_filters_large_probability_moves():
    # p goes 0.9 -> 0.1 in one token and stays elsewhere
    prox = torch.log(torch.tensor([[0.5, 0.9, 0.5]]))
    old = torch.log(torch.tensor([[0.5, 0.1, 0.5]]))
    a = apply_rejection_sampling(prox, old, torch.ones(1, 3), None, RS(metric="binary_kl", upper=0.5))
    b = apply_rejection_sampling(old, prox, torch.ones(1, 3), None, RS(metric="binary_kl", upper=0.5))
    assert a.loss_mask.tolist() == b.loss_mask.tolist() == [[1, 0, 1]]


# ---------------------------------------------------------------- sequence level
def test_sequence_ratio_is_the_geometric_mean_and_gives_one_weight_per_sequence():
    lr = torch.tensor([[0.6, 0.0, 0.0, 0.0], [1.0, 1.0, 1.0, 1.0]])
    r = apply_rejection_sampling(lr, torch.zeros_like(lr), torch.ones_like(lr), None, RS(level="sequence", metric="ratio", upper=2.0))
    assert r.loss_mask.tolist() == [[1] * 4, [0] * 4]                        # exp(0.15) stays, exp(1) leaves as a whole
    assert torch.allclose(r.behave_imp_weight[0], torch.full((4,), math.exp(0.15)))
    assert r.filtered_fraction == 0.5


def test_sequence_level_packed_equals_padded():
    lr_a, lr_b = [0.2, -0.1, 0.3], [1.5, 1.5]
    padded = _run([lr_a, lr_b + [0.0]], [[0.0] * 3] * 2, mask=[[1, 1, 1], [1, 1, 0]], level="sequence", metric="ratio", upper=2.0)
    packed = _run(lr_a + lr_b, [0.0] * 5, cu=[0, 3, 5], level="sequence", metric="ratio", upper=2.0)
    assert packed.loss_mask.tolist() == [1, 1, 1, 0, 0]
    assert padded.loss_mask.tolist() == [[1, 1, 1], [0, 0, 0]]
    assert torch.allclose(packed.behave_imp_weight[:3], padded.behave_imp_weight[0])
    assert packed.filtered_fraction == padded.filtered_fraction == 0.4


def test_sequence_kl_keeps_per_token_weights():
    lr = torch.tensor([[0.3, -0.3, 0.1]])
    r = apply_rejection_sampling(lr, torch.zeros_like(lr), torch.ones_like(lr), None, RS(level="sequence", metric="kl_k2", upper=1.0))
    assert r.loss_mask.tolist() == [[1, 1, 1]] and torch.allclose(r.behave_imp_weight, torch.exp(lr))


@pytest.mark.parametrize("agg,kept", [("mean", [1, 1, 1]), ("sum", [0, 0, 1]), ("max", [0, 1, 1])])
def test_sequence_aggregations(agg, kept):
    """k2 per token: sequence a has one token at 0.72 among zeros, b eight tokens at 0.18, c two tokens at 0.18. Under the
    bound 0.5 the mean keeps all three; the sum is length-sensitive (b: 1.44 leaves, c: 0.36 stays, same per-token value);
    the max sees a's single outlier."""
    a = [1.2] + [0.0] * 7
    b = [0.6] * 8
    c = [0.6] * 2 + [9.0] * 6                       # the tail is padding
    mask = [[1] * 8, [1] * 8, [1, 1] + [0] * 6]
    r = _run([a, b, c], [[0.0] * 8] * 3, mask=mask, level="sequence", metric="kl_k2", agg=agg, upper=0.5)
    assert [int(r.loss_mask[i].sum() > 0) for i in range(3)] == kept
    packed = _run(a + b + c[:2], [0.0] * 18, cu=[0, 8, 16, 18], level="sequence", metric="kl_k2", agg=agg, upper=0.5)
    assert [int(packed.loss_mask[x:y].sum() > 0) for x, y in ((0, 8), (8, 16), (16, 18))] == kept


def test_sequence_with_no_valid_token_is_harmless_under_max():
    r = _run([[5.0, 5.0], [0.1, 0.1]], [[0.0] * 2] * 2, mask=[[0, 0], [1, 1]], level="sequence", metric="kl_k2", agg="max", upper=0.5)
    assert r.loss_mask.tolist() == [[0, 0], [1, 1]] and r.filtered_fraction == 0.0


# ---------------------------------------------------------------- clamp
def test_clamp_truncates_weights_and_leaves_the_mask_alone():
    r = _run([[0.0, 2.0, -3.0]], [[0.0] * 3], action="clamp", metric="ratio", upper=3.0, lower=0.2)
    assert r.loss_mask.tolist() == [[1, 1, 1]]
    assert torch.allclose(r.behave_imp_weight, torch.tensor([[1.0, 3.0, 0.2]]))
    assert abs(r.filtered_fraction - 2 / 3) < 1e-9                           # reported as the clamped fraction


def test_clamp_at_sequence_level_truncates_the_shared_weight():
    lr = torch.tensor([[2.0, 2.0], [0.1, 0.1]])
    r = apply_rejection_sampling(lr, torch.zeros_like(lr), torch.ones_like(lr), None,
                                 RS(level="sequence", action="clamp", metric="ratio", upper=2.0))
    assert torch.allclose(r.behave_imp_weight, torch.tensor([[2.0, 2.0], [math.exp(0.1)] * 2]))
    assert r.loss_mask.tolist() == [[1, 1], [1, 1]] and r.filtered_fraction == 0.5


# ---------------------------------------------------------------- degenerate inputs
def test_empty_mask_single_token_and_everything_filtered():
    r = _run([[1.0, 2.0]], [[0.0, 0.0]], mask=[[0, 0]], metric="ratio", upper=2.0)
    assert r.filtered_fraction == 0.0 and r.loss_mask.sum() == 0 and r.behave_imp_weight.sum() == 0
    r = _run([[0.3]], [[0.0]], level="sequence", metric="ratio", upper=2.0)
    assert r.loss_mask.tolist() == [[1]]
    r = _run([[3.0, 3.0]], [[0.0, 0.0]], metric="ratio", upper=2.0)
    assert r.loss_mask.sum() == 0 and r.filtered_fraction == 1.0


def test_infinite_log_probs_do_not_poison_the_weights():
    ninf = float("-inf")
    r = _run([[ninf, 0.0, ninf]], [[ninf, 0.0, 0.0]], metric="ratio", upper=2.0)
    assert torch.isfinite(r.behave_imp_weight).all() and r.loss_mask[0, 1] == 1


def test_shape_and_rank_checks():
    with pytest.raises(ValueError, match="share a shape"):
        apply_rejection_sampling(torch.zeros(2, 3), torch.zeros(2, 4), torch.ones(2, 3), None, RS(upper=2.0))
    with pytest.raises(ValueError, match="1-D or padded 2-D"):
        apply_rejection_sampling(torch.zeros(1, 2, 3), torch.zeros(1, 2, 3), torch.ones(1, 2, 3), None, RS(upper=2.0))


def test_result_never_requires_grad_and_keeps_the_mask_dtype():
    prox = torch.zeros(1, 3, requires_grad=True)
    r = apply_rejection_sampling(prox, torch.zeros(1, 3), torch.ones(1, 3, dtype=torch.int32), None, RS(upper=2.0))
    assert not r.behave_imp_weight.requires_grad and r.loss_mask.dtype == torch.int32
