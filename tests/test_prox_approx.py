"""Proximal log-probs without a forward pass: the interpolation between the behaviour policy (per-token version) and
the current policy, the choice the loss makes between recomputed, approximated and reused log-probs, and what the
actor does for each ``prox_logp_method``."""
import math

import pytest
import torch

from areal_b200.algo import advantages as ADV
from areal_b200.api.cli_args import PPOActorConfig
from areal_b200.trainer.ppo.actor import grpo_loss_fn, resolve_proximal_logp


def test_loglinear_interpolates_by_version_distance():
    old, lp = torch.tensor([[-2.0, -2.0, -2.0]]), torch.tensor([[-1.0, -1.0, -1.0]])
    out = ADV.compute_prox_logp_approximation(old, lp, torch.tensor([[0, 2, 4]]), current_version=5, method="loglinear")
    # alpha = (v_prox - v_b) / (v_theta - v_b) with v_prox = 4: 4/5, 2/3, 0/1
    assert torch.allclose(out, torch.tensor([[-2.0 + 0.8, -2.0 + 2 / 3, -2.0]]), atol=1e-6)


def test_sample_from_the_previous_version_is_its_own_proximal_policy():
    old, lp = torch.tensor([-3.0]), torch.tensor([-0.5])
    out = ADV.compute_prox_logp_approximation(old, lp, torch.tensor([6]), current_version=7)
    assert out.item() == -3.0                                    # v_b == v_prox: alpha = 0


def test_alpha_is_clamped_and_future_or_equal_versions_fall_back_to_the_behaviour_policy():
    old, lp = torch.full((4,), -2.0), torch.full((4,), -1.0)
    out = ADV.compute_prox_logp_approximation(old, lp, torch.tensor([5, 6, 9, 0]), current_version=5)
    assert out[:3].tolist() == [-2.0, -2.0, -2.0]                # same version, newer than current (clock skew): alpha 0
    assert -2.0 < out[3].item() < -1.0 and out[3].item() == pytest.approx(-2.0 + 0.8)


def test_version_zero_current_and_prompt_tokens():
    old, lp = torch.tensor([-1.0, -1.0]), torch.tensor([-4.0, -4.0])
    out = ADV.compute_prox_logp_approximation(old, lp, torch.tensor([0, -1]), current_version=0)
    assert torch.isfinite(out).all() and out.tolist() == [-1.0, -1.0]     # no division by zero; prompt tokens (-1) untouched


def test_linear_variant_interpolates_probabilities():
    old, lp = torch.tensor([math.log(0.2)]), torch.tensor([math.log(0.6)])
    out = ADV.compute_prox_logp_approximation(old, lp, torch.tensor([1]), current_version=3, method="linear")
    assert out.item() == pytest.approx(math.log(0.2 + 0.5 * 0.4), abs=1e-6)   # alpha = (2 - 1) / (3 - 1)
    ll = ADV.compute_prox_logp_approximation(old, lp, torch.tensor([1]), current_version=3, method="loglinear")
    assert ll.item() == pytest.approx(0.5 * (math.log(0.2) + math.log(0.6)), abs=1e-6)
    assert out.item() > ll.item()                                 # arithmetic mean of probabilities >= geometric mean


@pytest.mark.parametrize("shape", [(7,), (3, 5)])
def test_shapes_dtypes_and_no_side_effects(shape):
    g = torch.Generator().manual_seed(0)
    old, lp = -torch.rand(shape, generator=g), (-torch.rand(shape, generator=g)).requires_grad_()
    versions = torch.randint(-1, 4, shape, generator=g)
    keep = versions.clone()
    for method in ("loglinear", "linear"):
        out = ADV.compute_prox_logp_approximation(old, lp, versions, 4, method)
        assert out.shape == shape and out.dtype == torch.float32 and not out.requires_grad
        lo, hi = torch.minimum(old, lp.detach()), torch.maximum(old, lp.detach())
        assert ((out >= lo - 1e-6) & (out <= hi + 1e-6)).all()   # an interpolation never leaves the two end points
    assert torch.equal(versions, keep)
    with pytest.raises(ValueError, match="unknown approximation"):
        ADV.compute_prox_logp_approximation(old, lp, versions, 4, "cubic")


def test_resolution_order_of_the_proximal_log_probs():
    old, lp, gt = torch.tensor([-2.0]), torch.tensor([-1.0]), torch.tensor([-1.7])
    v = torch.tensor([0])
    assert resolve_proximal_logp(gt, "recompute", old, lp, v, 2) is gt
    assert resolve_proximal_logp(None, "reuse_train_logp", old, lp, v, 2).item() == -1.0
    assert resolve_proximal_logp(gt, "loglinear", old, lp, v, 2).item() == pytest.approx(-1.5)   # the approximation wins over a given tensor
    with pytest.raises(ValueError, match="needs per-token versions"):
        resolve_proximal_logp(None, "loglinear", old, lp, None, 2)
    with pytest.raises(ValueError, match="needs per-token versions"):
        resolve_proximal_logp(None, "linear", old, lp, v, None)
    with pytest.raises(ValueError, match="prox_logp missing"):
        resolve_proximal_logp(None, "recompute", old, lp, v, 2)


def _mb(n=6, stale=True):
    g = torch.Generator().manual_seed(1)
    old = -torch.rand(n, generator=g) - 0.5
    return dict(logprobs=old, advantages=torch.randn(n, generator=g), loss_mask=torch.tensor([0, 1, 1, 1, 1, 1]),
                versions=torch.tensor([-1, 0, 0, 1, 1, 2]) if stale else torch.full((n,), 2),
                cu_seqlens=torch.tensor([0, n], dtype=torch.int32))


def test_loss_with_approximation_matches_loss_with_that_tensor_given():
    mb = _mb()
    lp = (mb["logprobs"] + 0.2 * torch.randn(6, generator=torch.Generator().manual_seed(2))).requires_grad_()
    ent = torch.zeros(6)
    a = grpo_loss_fn(lp, ent, dict(mb), 0.2, None, None, current_version=3, prox_logp_method="loglinear", use_decoupled_loss=True)
    prox = ADV.compute_prox_logp_approximation(mb["logprobs"], lp.detach(), mb["versions"], 3, "loglinear")
    b = grpo_loss_fn(lp, ent, dict(mb, prox_logp=prox), 0.2, None, None, current_version=3, prox_logp_method="recompute", use_decoupled_loss=True)
    assert torch.allclose(a, b)
    with pytest.raises(ValueError, match="needs per-token versions"):
        mb2 = dict(mb)
        mb2.pop("versions")
        grpo_loss_fn(lp, ent, mb2, 0.2, None, None, current_version=3, prox_logp_method="loglinear", use_decoupled_loss=True)


def test_reuse_train_logp_gives_a_ratio_of_one_and_the_plain_policy_gradient():
    """prox == theta: the clipped ratio is 1 everywhere, so the gradient is the policy gradient, times the behaviour
    importance weight pi_prox / pi_behave when a rejection-sampling rule (which owns that weight) is configured."""
    from areal_b200.api.cli_args import RejectionSamplingConfig

    mb = _mb()
    m = mb["loss_mask"].float()
    for rs in (None, RejectionSamplingConfig(upper=5.0)):
        lp = (mb["logprobs"] - 0.1).clone().requires_grad_()
        loss = grpo_loss_fn(lp, torch.zeros(6), dict(mb), 0.2, None, None, rejection_sampling=rs, current_version=3,
                            prox_logp_method="reuse_train_logp", use_decoupled_loss=True)
        loss.backward()
        w = torch.exp(lp.detach() - mb["logprobs"]) if rs is not None else torch.ones(6)
        assert torch.allclose(lp.grad, -(mb["advantages"] * w * m) / m.sum(), atol=1e-6)


def test_actor_skips_the_forward_pass_exactly_when_the_method_needs_none():
    calls = []

    class Eng:
        def eval(self):
            pass

        def forward_batch(self, data, **kw):
            calls.append(kw)
            return torch.zeros(1, 2)

    from areal_b200.trainer.ppo.actor import PPOActor

    for method, runs in (("recompute", True), ("loglinear", False), ("linear", False), ("reuse_train_logp", False)):
        calls.clear()
        cfg = PPOActorConfig(use_decoupled_loss=True, prox_logp_method=method, recompute_logprob=True, ppo_n_minibatches=1)
        out = PPOActor(cfg, Eng()).compute_logp({"input_ids": torch.zeros(1, 2)})
        assert (out is not None) == runs and bool(calls) == runs
    cfg = PPOActorConfig(use_decoupled_loss=False, recompute_logprob=False)
    assert PPOActor(cfg, Eng()).compute_logp({}) is None
    with pytest.raises(ValueError, match="unknown prox_logp_method"):
        PPOActorConfig(prox_logp_method="guess")
    with pytest.raises(ValueError, match="requires ppo_n_minibatches=1"):
        PPOActorConfig(prox_logp_method="reuse_train_logp", ppo_n_minibatches=4)


def test_metrics_method_trains_on_recomputed_log_probs_and_logs_approximation_errors():
    from areal_b200.utils import stats_tracker

    mb = _mb()
    lp = (mb["logprobs"] + 0.3).clone().requires_grad_()
    gt = mb["logprobs"] + 0.12
    stats_tracker.export_all()                                    # drop what earlier tests left
    a = grpo_loss_fn(lp, torch.zeros(6), dict(mb, prox_logp=gt), 0.2, None, None, current_version=3, prox_logp_method="metrics",
                     use_decoupled_loss=True)
    st = stats_tracker.export_all()
    b = grpo_loss_fn(lp, torch.zeros(6), dict(mb, prox_logp=gt), 0.2, None, None, current_version=3, prox_logp_method="recompute",
                     use_decoupled_loss=True)
    plain = stats_tracker.export_all()
    assert torch.allclose(a, b)
    keys = [k for k in st if "prox_approx/" in k]
    assert any("loglinear/abs_error" in k for k in keys) and any("linear/ratio_error" in k for k in keys)
    assert not [k for k in plain if "prox_approx/" in k]
    ll = ADV.compute_prox_logp_approximation(mb["logprobs"], lp.detach(), mb["versions"], 3, "loglinear")
    m = mb["loss_mask"].bool()
    want = float(((ll - gt).abs() * m).sum() / m.sum())
    got = next(v for k, v in st.items() if k.endswith("prox_approx/loglinear/abs_error/avg"))
    assert got == pytest.approx(want, rel=1e-5)
