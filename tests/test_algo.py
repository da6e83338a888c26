"""Loss functions, rejection sampling, GAE, normalisation: checked against direct formulas."""
import math

import pytest
import torch

from areal_b200.algo import advantages as ADV
from areal_b200.algo import functional as AF
from areal_b200.api.cli_args import NormConfig, PPOActorConfig, RejectionSamplingConfig
from areal_b200.utils.data import KLEstimator, Normalization


def _rand(T=40, seed=0):
    g = torch.Generator().manual_seed(seed)
    logp = torch.randn(T, generator=g) * 0.3 - 1
    prox = logp + torch.randn(T, generator=g) * 0.2
    old = prox + torch.randn(T, generator=g) * 0.3
    adv = torch.randn(T, generator=g)
    mask = torch.rand(T, generator=g) > 0.3
    return logp, prox, old, adv, mask


def test_ppo_loss_matches_formula_and_denominator_is_prefilter():
    logp, prox, old, adv, mask = _rand()
    logp = logp.clone().requires_grad_()
    rs = RejectionSamplingConfig(level="token", action="mask", metric="ratio", upper=1.2, lower=0.8)
    loss, stat = AF.ppo_actor_loss_fn(logp, prox, old, adv, 0.2, mask, eps_clip_higher=0.3, c_clip=3.0, rejection_sampling=rs)
    ratio = torch.exp(logp - prox)
    l = torch.max(-adv * ratio, -adv * ratio.clamp(0.8, 1.3))
    l = torch.min(l, torch.sign(adv) * 3.0 * adv)
    w = torch.exp(prox - old)
    keep = mask & (w <= 1.2) & (w >= 0.8)
    expect = (l * w * keep).sum() / mask.sum()
    assert torch.allclose(loss, expect, atol=1e-6)
    assert stat["filtered_fraction"] == pytest.approx(float((mask & ~keep).sum()) / float(mask.sum()))
    loss.backward()
    assert logp.grad[~keep].abs().sum() == 0


def test_rejection_clamp_and_sequence_level_geometric_mean():
    logp, prox, old, adv, mask = _rand(30, 1)
    cu = torch.tensor([0, 10, 30], dtype=torch.int32)
    rs = RejectionSamplingConfig(level="sequence", action="mask", metric="ratio", agg="mean", upper=1.05)
    res = AF.apply_rejection_sampling(prox, old, mask, cu, rs)
    for a, b in [(0, 10), (10, 30)]:
        m = mask[a:b]
        geo = torch.exp(((prox - old)[a:b] * m).sum() / m.sum().clamp(min=1))
        inb = geo <= 1.05
        assert bool((res.loss_mask[a:b].bool() == (m & inb)).all())
        kept = res.loss_mask[a:b].bool()
        assert torch.allclose(res.behave_imp_weight[a:b][kept], geo.expand(int(kept.sum())), atol=1e-6)
    rc = RejectionSamplingConfig(level="token", action="clamp", metric="ratio", upper=1.1, lower=0.9)
    res2 = AF.apply_rejection_sampling(prox, old, mask, None, rc)
    assert bool((res2.loss_mask == mask).all())
    assert res2.behave_imp_weight[mask].max() <= 1.1 + 1e-6 and res2.behave_imp_weight[mask].min() >= 0.9 - 1e-6


@pytest.mark.parametrize("metric", ["kl_k1", "kl_k2", "kl_k3", "binary_kl"])
def test_rejection_metrics_padded_equals_packed(metric):
    g = torch.Generator().manual_seed(2)
    B, L = 3, 7
    prox = torch.randn(B, L, generator=g) * 0.3 - 1
    old = prox + torch.randn(B, L, generator=g) * 0.4
    mask = torch.rand(B, L, generator=g) > 0.2
    cfg = RejectionSamplingConfig(level="sequence", action="mask", metric=metric, agg="max", upper=0.2)
    r2 = AF.apply_rejection_sampling(prox, old, mask, None, cfg)
    cu = torch.arange(0, B * L + 1, L, dtype=torch.int32)
    r1 = AF.apply_rejection_sampling(prox.reshape(-1), old.reshape(-1), mask.reshape(-1), cu, cfg)
    assert bool((r2.loss_mask.reshape(-1) == r1.loss_mask).all())
    assert torch.allclose(r2.behave_imp_weight.reshape(-1), r1.behave_imp_weight)


def test_gspo_sequence_ratio():
    logp, prox, old, adv, mask = _rand(20, 3)
    cu = torch.tensor([0, 8, 20], dtype=torch.int32)
    loss, stat = AF.ppo_actor_loss_fn(logp, prox, old, adv, 0.2, mask, importance_sampling_level="sequence", cu_seqlens=cu)
    r = stat["importance_weight"]
    for a, b in [(0, 8), (8, 20)]:
        m = mask[a:b]
        geo = torch.exp(((logp - prox)[a:b] * m).sum() / m.sum())
        assert torch.allclose(r[a:b][m], geo.expand(int(m.sum())), atol=1e-6)


def test_sapo_cispo_critic_dpo():
    logp, prox, old, adv, mask = _rand(25, 4)
    l, st = AF.sapo_loss_fn(logp, old, adv, 1.0, 1.05, mask)
    ratio = torch.exp(logp - old)
    gate = torch.where(adv > 0, torch.sigmoid(ratio - 1) * 4, torch.sigmoid(1.05 * (ratio - 1)) * 4 / 1.05)
    assert torch.allclose(l, (-(gate * adv) * mask).sum() / mask.sum(), atol=1e-6)
    lp = logp.clone().requires_grad_()
    l2, _ = AF.cispo_loss_fn(lp, prox, old, adv, 0.2, mask)
    l2.backward()
    w = torch.exp(logp - prox).clamp(0.8, 1.2)
    assert torch.allclose(lp.grad, (-(w * adv) * mask) / mask.sum(), atol=1e-6)
    v, vo, ret = torch.randn(25), torch.randn(25), torch.randn(25)
    lc, _ = AF.ppo_critic_loss_fn(v, vo, ret, 0.5, mask)
    exp = torch.max(0.5 * (v - ret) ** 2, 0.5 * (vo + (v - vo).clamp(-0.5, 0.5) - ret) ** 2)
    assert torch.allclose(lc, (exp * mask).sum() / mask.sum(), atol=1e-6)
    pc, pr, rc_, rr = torch.tensor([-5.0, -3.0]).double(), torch.tensor([-6.0, -2.0]).double(), torch.tensor([-5.5, -3.0]).double(), torch.tensor([-5.5, -3.0]).double()
    ld, sd = AF.dpo_preference_loss(pc, pr, rc_, rr, 0.1)
    delta = (pc - rc_) - (pr - rr)
    assert torch.allclose(ld.double(), (-torch.nn.functional.logsigmoid(0.1 * delta)).mean(), atol=1e-6)


def _gae_loop(rewards, values, loss_mask, no_eos, gamma, lam):
    B, L = rewards.shape
    adv = torch.zeros(B, L)
    last = torch.zeros(B)
    nextv = values[:, L - 1] * no_eos
    for t in reversed(range(L - 1)):
        delta = rewards[:, t] + gamma * nextv - values[:, t]
        new = delta + gamma * lam * last
        m = loss_mask[:, t]
        nextv = nextv * (1 - m) + values[:, t] * m
        last = last * (1 - m) + new * m
        adv[:, t] = last
    return adv


@pytest.mark.parametrize("gamma,lam,critic", [(1.0, 1.0, False), (0.99, 0.95, True), (1.0, 0.9, False)])
def test_token_gae_matches_loop(gamma, lam, critic):
    g = torch.Generator().manual_seed(5)
    B, L = 4, 12
    r = torch.randn(B, L, generator=g)
    v = torch.randn(B, L, generator=g) if critic else torch.zeros(B, L)
    m = (torch.rand(B, L, generator=g) > 0.3).float()
    ne = torch.tensor([1.0, 0.0, 1.0, 0.0])
    adv, ret = ADV.token_level_gae(r, v, m, ne, gamma, lam)
    assert torch.allclose(adv, _gae_loop(r, v, m, ne, gamma, lam), atol=1e-5)
    assert torch.allclose(ret, adv + v)


def test_turn_level_gae_single_turn_equals_outcome():
    B, L = 2, 8
    rewards = torch.zeros(B, L); rewards[:, 5] = torch.tensor([1.0, -2.0])
    mask = torch.zeros(B, L); mask[:, 3:6] = 1
    turn_ids = torch.full((B, L), -1); turn_ids[:, 3:6] = 0
    adv, ret = ADV.turn_level_gae(rewards, torch.zeros(B, L), mask, turn_ids, torch.zeros(B), 1.0, 1.0)
    assert torch.allclose(adv[:, 3:6], torch.tensor([[1.0] * 3, [-2.0] * 3]))
    assert adv[:, :3].abs().sum() == 0


def test_lambda_schedules_and_kl_and_norm():
    lens = torch.tensor([0, 1, 5, 50])
    assert torch.allclose(ADV.vapo_length_adaptive_gae(lens, 0.5), torch.tensor([0.0, 0.0, 0.6, 0.96]))
    q = ADV.relative_position_gae_lambda(lens, 0.5)
    assert q[0] == 0 and q[1] == 1 and abs(float(q[2]) - 0.5 ** 0.25) < 1e-6
    lp, lb = torch.tensor([-1.0, -2.0]), torch.tensor([-1.5, -1.0])
    d = lp - lb
    assert torch.allclose(KLEstimator("k1")(lp, lb), d)
    assert torch.allclose(KLEstimator("k2")(lp, lb), 0.5 * d * d)
    assert torch.allclose(KLEstimator("k3")(lp, lb), torch.exp(-d) - 1 + d)
    x = torch.tensor([1.0, 2.0, 3.0, 10.0, 20.0, 30.0])
    n = Normalization(NormConfig(mean_level="group", std_level="group", group_size=3))(x)
    assert torch.allclose(n[:3], torch.tensor([-1.0, 0.0, 1.0]), atol=1e-4) and torch.allclose(n[3:], torch.tensor([-1.0, 0.0, 1.0]), atol=1e-4)
    rl = Normalization(NormConfig(mean_level="group", mean_leave1out=True, std_level="none", group_size=3))(x)
    assert torch.allclose(rl[:3], torch.tensor([1 - 2.5, 2 - 2.0, 3 - 1.5]))
    b = Normalization(NormConfig(mean_level="batch", std_level="batch"))(x)
    assert abs(float(b.mean())) < 1e-5 and abs(float(b.std()) - 1) < 1e-3


def test_prox_approx_and_m2po():
    old = torch.tensor([-1.0, -1.0, -1.0, -1.0])
    lp = torch.tensor([-2.0, -2.0, -2.0, -2.0])
    versions = torch.tensor([-1, 3, 1, 0])
    out = ADV.compute_prox_logp_approximation(old, lp, versions, current_version=3, method="loglinear")
    # alpha: prompt 0; v_b == v_theta -> 0; (2-1)/(3-1) = .5; (2-0)/3
    assert torch.allclose(out, torch.tensor([-1.0, -1.0, -1.5, -1.0 - 2 / 3]), atol=1e-6)
    lin = ADV.compute_prox_logp_approximation(old, lp, versions, 3, "linear")
    assert lin[2] == pytest.approx(math.log(0.5 * (math.exp(-1) + math.exp(-2))), abs=1e-6)
    o = torch.tensor([0.0, 0.0, 0.0, 0.0, 0.0]); p = torch.tensor([3.0, 0.1, 0.2, 2.0, 0.0])
    mask = torch.tensor([1, 1, 1, 1, 0])
    m = ADV.m2po_mask(o, p, mask, m2_threshold=0.05)
    assert m.tolist() == [0, 1, 1, 0, 0]


def test_advantage_pipeline_grpo_shape_and_values():
    cfg = PPOActorConfig(kl_ctl=0.0, reward_scaling=2.0, reward_bias=-0.5, reward_norm=None, adv_norm=None,
                         use_decoupled_loss=True, recompute_logprob=True)
    B, L = 2, 6
    data = dict(input_ids=torch.zeros(B, L, dtype=torch.long), attention_mask=torch.tensor([[1] * 6, [1] * 4 + [0] * 2]).bool(),
                loss_mask=torch.tensor([[0, 0, 1, 1, 1, 1], [0, 0, 1, 1, 0, 0]]), logprobs=torch.full((B, L), -1.0),
                rewards=torch.tensor([1.0, 0.0]), prox_logp=torch.full((B, L), -1.0))
    out = ADV.AdvantageComputer(cfg)(data)
    # rolled mask: generated tokens are predicted from positions 1..4 (seq 0) and 1..2 (seq 1)
    assert out["loss_mask"].tolist() == [[0, 1, 1, 1, 1, 0], [0, 1, 1, 0, 0, 0]]
    assert torch.allclose(out["advantages"][0, 1:5], torch.full((4,), 1.0))      # (1 - .5) * 2
    assert torch.allclose(out["advantages"][1, 1:3], torch.full((2,), -1.0))     # (0 - .5) * 2


# --------------------------------------------------------------------------- optimizer variants
def _opt_setup(kind, wd=0.1, **kw):
    import torch.nn as nn

    from areal_b200.api.cli_args import OptimizerConfig
    from areal_b200.engine.flat_params import FlatParamStore
    from areal_b200.engine.optimizer import ShardedAdamW

    torch.manual_seed(0)
    m = nn.Linear(64, 32, bias=True)
    ref = nn.Linear(64, 32, bias=True)
    ref.load_state_dict(m.state_dict())
    store = FlatParamStore(m, 1, 0)
    opt = ShardedAdamW(store, OptimizerConfig(type=kind, lr=1e-2, weight_decay=wd, gradient_clipping=0.0, warmup_steps=0, **kw))
    return m, ref, store, opt


def test_sgd_applies_weight_decay_like_torch():
    m, ref, store, opt = _opt_setup("sgd")
    topt = torch.optim.SGD(ref.parameters(), lr=1e-2, weight_decay=0.1)
    for step in range(3):
        g = torch.randn(store.padded)
        store.flat_grad.copy_(g)
        for p, off in zip(ref.parameters(), store.offsets):
            p.grad = g[off:off + p.numel()].view(p.shape).clone()
        opt.step(store.grad_shard)
        topt.step()
    for p, q in zip(m.parameters(), ref.parameters()):
        assert torch.allclose(p, q, atol=1e-6)
    # a non-finite gradient norm skips the step entirely, decay included
    before = store.flat_param.clone()
    store.flat_grad.fill_(float("nan"))
    res = opt.step(store.grad_shard)
    assert float(res["state"][2]) == 0.0 and torch.equal(store.flat_param, before)


def test_adam_with_bf16_state_tracks_fp32_adamw():
    """bf16 moments + Kahan-compensated bf16 weights stay close to fp32 AdamW over many small steps,
    where plain bf16 weights would stall (updates below half a bf16 ulp are rounded away)."""
    import torch.nn as nn

    from areal_b200.api.cli_args import OptimizerConfig
    from areal_b200.engine.flat_params import FlatParamStore
    from areal_b200.engine.optimizer import ShardedAdamW

    torch.manual_seed(1)
    m = nn.Linear(48, 16, bias=False).to(torch.bfloat16)
    w0 = m.weight.detach().float().clone()
    store = FlatParamStore(m, 1, 0)
    opt = ShardedAdamW(store, OptimizerConfig(type="adam_bf16", lr=1e-5, weight_decay=0.0, gradient_clipping=0.0, warmup_steps=0))
    assert opt.exp_avg.dtype == torch.bfloat16 and opt.master.dtype == torch.bfloat16
    ref = nn.Parameter(w0.clone())
    topt = torch.optim.AdamW([ref], lr=1e-5, weight_decay=0.0)
    g = torch.randn(store.padded).sign()                    # constant-sign gradient: every step moves each weight by about lr
    for _ in range(200):
        store.flat_grad.copy_(g)
        ref.grad = g[:ref.numel()].view(ref.shape).clone()
        opt.step(store.grad_shard)
        topt.step()
    moved = (m.weight.float() + opt.master[:ref.numel()].view(ref.shape).float()) - w0     # weights + carried low-order bits
    want = ref.detach() - w0
    assert (want.abs() > 1e-3).all()
    assert float((moved - want).abs().max()) < 0.1 * float(want.abs().max())
    stalled = (w0.to(torch.bfloat16).float() - w0).abs().max()          # scale of one bf16 rounding error, for reference
    assert float((m.weight.float() - ref.detach()).abs().max()) <= 2 * float(stalled) + 1e-3


@pytest.mark.parametrize("resp,gold,want", [
    ("so we get \\boxed{\\frac{3}{4}}", "0.75", 1.0),
    ("The answer is 1,234.", "#### 1234", 1.0),
    ("thus \\boxed{\\dfrac{\\sqrt{2}}{2}} is the value", "\\frac{\\sqrt{2}}{2}", 1.0),
    ("<answer> 45% </answer>", "0.45", 1.0),
    ("it costs $12.50", "12.5", 1.0),
    ("\\boxed{12 \\text{ cm}}", "12", 1.0),
    ("\\boxed{(1, 2)}", "(1,2)", 1.0),
    ("\\boxed{\\{3, 1\\}}".replace("\\{", "{").replace("\\}", "}"), "{1, 3}", 1.0),
    ("\\boxed{x^2+1}", "x^2 + 1", 1.0),
    ("\\boxed{2\\pi}", "6.283185", 1.0),
    ("the result is 7", "8", 0.0),
    ("\\boxed{(1, 3)}", "(1,2)", 0.0),
    ("no number here", "5", 0.0),
    ("\\boxed{3.14159}", "3.14160", 0.0),
    ("1e3", "1000", 1.0),
])
def test_math_verifier_equivalences(resp, gold, want):
    from areal_b200.reward import get_math_verify_worker

    assert get_math_verify_worker().verify(resp, gold) == want


def test_named_dataset_rewards():
    from areal_b200.reward import MathVerifyWorker, clevr_count_70k_reward_fn, geometry3k_reward_fn, gsm8k_reward_fn, math_verify_reward_fn
    from areal_b200.reward.math_verify import last_boxed

    assert last_boxed("a \\boxed{1} b \\boxed{\\frac{a}{b{c}}} c") == "\\frac{a}{b{c}}" and last_boxed("\\boxed{unclosed") is None
    assert geometry3k_reward_fn("", "angle is [45]", [], [], answer="45") == 1.0
    assert geometry3k_reward_fn("", "i think 44.9", [], [], answer="[45]") == 0.0
    assert clevr_count_70k_reward_fn("", "there are [3] cubes", [], [], answer="3") == 1.0
    assert clevr_count_70k_reward_fn("", "maybe four", [], [], answer="4") == 0.0
    assert math_verify_reward_fn("", "x = \\boxed{-\\frac{1}{2}}", [], [], answer="-0.5") == 1.0
    assert gsm8k_reward_fn("", "... #### 72", [], [], answer="blah #### 72") == 1.0
    strict = MathVerifyWorker(try_extract_without_anchor=False)
    assert strict.verify("the number 5 appears", "5") == 0.0 and strict.verify("answer: 5", "5") == 1.0
