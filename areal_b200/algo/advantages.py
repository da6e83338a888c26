"""Reward shaping, GAE (token- and turn-level), lambda schedules, proximal-logprob
approximations and M2PO masking.

Semantics follow the reference's ``areal/trainer/ppo/actor.py:178-323`` (advantage
pipeline), ``ppo/gae.py:10-36`` (token GAE), ``:82-163`` (turn GAE), ``ppo/lambda_fn.py:37-115``
(lambda schedules), ``actor.py:768-930`` (proximal approximations) and ``:933-1006`` (M2PO).

The token-level GAE here is a vectorised masked reverse scan: skipped (non-loss) positions
carry the running advantage and the "next value" forward, which is exactly what the
reference's Python loop over T does, but without the per-step launches when
``discount * lambda == 1`` and there is no critic (the GRPO case, solved with one reversed
cumulative sum).
"""
from __future__ import annotations

import math
from typing import Any, Callable, Optional, Union

import torch

from ..utils.data import KLEstimator, Normalization
from . import functional as AF


# --------------------------------------------------------------------------- lambda schedules
def constant_gae_lambda(lengths: torch.Tensor, value: float) -> torch.Tensor:
    return torch.full_like(lengths, float(value), dtype=torch.float32)


def vapo_length_adaptive_gae(lengths: torch.Tensor, alpha: float) -> torch.Tensor:
    """VAPO: ``lambda = 1 - 1/(alpha * L)``, clamped at 0; empty trajectories get 0."""
    if isinstance(alpha, bool) or alpha <= 0:
        raise ValueError("alpha must be positive")
    lf = lengths.float().clamp(min=1.0)
    lam = (1.0 - 1.0 / (float(alpha) * lf)).clamp(min=0.0)
    return torch.where(lengths > 0, lam, torch.zeros_like(lam))


def relative_position_gae_lambda(lengths: torch.Tensor, q: float) -> torch.Tensor:
    """``lambda = q ** (1/(L-1))``: the first step keeps fraction ``q`` of a terminal reward
    whatever the length; L == 1 -> 1, L == 0 -> 0."""
    if isinstance(q, bool) or not math.isfinite(q) or not 0 < q <= 1:
        raise ValueError("q must be in (0, 1]")
    steps = (lengths - 1).clamp(min=1).float()
    lam = torch.exp(math.log(float(q)) / steps)
    return torch.where(lengths > 1, lam, torch.where(lengths == 1, torch.ones_like(lam), torch.zeros_like(lam)))


# --------------------------------------------------------------------------- GAE
def token_level_gae(rewards: torch.Tensor, values: torch.Tensor, loss_mask: torch.Tensor,
                    seq_no_eos_mask: torch.Tensor, discount: float,
                    gae_lambda: Union[float, torch.Tensor]) -> tuple[torch.Tensor, torch.Tensor]:
    """GAE over ``[B, L]`` where only positions with ``loss_mask == 1`` are timesteps.

    ``delta_t = r_t + gamma * V_next - V_t``; ``A_t = delta_t + gamma*lambda*A_next``; masked
    positions repeat the running advantage. ``advantages[:, L-1] = 0``. Returns
    ``(advantages, advantages + values)``."""
    B, L = rewards.shape
    dev = rewards.device
    mask = loss_mask.float()
    lam_is_scalar = not torch.is_tensor(gae_lambda)
    no_critic = not bool(values.any()) if values.numel() else True
    if lam_is_scalar and no_critic and abs(discount * float(gae_lambda) - 1.0) < 1e-12 and abs(discount - 1.0) < 1e-12:
        # A_t = sum of rewards at loss positions >= t (for loss positions), carried otherwise.
        contrib = rewards[:, : L - 1].float() * mask[:, : L - 1]
        suffix = torch.flip(torch.cumsum(torch.flip(contrib, dims=[1]), dim=1), dims=[1])
        # a masked position shows the value of the next loss position to its right
        nxt_loss_suffix = suffix - contrib  # sum strictly right of t
        adv_body = torch.where(mask[:, : L - 1] > 0, suffix, nxt_loss_suffix)
        adv = torch.cat([adv_body, torch.zeros(B, 1, device=dev)], dim=1)
        return adv, adv + values.float()
    if rewards.is_cuda:
        from ..ops import functional as OF

        return OF.gae_scan(rewards, values, loss_mask, seq_no_eos_mask, discount, gae_lambda)    # one thread per sequence
    gl = gae_lambda.float().to(dev) if torch.is_tensor(gae_lambda) else torch.full((B,), float(gae_lambda), device=dev)
    dl = discount * gl
    adv = torch.zeros(B, L, dtype=torch.float32, device=dev)
    last = torch.zeros(B, dtype=torch.float32, device=dev)
    nextv = values[:, L - 1].float() * seq_no_eos_mask.float()
    vf, rf = values.float(), rewards.float()
    for t in range(L - 2, -1, -1):
        delta = rf[:, t] + discount * nextv - vf[:, t]
        new = delta + dl * last
        m = mask[:, t]
        nextv = nextv * (1 - m) + vf[:, t] * m
        last = last * (1 - m) + new * m
        adv[:, t] = last
    return adv, adv + vf


def turn_level_gae(rewards: torch.Tensor, values: torch.Tensor, loss_mask: torch.Tensor, turn_ids: torch.Tensor,
                   seq_no_eos_mask: torch.Tensor, discount: float,
                   gae_lambda: Union[float, torch.Tensor]) -> tuple[torch.Tensor, torch.Tensor]:
    """GAE where every generated turn is one macro timestep: the turn's reward is the sum of
    its token rewards, its value is the value at its first generated token, and the turn's
    advantage is broadcast to its tokens."""
    if turn_ids.shape != loss_mask.shape:
        raise ValueError("turn_ids must have the shape of loss_mask")
    if turn_ids.dtype not in (torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64):
        raise ValueError("turn_ids must be integral")
    B, L = rewards.shape
    dev = rewards.device
    valid = loss_mask.bool()
    tid = turn_ids.long().clamp(0, L - 1)
    turn_r = torch.zeros(B, L, device=dev, dtype=torch.float32).scatter_add_(1, tid, rewards.float() * valid.float())
    pos = torch.arange(L, device=dev).expand(B, -1)
    first = torch.full((B, L), L, device=dev, dtype=torch.long)
    first.scatter_reduce_(1, tid, torch.where(valid, pos, torch.full_like(pos, L)), reduce="amin", include_self=True)
    turn_valid = first < L
    turn_v = values.float().gather(1, first.clamp(max=L - 1)) * turn_valid.float()
    n_slots = L
    if dev.type == "cpu":
        n_slots = int(torch.where(valid, tid, torch.full_like(tid, -1)).amax().item()) + 1
    gl = gae_lambda.float().to(dev) if torch.is_tensor(gae_lambda) else torch.full((B,), float(gae_lambda), device=dev)
    dl = discount * gl
    turn_adv = torch.zeros(B, L, device=dev, dtype=torch.float32)
    last = torch.zeros(B, device=dev)
    nextv = values[:, L - 1].float() * seq_no_eos_mask.float()
    for k in range(n_slots - 1, -1, -1):
        delta = turn_r[:, k] + discount * nextv - turn_v[:, k]
        new = delta + dl * last
        m = turn_valid[:, k]
        turn_adv[:, k] = torch.where(m, new, torch.zeros_like(new))
        nextv = torch.where(m, turn_v[:, k], nextv)
        last = torch.where(m, new, last)
    adv = turn_adv.gather(1, tid) * loss_mask.float()
    ret = (turn_adv + turn_v).gather(1, tid) * loss_mask.float() + values.float() * (1 - loss_mask.float())
    return adv, ret


# --------------------------------------------------------------------------- advantage pipeline
class AdvantageComputer:
    """Turns a padded rollout batch (rewards, behaviour logprobs, masks) into advantages,
    returns and shaped rewards. One instance per actor config."""

    def __init__(self, config, reduce_group=None):
        self.config = config
        self.reduce_group = reduce_group
        self.reward_norm = Normalization(config.reward_norm) if config.reward_norm else None
        self.adv_norm = Normalization(config.adv_norm) if config.adv_norm else None
        self.kl_estimator = KLEstimator(config.kl_estimator)
        self.gae_lambda_fn: Optional[Callable] = None
        lam = config.gae_lambda
        if isinstance(lam, str):
            from ..utils.dynamic_import import import_from_string

            self.gae_lambda_fn = import_from_string(lam)

    def _lambda(self, loss_mask, turn_ids):
        if self.gae_lambda_fn is None:
            lam = float(self.config.gae_lambda)
            if not math.isfinite(lam):
                raise ValueError("gae_lambda must be finite")
            return lam
        if self.config.gae_timestep_unit == "turn":
            valid = loss_mask.bool()
            tid = torch.where(valid, turn_ids.long(), torch.full_like(turn_ids.long(), -1))
            lengths = torch.tensor([len(set(r[r >= 0].tolist())) for r in tid], device=loss_mask.device)
        else:
            lengths = loss_mask.sum(-1).long()
        return self.gae_lambda_fn(lengths, **dict(getattr(self.config, "gae_lambda_kwargs", None) or {}))

    @torch.no_grad()
    def __call__(self, data: dict[str, Any], group_sizes: Optional[list[int]] = None) -> dict[str, Any]:
        cfg = self.config
        B = data["input_ids"].shape[0]
        dev = data["input_ids"].device
        rows = torch.arange(B, device=dev)
        rewards_in = data["rewards"].float()
        attn = data["attention_mask"]
        seqlens = attn.sum(-1).long()
        if cfg.overlong_reward_penalty:
            if cfg.overlong_tokens is None or cfg.overlong_penalty_factor is None:
                raise ValueError("overlong penalty needs overlong_tokens and overlong_penalty_factor")
            resp_len = data["loss_mask"].sum(-1)
            rewards_in = AF.reward_overlong_penalty(rewards_in, resp_len, cfg.overlong_tokens,
                                                    cfg.overlong_penalty_factor, cfg.max_new_tokens)
        score = ((rewards_in + cfg.reward_bias) * cfg.reward_scaling).clamp(-cfg.reward_clip, cfg.reward_clip)
        if self.reward_norm is not None:
            score = self.reward_norm(score, group_sizes=group_sizes, reduce_group=self.reduce_group)
        loss_mask = torch.roll(data["loss_mask"].float(), shifts=-1, dims=-1)
        turn_ids = data.get("turn_ids")
        if turn_ids is not None:
            turn_ids = torch.roll(turn_ids, shifts=-1, dims=-1)
            turn_ids[:, -1] = -1
        elif cfg.gae_timestep_unit == "turn":
            raise ValueError("gae_timestep_unit='turn' needs 'turn_ids' in the rollout data")
        if not cfg.use_decoupled_loss and cfg.recompute_logprob:
            if data.get("prox_logp") is None:
                raise ValueError("recompute_logprob=True but prox_logp is missing (compute_logp was skipped)")
            old_logp = data["logprobs"] = data["prox_logp"]
        else:
            old_logp = torch.roll(data["logprobs"].float(), shifts=-1, dims=-1)
            if not cfg.use_decoupled_loss:
                data["prox_logp"] = old_logp
        ref_logp = data.get("ref_logp")
        ref_logp = torch.zeros_like(old_logp) if ref_logp is None else ref_logp.float()
        ref_logp = ref_logp * loss_mask
        old_logp = old_logp * loss_mask
        no_eos = seqlens == attn.shape[1]
        kl_r = -cfg.kl_ctl * self.kl_estimator(old_logp, ref_logp)
        kl_rewards = kl_r.clone()
        kl_r[rows, seqlens - 1] = 0
        gae_kl = kl_r.clone()
        outcome = torch.zeros_like(kl_r)
        idx = (seqlens - 2).clamp(min=0)
        outcome[rows, idx] = torch.where(no_eos, torch.zeros_like(score), score) if cfg.mask_no_eos_with_zero else score
        values = data["values"].float() if "values" in data else torch.zeros_like(kl_r)
        lam = self._lambda(loss_mask, turn_ids)
        if cfg.gae_timestep_unit == "turn":
            adv, ret = turn_level_gae(outcome, values, loss_mask, turn_ids, no_eos, cfg.discount, lam)
            adv = adv + gae_kl
        else:
            adv, ret = token_level_gae(gae_kl + outcome, values, loss_mask, no_eos, cfg.discount, lam)
        data["returns"] = ret
        if self.adv_norm is not None:
            adv = self.adv_norm(adv, loss_mask, group_sizes=group_sizes, reduce_group=self.reduce_group)
        data["advantages"] = adv
        data["kl_rewards"] = kl_rewards
        data["tot_rewards"] = gae_kl + outcome
        data["loss_mask"] = loss_mask
        data["logprobs"] = old_logp
        return data


# --------------------------------------------------------------------------- proximal approximations
@torch.no_grad()
def compute_prox_logp_approximation(old_logp: torch.Tensor, logprobs: torch.Tensor, versions: torch.Tensor,
                                    current_version: int, method: str = "loglinear") -> torch.Tensor:
    """Approximates the proximal policy's log-prob without a forward pass by interpolating
    between the behaviour policy (version ``v_b`` per token) and the current policy
    (version ``v_theta``) at ``v_prox = v_theta - 1``:

        alpha = clamp((v_prox - v_b) / (v_theta - v_b), 0, 1)   (0 for prompt tokens, v_theta <= v_b)
        loglinear: prox = old + alpha * (logp - old)
        linear   : prox = log(p_old + alpha * (p - p_old))
    """
    v_theta = float(current_version)
    v_b = versions.float()
    v_prox = v_theta - 1.0
    gap = v_theta - v_b
    alpha = torch.where((v_b >= 0) & (gap > 0), ((v_prox - v_b) / gap.clamp(min=1e-9)).clamp(0.0, 1.0),
                        torch.zeros_like(v_b))
    lp, old = logprobs.detach().float(), old_logp.float()
    if method == "loglinear":
        return old + alpha * (lp - old)
    if method == "linear":
        p_old, p = torch.exp(old), torch.exp(lp)
        return torch.log((p_old + alpha * (p - p_old)).clamp(min=1e-30))
    raise ValueError(f"unknown approximation method {method}")


@torch.no_grad()
def m2po_mask(old_logp: torch.Tensor, prox_logp: torch.Tensor, loss_mask: torch.Tensor, m2_threshold: float
              ) -> torch.Tensor:
    """M2PO: drops the tokens with the largest second moment ``(old - prox)^2`` until the mean
    over the kept tokens falls below ``m2_threshold`` (at least one token is kept)."""
    mask = loss_mask.bool()
    flat_mask = mask.reshape(-1)
    m2 = ((old_logp.float() - prox_logp.float()) ** 2).reshape(-1)
    idx = flat_mask.nonzero(as_tuple=True)[0]
    if idx.numel() == 0:
        return loss_mask
    vals = m2[idx]
    order = torch.argsort(vals, descending=True)
    sorted_vals = vals[order]
    n = sorted_vals.numel()
    # suffix means: mean of the remainder after dropping the k largest
    suffix_sum = torch.flip(torch.cumsum(torch.flip(sorted_vals, [0]), 0), [0])
    counts = torch.arange(n, 0, -1, device=vals.device, dtype=vals.dtype)
    suffix_mean = suffix_sum / counts
    ok = (suffix_mean < m2_threshold).nonzero(as_tuple=True)[0]
    k = int(ok[0].item()) if ok.numel() > 0 else n - 1
    k = min(k, n - 1)
    drop = idx[order[:k]]
    new = flat_mask.clone()
    new[drop] = False
    return new.reshape(loss_mask.shape).to(loss_mask.dtype)
