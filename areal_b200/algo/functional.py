"""Policy-optimisation math: rejection sampling between proximal and behaviour policies,
decoupled PPO / GRPO / GSPO actor loss, SAPO, CISPO, critic loss, DPO, DAPO overlong
penalty, masked normalisation.

Numerical semantics match the reference's ``areal/utils/functional/functional.py``
(masked_normalization :16, sequence-level ratio :56, apply_rejection_sampling :185-437,
ppo_actor_loss_fn :452-596, sapo_loss_fn :599, cispo_loss_fn :678, dpo :796-857,
ppo_critic_loss_fn :869, reward_overlong_penalty :937). Padded ``[B, L]`` and packed ``[T]``
inputs are handled by one code path: both are reduced per sequence through a segment index.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F


# --------------------------------------------------------------------------- segment helpers
def _segment_index(shape_like: torch.Tensor, cu_seqlens: Optional[torch.Tensor]):
    """Returns (flat view fn, segment ids [N], number of segments) for padded or packed input."""
    if shape_like.dim() == 2:
        B, L = shape_like.shape
        seg = torch.arange(B, device=shape_like.device).repeat_interleave(L)
        return seg, B
    if cu_seqlens is None:
        raise ValueError("cu_seqlens is required for 1-D packed tensors at sequence level")
    nseg = cu_seqlens.numel() - 1
    lens = (cu_seqlens[1:] - cu_seqlens[:-1]).long()
    seg = torch.arange(nseg, device=shape_like.device).repeat_interleave(lens)
    if seg.numel() < shape_like.numel():  # trailing pad tokens join the last segment
        seg = torch.cat([seg, seg.new_full((shape_like.numel() - seg.numel(),), max(nseg - 1, 0))])
    return seg, nseg


def _seg_sum(x: torch.Tensor, seg: torch.Tensor, nseg: int) -> torch.Tensor:
    return torch.zeros(nseg, device=x.device, dtype=x.dtype).scatter_add_(0, seg, x.reshape(-1))


def _seg_max(x: torch.Tensor, seg: torch.Tensor, nseg: int) -> torch.Tensor:
    out = torch.full((nseg,), float("-inf"), device=x.device, dtype=x.dtype)
    return out.scatter_reduce_(0, seg, x.reshape(-1), reduce="amax")


# --------------------------------------------------------------------------- normalisation
@torch.no_grad()
def masked_normalization(x: torch.Tensor, mask: Optional[torch.Tensor] = None, dim=None, unbiased: bool = False,
                         eps: float = 1e-5, high_precision: bool = True, all_reduce: bool = True,
                         reduce_group=None) -> torch.Tensor:
    """Whitening of ``x`` over the masked entries (global across ``reduce_group``)."""
    dtype = torch.float64 if high_precision else torch.float32
    xf = x.to(dtype)
    if dim is None:
        dim = tuple(range(x.dim()))
    m = torch.ones_like(xf) if mask is None else mask.to(dtype)
    xf = xf * m
    n = m.sum(dim, keepdim=True)
    s = xf.sum(dim, keepdim=True)
    ss = (xf * xf).sum(dim, keepdim=True)
    if all_reduce and dist.is_initialized():
        for t in (n, s, ss):
            dist.all_reduce(t, group=reduce_group)
    mean = s / n
    var = ss / n - mean * mean
    if unbiased:
        var = var * (n / (n - 1).clamp(min=1))
    return (((xf - mean) * m) / (var.clamp(min=0).sqrt() + eps)).float()


# --------------------------------------------------------------------------- rejection sampling
@dataclass
class RejectionSamplingResult:
    loss_mask: torch.Tensor
    behave_imp_weight: torch.Tensor
    filtered_fraction: float


def bernoulli_kl(log_p: torch.Tensor, log_q: torch.Tensor, eps: float = 1e-8) -> torch.Tensor:
    """KL between Bernoulli(p) and Bernoulli(q) given log p and log q."""
    p = torch.exp(log_p).clamp(eps, 1 - eps)
    q = torch.exp(log_q).clamp(eps, 1 - eps)
    return p * torch.log(p / q) + (1 - p) * torch.log((1 - p) / (1 - q))


def _in_bounds(v: torch.Tensor, cfg) -> torch.Tensor:
    ok = torch.ones_like(v, dtype=torch.bool)
    if cfg.upper is not None:
        ok &= v <= cfg.upper
    if cfg.lower is not None:
        ok &= v >= cfg.lower
    return ok


def _rs_metric(cfg, log_ratio, prox, old):
    if cfg.metric == "ratio":
        return torch.exp(log_ratio)
    if cfg.metric == "kl_k1":
        return log_ratio
    if cfg.metric == "kl_k2":
        return 0.5 * log_ratio * log_ratio
    if cfg.metric == "kl_k3":
        return torch.exp(-log_ratio) - 1 + log_ratio
    if cfg.metric == "binary_kl":
        return torch.maximum(bernoulli_kl(prox, old), bernoulli_kl(old, prox))
    raise ValueError(f"unknown rejection metric {cfg.metric}")


@torch.no_grad()
def apply_rejection_sampling(proximal_logprobs: torch.Tensor, old_logprobs: torch.Tensor, loss_mask: torch.Tensor,
                             cu_seqlens: Optional[torch.Tensor], config) -> RejectionSamplingResult:
    """Filters (``mask``) or truncates (``clamp``) tokens / sequences whose proximal-vs-behaviour
    divergence leaves ``[lower, upper]``; returns the importance weight ``pi_prox / pi_behave``."""
    if proximal_logprobs.shape != old_logprobs.shape or proximal_logprobs.shape != loss_mask.shape:
        raise ValueError("proximal_logprobs, old_logprobs and loss_mask must share a shape")
    if proximal_logprobs.dim() not in (1, 2):
        raise ValueError("expected packed 1-D or padded 2-D tensors")
    prox, old = proximal_logprobs.detach().float(), old_logprobs.detach().float()
    lr = prox - old
    lr = torch.where(torch.isfinite(lr), lr, torch.zeros_like(lr))
    metric = _rs_metric(config, lr, prox, old)
    weight = torch.exp(lr)
    raw_weight = weight
    valid = loss_mask.bool()
    lo = config.lower if config.lower is not None else 0.0
    inb = None
    if config.level == "sequence":
        seg, nseg = _segment_index(loss_mask, cu_seqlens)
        vflat = valid.reshape(-1)
        counts = _seg_sum(vflat.float(), seg, nseg)
        geometric = config.metric == "ratio"
        agg_src = (lr if geometric else metric).reshape(-1)
        masked = torch.where(vflat, agg_src, torch.zeros_like(agg_src))
        if geometric:
            seq_w = torch.exp(_seg_sum(masked, seg, nseg) / counts.clamp(min=1))
            weight = seq_w[seg].reshape(loss_mask.shape)
            raw_weight = weight
        if config.agg == "sum":
            seq_val = _seg_sum(masked, seg, nseg)
        elif config.agg == "mean":
            seq_val = _seg_sum(masked, seg, nseg) / counts.clamp(min=1)
        elif config.agg == "max":
            seq_val = _seg_max(torch.where(vflat, agg_src, torch.full_like(agg_src, float("-inf"))), seg, nseg)
            seq_val = torch.where(counts == 0, torch.zeros_like(seq_val), seq_val)
        else:
            raise ValueError(f"unknown aggregation {config.agg}")
        seq_metric = torch.exp(seq_val) if geometric else seq_val
        seq_ok = _in_bounds(seq_metric, config)
        tok_ok = seq_ok[seg].reshape(loss_mask.shape)
        if config.action == "mask":
            inb = tok_ok
        else:
            weight = torch.where(tok_ok, weight, weight.clamp(min=lo, max=config.upper))
    else:
        if config.action == "mask":
            inb = _in_bounds(metric, config)
        else:
            weight = weight.clamp(min=lo, max=config.upper)
    total = int(valid.sum().item())
    if config.action == "mask":
        new_mask = (valid & inb).to(loss_mask.dtype)
        frac = int((valid & ~inb).sum().item()) / max(total, 1)
    else:
        new_mask = loss_mask
        frac = int((valid & (raw_weight != weight)).sum().item()) / max(total, 1)
    weight = torch.where(new_mask.bool(), weight, torch.zeros_like(weight))
    return RejectionSamplingResult(new_mask, weight, frac)


# --------------------------------------------------------------------------- actor losses
def sequence_level_ratio_and_advantages(log_ratio, advantages, loss_mask, cu_seqlens):
    """GSPO: per-sequence geometric-mean ratio and mean advantage, broadcast to tokens."""
    seg, nseg = _segment_index(loss_mask, cu_seqlens)
    m = loss_mask.bool().reshape(-1)
    cnt = _seg_sum(m.to(log_ratio.dtype), seg, nseg).clamp(min=1)
    lr_mean = _seg_sum(torch.where(m, log_ratio.reshape(-1), torch.zeros_like(log_ratio.reshape(-1))), seg, nseg) / cnt
    adv_flat = advantages.reshape(-1)
    adv_mean = _seg_sum(torch.where(m, adv_flat, torch.zeros_like(adv_flat)), seg, nseg) / cnt.to(adv_flat.dtype)
    ratio = torch.where(m, torch.exp(lr_mean)[seg], torch.zeros_like(adv_flat, dtype=log_ratio.dtype))
    adv = torch.where(m, adv_mean[seg], torch.zeros_like(adv_flat))
    return ratio.reshape(loss_mask.shape), adv.reshape(loss_mask.shape)


def ppo_actor_loss_fn(logprobs: torch.Tensor, proximal_logprobs: torch.Tensor, old_logprobs: torch.Tensor,
                      advantages: torch.Tensor, eps_clip: float, loss_mask: torch.Tensor,
                      eps_clip_higher: Optional[float] = None, c_clip: Optional[float] = None,
                      rejection_sampling=None, importance_sampling_level: str = "token",
                      cu_seqlens: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, dict]:
    """Clipped surrogate with decoupled proximal / behaviour policies.

    ``ratio = exp(logp - prox)``; ``L = max(-A*ratio, -A*clip(ratio))``; optional dual clip
    ``min(L, sign(A)*c*A)``; optional behaviour importance weight ``exp(prox - old)`` from
    rejection sampling. The denominator is the number of valid tokens *before* rejection so
    the loss weight stays consistent with the engine's global token count."""
    if (logprobs.is_cuda and importance_sampling_level == "token" and _FUSED_LOSS
            and (rejection_sampling is None or rejection_sampling.level == "token")):
        if c_clip is not None and c_clip <= 1.0:
            raise ValueError("c_clip must be > 1")
        return _ppo_actor_loss_fused(logprobs, proximal_logprobs, old_logprobs, advantages, eps_clip, loss_mask, eps_clip_higher,
                                     c_clip, rejection_sampling)
    loss_mask = loss_mask.bool()
    denom = loss_mask.count_nonzero().clamp(min=1)
    stat_mask = loss_mask
    rs = None
    if rejection_sampling is not None:
        rs = apply_rejection_sampling(proximal_logprobs, old_logprobs, loss_mask, cu_seqlens, rejection_sampling)
        loss_mask = rs.loss_mask.bool()
    if importance_sampling_level == "sequence":
        ratio, advantages = sequence_level_ratio_and_advantages(logprobs - proximal_logprobs, advantages, loss_mask,
                                                                cu_seqlens)
    elif importance_sampling_level == "token":
        ratio = torch.where(stat_mask, torch.exp(logprobs - proximal_logprobs), torch.zeros_like(logprobs))
    else:
        raise ValueError("importance_sampling_level must be 'token' or 'sequence'")
    hi = eps_clip if eps_clip_higher is None else eps_clip_higher
    clipped = ratio.clamp(1.0 - eps_clip, 1.0 + hi)
    l1, l2 = -advantages * ratio, -advantages * clipped
    clip_mask = l1.detach() < l2.detach()
    loss = torch.max(l1, l2)
    if c_clip is not None:
        if c_clip <= 1.0:
            raise ValueError("c_clip must be > 1")
        l3 = torch.sign(advantages) * c_clip * advantages
        dual_mask = l3.detach() < loss.detach()
        loss = torch.min(loss, l3)
    else:
        dual_mask = torch.zeros_like(clip_mask)
    stat: dict = {}
    if rs is not None:
        bkl = proximal_logprobs.detach() - old_logprobs.detach()
        bmask = (rs.behave_imp_weight > 0) & loss_mask
        stat.update(behave_approx_kl=torch.where(bmask, bkl, torch.zeros_like(bkl)),
                    behave_imp_weight=rs.behave_imp_weight, behave_mask=bmask,
                    filtered_fraction=rs.filtered_fraction)
        loss = loss * rs.behave_imp_weight
    per_token = loss.detach()
    total = torch.where(loss_mask, loss, torch.zeros_like(loss)).sum() / denom
    n_tot = stat_mask.numel()
    n_valid = int(stat_mask.count_nonzero().item())
    stat.update(loss=per_token, importance_weight=ratio.detach(), approx_kl=(logprobs - proximal_logprobs).detach(),
                clip_mask=clip_mask & stat_mask, dual_clip_mask=dual_mask & stat_mask,
                n_total_tokens=float(n_tot), n_valid_tokens=float(n_valid), n_masked_tokens=float(n_tot - n_valid),
                masked_token_ratio=1.0 - n_valid / max(n_tot, 1))
    return total, stat


_FUSED_LOSS = __import__("os").environ.get("AREAL_FUSED_LOSS", "1") != "0"
_RS_METRICS = {"ratio": 0, "kl_k1": 1, "kl_k2": 2, "kl_k3": 3, "binary_kl": 4}


def _ppo_actor_loss_fused(logprobs, proximal_logprobs, old_logprobs, advantages, eps_clip, loss_mask, eps_clip_higher, c_clip,
                          rs_cfg) -> tuple[torch.Tensor, dict]:
    """The token-level loss, its gradient and all per-token statistics from one kernel pass
    (``ops/csrc/rl_loss.cu``); same outputs as the eager statement above."""
    from ..ops import functional as OF

    shape = logprobs.shape
    stat_mask = loss_mask.bool()
    action = 0 if rs_cfg is None else (1 if rs_cfg.action == "mask" else 2)
    if rs_cfg is not None and rs_cfg.metric not in _RS_METRICS:
        raise ValueError(f"unknown rejection metric {rs_cfg.metric}")
    total, loss_tok, ratio, behave_w, flags, sums = OF.ppo_token_loss(
        logprobs, proximal_logprobs, old_logprobs, advantages, stat_mask, eps_clip, eps_clip_higher, c_clip, rs_action=action,
        rs_metric=_RS_METRICS[rs_cfg.metric] if rs_cfg is not None else 0,
        rs_lower=rs_cfg.lower if rs_cfg is not None else None, rs_upper=rs_cfg.upper if rs_cfg is not None else None)
    flags = flags.view(shape)
    stat: dict = dict(loss=loss_tok.view(shape), importance_weight=ratio.view(shape),
                      approx_kl=(logprobs.detach() - proximal_logprobs.detach()),
                      clip_mask=(flags & 1).bool(), dual_clip_mask=(flags & 2).bool())
    if rs_cfg is not None:
        bmask = (flags & 4).bool()
        bkl = proximal_logprobs.detach() - old_logprobs.detach()
        stat.update(behave_approx_kl=torch.where(bmask, bkl, torch.zeros_like(bkl)), behave_imp_weight=behave_w.view(shape),
                    behave_mask=bmask, filtered_fraction=(sums[3] / sums[1].clamp(min=1.0)).float())
    n_tot = stat_mask.numel()
    stat.update(n_total_tokens=float(n_tot), n_valid_tokens=sums[1].float(), n_masked_tokens=(n_tot - sums[1]).float(),
                masked_token_ratio=(1.0 - sums[1] / max(n_tot, 1)).float())
    return total, stat


def sapo_loss_fn(logprobs, old_logprobs, advantages, tau_pos: float, tau_neg: float, loss_mask,
                 importance_sampling_level: str = "token", cu_seqlens=None) -> tuple[torch.Tensor, dict]:
    """Soft adaptive policy optimisation: ``L = -gate * A`` with
    ``gate = sigmoid(tau * (ratio - 1)) * 4 / tau`` and tau chosen by the sign of A."""
    if tau_pos <= 0 or tau_neg <= 0:
        raise ValueError("SAPO temperatures must be positive")
    loss_mask = loss_mask.bool()
    denom = loss_mask.count_nonzero().clamp(min=1)
    if importance_sampling_level == "sequence":
        ratio, advantages = sequence_level_ratio_and_advantages(logprobs - old_logprobs, advantages, loss_mask, cu_seqlens)
    else:
        ratio = torch.exp(logprobs - old_logprobs)
    gate_pos = torch.sigmoid(tau_pos * (ratio - 1.0)) * (4.0 / tau_pos)
    gate_neg = torch.sigmoid(tau_neg * (ratio - 1.0)) * (4.0 / tau_neg)
    gate = torch.where(advantages > 0, gate_pos, gate_neg)
    loss = -gate * advantages
    per_token = loss.detach()
    total = torch.where(loss_mask, loss, torch.zeros_like(loss)).sum() / denom
    stat = dict(loss=per_token, importance_weight=ratio.detach(), approx_kl=(logprobs - old_logprobs).detach(),
                sapo_soft_gate=gate.detach(), clip_mask=torch.zeros_like(loss_mask),
                dual_clip_mask=torch.zeros_like(loss_mask))
    return total, stat


def cispo_loss_fn(logprobs, proximal_logprobs, old_logprobs, advantages, eps_clip: float, loss_mask,
                  eps_clip_higher: Optional[float] = None, rejection_sampling=None,
                  cu_seqlens=None) -> tuple[torch.Tensor, dict]:
    """Clipped-IS-weight policy optimisation: ``L = -sg(clip(ratio)) * A * logp`` (token level)."""
    loss_mask = loss_mask.bool()
    denom = loss_mask.count_nonzero().clamp(min=1)
    stat_mask = loss_mask
    rs = None
    if rejection_sampling is not None:
        rs = apply_rejection_sampling(proximal_logprobs, old_logprobs, loss_mask, cu_seqlens, rejection_sampling)
        loss_mask = rs.loss_mask.bool()
    ratio = torch.exp(logprobs.detach() - proximal_logprobs)
    hi = eps_clip if eps_clip_higher is None else eps_clip_higher
    w = ratio.clamp(1.0 - eps_clip, 1.0 + hi).detach()
    loss = -w * advantages * logprobs
    stat: dict = {}
    if rs is not None:
        loss = loss * rs.behave_imp_weight
        stat.update(behave_imp_weight=rs.behave_imp_weight, filtered_fraction=rs.filtered_fraction,
                    behave_mask=(rs.behave_imp_weight > 0) & loss_mask,
                    behave_approx_kl=torch.where(loss_mask, proximal_logprobs.detach() - old_logprobs.detach(),
                                                 torch.zeros_like(old_logprobs)))
    per_token = loss.detach()
    total = torch.where(loss_mask, loss, torch.zeros_like(loss)).sum() / denom
    clip_mask = (ratio != w) & stat_mask
    stat.update(loss=per_token, importance_weight=torch.where(stat_mask, ratio, torch.zeros_like(ratio)),
                approx_kl=(logprobs - proximal_logprobs).detach(), clip_mask=clip_mask,
                dual_clip_mask=torch.zeros_like(clip_mask))
    return total, stat


# --------------------------------------------------------------------------- critic / DPO / misc
def ppo_critic_loss_fn(value: torch.Tensor, old_value: torch.Tensor, target_value: torch.Tensor, value_eps_clip: float,
                       loss_mask: torch.Tensor, loss_fn_type: str = "mse") -> tuple[torch.Tensor, dict]:
    """``max(l(v, R), l(v_old + clamp(v - v_old, +-eps), R))`` with l = 0.5*sq or Huber(10)."""
    loss_mask = loss_mask.bool()
    if loss_fn_type == "huber":
        def l(a, b):
            return F.huber_loss(a, b, reduction="none", delta=10.0)
    elif loss_fn_type == "mse":
        def l(a, b):
            return 0.5 * (a - b) ** 2
    else:
        raise ValueError(f"unknown value loss {loss_fn_type}")
    orig = l(value, target_value)
    clipped_v = old_value + (value - old_value).clamp(-value_eps_clip, value_eps_clip)
    clip = l(clipped_v, target_value)
    loss = torch.max(orig, clip)
    clip_mask = (clip.detach() > orig.detach()) & loss_mask
    total = torch.where(loss_mask, loss, torch.zeros_like(loss)).sum() / loss_mask.count_nonzero().clamp(min=1)
    return total, dict(clip_mask=clip_mask, loss=loss.detach())


def dpo_pair_logratios(logprobs: torch.Tensor, ref_logprobs: torch.Tensor, loss_mask: torch.Tensor,
                       cu_seqlens: torch.Tensor):
    """Per-sequence summed log-ratios (fp64); sequences alternate chosen, rejected."""
    seg, nseg = _segment_index(loss_mask, cu_seqlens)
    m = loss_mask.reshape(-1).to(torch.float64)
    pol = _seg_sum(logprobs.reshape(-1).to(torch.float64) * m, seg, nseg)
    ref = _seg_sum(ref_logprobs.reshape(-1).to(torch.float64) * m, seg, nseg)
    lens = _seg_sum(m, seg, nseg)
    return pol[0::2], pol[1::2], ref[0::2], ref[1::2], lens[0::2], lens[1::2]


def dpo_preference_loss(pol_c, pol_r, ref_c, ref_r, beta: float, loss_type: str = "sigmoid", len_c=None, len_r=None):
    delta = (pol_c - ref_c) - (pol_r - ref_r)
    if loss_type == "sigmoid":
        loss = -F.logsigmoid(beta * delta)
    elif loss_type == "ipo":
        if len_c is None or len_r is None:
            raise ValueError("IPO needs sequence lengths")
        d = (pol_c - ref_c) / len_c.clamp(min=1) - (pol_r - ref_r) / len_r.clamp(min=1)
        loss = (d - 1.0 / (2.0 * beta)) ** 2
    else:
        raise ValueError(f"unknown DPO loss {loss_type}")
    stats = dict(reward_chosen=(beta * (pol_c - ref_c)).detach(), reward_rejected=(beta * (pol_r - ref_r)).detach(),
                 accuracy=(delta > 0).float().detach())
    return loss.mean().float(), stats


def reward_overlong_penalty(rewards: torch.Tensor, response_lens: torch.Tensor, overlong_tokens: int,
                            overlong_penalty_factor: float, max_response_length: int) -> torch.Tensor:
    """DAPO soft overlong punishment: linear penalty inside the last ``overlong_tokens``."""
    expected = max_response_length - overlong_tokens
    exceed = response_lens.float() - expected
    pen = (-exceed / overlong_tokens * overlong_penalty_factor).clamp(max=0.0)
    return rewards + pen.to(rewards.dtype)


def sft_loss_fn(logprobs: torch.Tensor, loss_mask: torch.Tensor) -> torch.Tensor:
    loss_mask = loss_mask.bool()
    return -torch.where(loss_mask, logprobs, torch.zeros_like(logprobs)).sum() / loss_mask.count_nonzero().clamp(min=1)


def rw_loss_fn(scores: torch.Tensor) -> tuple[torch.Tensor, dict]:
    """Bradley-Terry on terminal-token scores; rows alternate chosen, rejected."""
    c, r = scores[0::2].float(), scores[1::2].float()
    loss = -F.logsigmoid(c - r).mean()
    return loss, dict(acc=(c > r).float().mean().detach(), margin=(c - r).mean().detach())
