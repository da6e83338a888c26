"""PPO / GRPO actor logic on top of a :class:`TrainEngine`: proximal log-prob recompute,
advantage pipeline, mini-batched policy update with the decoupled loss family.

Behaviour follows the reference's ``areal/trainer/ppo/actor.py`` (compute_logp :162,
_compute_advantages :178-323, _ppo_update :369-484, grpo_loss_fn :527-760, proximal
resolution :851-930, staleness stats :1138-1273).
"""
from __future__ import annotations

import functools
from typing import Any, Optional

import torch

from ...algo import advantages as ADV
from ...algo import functional as AF
from ...utils import data as D
from ...utils import stats_tracker


class PPOActor:
    def __init__(self, config, engine):
        self.config = config
        self.engine = engine
        self.adv = ADV.AdvantageComputer(config)
        self.temperature = config.temperature

    # ------------------------------------------------------------------ logp / advantages
    @torch.no_grad()
    def compute_logp(self, data: dict[str, Any]) -> Optional[torch.Tensor]:
        """Recomputed (proximal) log-probs ``[B, L]``, aligned so that position t holds the
        log-prob of token t+1. Skipped when the loss does not need them."""
        cfg = self.config
        if not cfg.recompute_logprob and not cfg.use_decoupled_loss:
            return None
        if cfg.use_decoupled_loss and cfg.prox_logp_method in ("loglinear", "linear", "reuse_train_logp"):
            return None
        self.engine.eval()
        return self.engine.forward_batch(data, output="logprobs", temperature=self.temperature)

    @torch.no_grad()
    def compute_advantages(self, data: dict[str, Any], group_sizes: Optional[list[int]] = None) -> dict[str, Any]:
        self.adv.reduce_group = getattr(self.engine, "cpu_group", None) if getattr(self.engine, "dp_size", 1) > 1 else None
        return self.adv(data, group_sizes=group_sizes)

    # ------------------------------------------------------------------ update
    def ppo_update(self, data: dict[str, Any]) -> list[dict[str, float]]:
        cfg = self.config
        attn = data["attention_mask"]
        loss_mask = data["loss_mask"]
        reward = data["rewards"].float()
        seqlens = attn.sum(-1)
        # ---- batch-level statistics (once per step)
        with stats_tracker.scope("ppo_actor"):
            stats_tracker.denominator(n_seqs=torch.ones_like(reward, dtype=torch.bool),
                                      n_tokens=attn.bool(), n_valid_tokens=loss_mask.bool())
            stats_tracker.stat(task_reward=reward, seq_len=seqlens.float(),
                               no_eos_ratios=(seqlens == attn.shape[1]).float(), denominator="n_seqs")
            stats_tracker.stat(advantages=data["advantages"], kl_rewards=data["kl_rewards"],
                               final_reward=data["tot_rewards"], denominator="n_valid_tokens")
            prompt_lens = (attn.long().sum(-1) - data["loss_mask"].long().sum(-1)).float()
            stats_tracker.stat(prompt_len=prompt_lens, denominator="n_seqs")
            reward_pos = reward > 0
            stats_tracker.denominator(correct_n_seqs=reward_pos, incorrect_n_seqs=~reward_pos)
            stats_tracker.stat(correct_seq_len=seqlens.float(), denominator="correct_n_seqs")
            stats_tracker.stat(incorrect_seq_len=seqlens.float(), denominator="incorrect_n_seqs")
            if getattr(cfg, "log_agent_stats", False):
                # per-trajectory quantities an agent workflow attached to its first exported sequence (tool calls, turns ...):
                # averaged over the rows that begin a trajectory (reference: areal/trainer/ppo/actor.py:385-444)
                if "begin_of_trajectory" not in data:
                    raise RuntimeError("'begin_of_trajectory' is expected in the batch to log agent statistics")
                if not cfg.log_agent_stats_keys:
                    raise RuntimeError("`log_agent_stats_keys` must not be empty when log_agent_stats=True")
                stats_tracker.denominator(agent=(data["begin_of_trajectory"] > 0).bool())
                stats_tracker.stat(**{k: data[k].float() for k in cfg.log_agent_stats_keys}, denominator="agent")
        for k in ("rewards", "tot_rewards", "kl_rewards"):
            data.pop(k, None)
        self.engine.train()
        n_mini = max(1, cfg.ppo_n_minibatches)
        B = attn.shape[0]
        lens = seqlens.tolist()
        from ...utils.seqpack import balanced_greedy_partition

        groups = [g for g in balanced_greedy_partition(lens, min(n_mini, B), equal_count=True) if g]
        loss_fn = functools.partial(
            grpo_loss_fn, eps_clip=cfg.eps_clip, eps_clip_higher=cfg.eps_clip_higher, c_clip=cfg.c_clip,
            rejection_sampling=cfg.rejection_sampling, m2_threshold=cfg.m2_threshold,
            importance_sampling_level=cfg.importance_sampling_level, current_version=self.engine.get_version(),
            prox_logp_method=cfg.prox_logp_method, use_sapo_loss=cfg.use_sapo_loss, sapo_tau_pos=cfg.sapo_tau_pos,
            sapo_tau_neg=cfg.sapo_tau_neg, use_cispo_loss=cfg.use_cispo_loss, use_decoupled_loss=cfg.use_decoupled_loss)
        all_stats = []
        for g in groups:
            mb = D.select_batch(data, g)
            with stats_tracker.scope("ppo_actor"), stats_tracker.scope("update"):
                st = self.engine.train_batch(mb, loss_fn=loss_fn,
                                             loss_weight_fn=lambda x: x["loss_mask"].count_nonzero())
                stats_tracker.scalar(**st)
            all_stats.append(st)
        return all_stats


def resolve_proximal_logp(prox_logp_gt, method: str, old_logp, logprobs, versions, current_version):
    """Which proximal log-probs the loss uses (recomputed forward, an approximation, or the
    training log-probs themselves)."""
    if method == "metrics":
        method = "recompute"            # the loss uses the recomputed log-probs; the approximations are only measured
    if method == "reuse_train_logp":
        return logprobs.detach()
    if method in ("loglinear", "linear"):
        if versions is None or current_version is None:
            raise ValueError(f"prox_logp_method={method} needs per-token versions and the current version")
        return ADV.compute_prox_logp_approximation(old_logp, logprobs, versions, current_version, method)
    if prox_logp_gt is None:
        raise ValueError("prox_logp missing: compute_logp() must run when prox_logp_method='recompute'")
    return prox_logp_gt


def grpo_loss_fn(logprobs: torch.Tensor, entropy: torch.Tensor, input_data: dict, eps_clip: float,
                 eps_clip_higher: Optional[float], c_clip: Optional[float], rejection_sampling=None,
                 m2_threshold: Optional[float] = None, importance_sampling_level: str = "token",
                 current_version: Optional[int] = None, prox_logp_method: str = "recompute",
                 use_sapo_loss: bool = False, sapo_tau_pos: float = 1.0, sapo_tau_neg: float = 1.05,
                 use_cispo_loss: bool = False, use_decoupled_loss: bool = False) -> torch.Tensor:
    """Actor loss of one packed micro-batch plus logging statistics."""
    old_logp = input_data["logprobs"]
    adv = input_data["advantages"]
    loss_mask = input_data["loss_mask"].bool()
    entropy = entropy.detach()
    prox = resolve_proximal_logp(input_data.get("prox_logp"), prox_logp_method, old_logp, logprobs.detach(),
                                 input_data.get("versions"), current_version)
    if m2_threshold is not None:
        loss_mask = ADV.m2po_mask(old_logp, prox, loss_mask, m2_threshold).bool()
    cu = input_data.get("cu_seqlens")
    if use_cispo_loss:
        if use_sapo_loss:
            raise ValueError("CISPO and SAPO are mutually exclusive")
        if importance_sampling_level != "token":
            raise ValueError("CISPO supports token-level importance sampling only")
        loss, stat = AF.cispo_loss_fn(logprobs, prox, old_logp, adv, eps_clip, loss_mask, eps_clip_higher,
                                      rejection_sampling, cu)
    elif use_sapo_loss:
        if use_decoupled_loss:
            raise ValueError("SAPO is incompatible with use_decoupled_loss=True")
        loss, stat = AF.sapo_loss_fn(logprobs, old_logp, adv, sapo_tau_pos, sapo_tau_neg, loss_mask,
                                     importance_sampling_level, cu)
    else:
        loss, stat = AF.ppo_actor_loss_fn(logprobs, prox, old_logp, adv, eps_clip, loss_mask, eps_clip_higher, c_clip,
                                          rejection_sampling, importance_sampling_level, cu)
    teacher = input_data.get("teacher_logp")
    if teacher is not None:
        teacher = teacher.detach()
        rl_w = input_data.get("rl_loss_weight", 1.0)
        kd_w = input_data.get("distill_loss_weight", 0.005)
        denom = loss_mask.sum().clamp(min=1)
        if rl_w == 0:
            term = torch.exp(logprobs - old_logp) * (teacher - logprobs.detach()) * loss_mask
            loss = -kd_w * term.sum() / denom
        else:
            loss = rl_w * loss + kd_w * ((logprobs - teacher) * loss_mask).sum() / denom
    # ---- statistics
    stats_tracker.denominator(n_valid_tokens=loss_mask, clipped_tokens=stat["clip_mask"],
                              dual_clipped_tokens=stat["dual_clip_mask"])
    diff = (old_logp - logprobs.detach()) * loss_mask
    stats_tracker.stat(importance_weight=stat["importance_weight"], approx_kl=stat["approx_kl"],
                       new_logp=logprobs.detach(), old_logp=old_logp, entropy=entropy.float(),
                       actor_loss=stat["loss"], clip_ratio=stat["clip_mask"].float(),
                       dual_clip_ratio=stat["dual_clip_mask"].float(), logp_diff=diff, logp_abs_diff=diff.abs(),
                       denominator="n_valid_tokens")
    if "behave_imp_weight" in stat:
        stats_tracker.denominator(unclipped_behave_tokens=stat["behave_mask"])
        stats_tracker.stat(behave_imp_weight=stat["behave_imp_weight"], behave_approx_kl=stat["behave_approx_kl"],
                           denominator="unclipped_behave_tokens")
        stats_tracker.stat(behave_filtered_ratio=(loss_mask & ~stat["behave_mask"]).float(), denominator="n_valid_tokens")
    if "filtered_fraction" in stat:
        stats_tracker.scalar(rs_filtered_fraction=stat["filtered_fraction"])
    versions = input_data.get("versions")
    if prox_logp_method == "metrics" and versions is not None and current_version is not None and input_data.get("prox_logp") is not None:
        # how far each approximation of the proximal policy is from the recomputed one, on the trained tokens
        # (reference: the 'metrics' method of areal/api/cli_args.py:1832-1845 and its logging in the actor)
        gt = input_data["prox_logp"].float()
        for name in ("loglinear", "linear"):
            ap = ADV.compute_prox_logp_approximation(old_logp, logprobs.detach(), versions, current_version, name)
            err = (ap - gt) * loss_mask
            stats_tracker.stat(**{f"prox_approx/{name}/abs_error": err.abs(), f"prox_approx/{name}/error": err,
                                  f"prox_approx/{name}/ratio_error": (torch.exp(err) - 1).abs() * loss_mask},
                               denominator="n_valid_tokens")
    if versions is not None and current_version is not None:
        m = stat.get("behave_mask", loss_mask) & (versions >= 0)
        stale = (current_version - versions).float()
        stats_tracker.denominator(versioned_tokens=m)
        stats_tracker.stat(staleness=stale, denominator="versioned_tokens")
    return loss
