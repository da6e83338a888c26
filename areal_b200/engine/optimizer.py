"""Sharded AdamW over a :class:`FlatParamStore` plus learning-rate schedules.

Step protocol (reference: ``areal/engine/fsdp_engine.py:696-727`` and
``fsdp_utils/grad.py:112-232``): global L2 grad norm over all shards -> clip coefficient ->
non-finite norm skips the update (``update_successful = 0``) -> fused AdamW on the local
shard (fp32 master, bf16 compute copy refreshed in the same kernel). The clip coefficient
and the skip flag stay on the device, so a step issues no host synchronisation until the
caller reads the returned statistics.

Variants selected by ``OptimizerConfig`` (reference ``areal/engine/fsdp_utils/optimizer.py``):

* ``type: adam_bf16`` -- ``AnyPrecisionAdamW`` (:44-192): moments kept in bf16 and a bf16 Kahan
  compensation buffer beside the bf16 weights instead of an fp32 master copy: 8 bytes of state
  per parameter instead of 12, at the numerics of compensated summation;
* ``offload: true`` -- ``PerLayerOptimWrapper`` (:324-633): master weights and moments live in
  pinned host memory and travel through the GPU in chunks (copy-in of chunk i + 1 overlaps the
  update of chunk i and the copy-out of chunk i - 1), so a model whose optimizer state does not
  fit beside its activations still trains;
* ``type: sgd`` -- L2 weight decay as ``torch.optim.SGD`` applies it.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import functional as OF
from .flat_params import FlatParamStore


def lr_lambda(step: int, total_steps: int, warmup_steps: int, kind: str, min_lr_ratio: float) -> float:
    """Multiplier of the base LR at ``step`` (0-based): linear warm-up, then constant /
    linear / cosine decay to ``min_lr_ratio``."""
    if warmup_steps > 0 and step < warmup_steps:
        return float(step + 1) / float(warmup_steps)
    if kind == "constant":
        return 1.0
    span = max(1, total_steps - warmup_steps)
    prog = min(1.0, max(0.0, (step - warmup_steps) / span))
    if kind == "linear":
        return min_lr_ratio + (1.0 - min_lr_ratio) * (1.0 - prog)
    if kind == "cosine":
        return min_lr_ratio + (1.0 - min_lr_ratio) * 0.5 * (1.0 + math.cos(math.pi * prog))
    raise ValueError(f"unknown lr scheduler {kind}")


class ShardedAdamW:
    def __init__(self, store: FlatParamStore, cfg, total_steps: int = 1, group=None, optimizer_dtype=torch.float32):
        self.store, self.cfg, self.group = store, cfg, group
        n, dev = store.shard_numel, store.device
        self.bf16_state = cfg.type == "adam_bf16"
        self.offload = bool(getattr(cfg, "offload", False)) and dev.type == "cuda" and not self.bf16_state
        if self.bf16_state:
            # no fp32 master: the bf16 weights plus a bf16 compensation term carry the low-order bits
            self.master = torch.zeros(n, dtype=torch.bfloat16, device=dev)           # Kahan compensation
            self.exp_avg = torch.zeros(n, dtype=torch.bfloat16, device=dev)
            self.exp_avg_sq = torch.zeros(n, dtype=torch.bfloat16, device=dev)
        elif self.offload:
            pin = lambda t: t.pin_memory()
            self.master = pin(store.param_shard.detach().to("cpu", torch.float32))
            self.exp_avg = pin(torch.zeros(n, dtype=torch.float32))
            self.exp_avg_sq = pin(torch.zeros(n, dtype=torch.float32))
            self._chunk = int(getattr(cfg, "offload_chunk_numel", 0) or (1 << 26))
            self._copy_stream = torch.cuda.Stream(device=dev)
            self._bufs = [[torch.empty(min(self._chunk, n), dtype=torch.float32, device=dev) for _ in range(3)] for _ in range(2)]
        else:
            self.master = store.param_shard.detach().to(torch.float32).clone()
            self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev)
            self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev)
        self.state = torch.zeros(4, dtype=torch.float32, device=dev)
        self.step_count = 0
        self.sched_step = 0
        self.total_steps = max(1, total_steps)
        ws = cfg.warmup_steps
        self.warmup_steps = ws if ws is not None else int(math.ceil(cfg.warmup_steps_proportion * self.total_steps))
        self.sgd = cfg.type == "sgd"

    # ------------------------------------------------------------------ lr
    def current_lr(self) -> float:
        return self.cfg.lr * lr_lambda(self.sched_step, self.total_steps, self.warmup_steps,
                                       self.cfg.lr_scheduler_type, self.cfg.min_lr_ratio)

    def lr_scheduler_step(self) -> None:
        self.sched_step += 1

    # ------------------------------------------------------------------ step
    def step(self, grad_shard: torch.Tensor, inv_scale: float = 1.0, norm_already_global: bool = False,
             precomputed_sumsq: Optional[torch.Tensor] = None) -> dict:
        """``grad_shard``: reduced fp32 gradient of this rank's shard. Returns the statistics
        tensor (device): [sumsq, coef, finite, norm]. ``precomputed_sumsq``: global squared norm
        worked out by the caller (tensor parallelism de-duplicates replicated parameters)."""
        st = self.state
        st.zero_()
        if precomputed_sumsq is not None:
            st[0:1].copy_(precomputed_sumsq.to(st.dtype))
        else:
            OF.sqnorm_accumulate_(grad_shard, st)
            if not norm_already_global and self.group is not None and dist.is_initialized() and dist.get_world_size(self.group) > 1:
                dist.all_reduce(st[0:1], group=self.group)
        OF.clip_coef_(st, float(self.cfg.gradient_clipping or 0.0), inv_scale)
        self.step_count += 1
        lr = self.current_lr()
        if self.sgd:
            # p <- p - lr * (coef * g + wd * p), skipped entirely when the norm was not finite (st[2] = 0)
            wd = float(self.cfg.weight_decay or 0.0)
            new = torch.addcmul(self.master * (1.0 - lr * wd) if wd else self.master, grad_shard, st[1], value=-lr)
            self.master.copy_(torch.where(st[2] > 0, new, self.master))      # (0 * nan is nan: select, do not scale)
            self.store.param_shard.copy_(self.master)
        elif self.bf16_state:
            self._step_bf16_state(grad_shard, st, lr)
        elif self.offload:
            self._step_offloaded(grad_shard, st, lr)
        else:
            OF.adamw_step_(self.master, self.exp_avg, self.exp_avg_sq, grad_shard, self.store.param_shard, st, lr,
                           self.cfg.beta1, self.cfg.beta2, self.cfg.eps, self.cfg.weight_decay, self.step_count)
        return {"state": st, "lr": lr}

    @torch.no_grad()
    def _step_bf16_state(self, g: torch.Tensor, st: torch.Tensor, lr: float, chunk: int = 1 << 24) -> None:
        """AdamW with bf16 moments and Kahan-compensated bf16 weights, in chunks so the fp32
        temporaries stay small. Skipped (weights untouched) when the gradient norm was not finite."""
        c = self.cfg
        b1, b2, eps, wd = c.beta1, c.beta2, c.eps, float(c.weight_decay or 0.0)
        bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
        w_all = self.store.param_shard
        ok = st[2]
        for a in range(0, g.numel(), chunk):
            sl = slice(a, min(g.numel(), a + chunk))
            gi = g[sl].float() * st[1]
            m = self.exp_avg[sl].float().mul_(b1).add_(gi, alpha=1 - b1)
            v = self.exp_avg_sq[sl].float().mul_(b2).addcmul_(gi, gi, value=1 - b2)
            w = w_all[sl].float()
            upd = (m / bc1).div_((v / bc2).sqrt_().add_(eps)).mul_(-lr).add_(w, alpha=-lr * wd)
            upd = torch.where(ok > 0, upd, torch.zeros_like(upd))      # no update on a non-finite step (0 * nan is nan: select)
            # Kahan: add the carried low-order bits, round to bf16, keep what the rounding lost
            y = upd.add_(self.master[sl].float())
            new_w = (w + y).to(torch.bfloat16)
            self.master[sl] = (y - (new_w.float() - w)).to(torch.bfloat16)
            w_all[sl] = new_w.to(w_all.dtype)
            keep = ok.to(torch.bool)
            self.exp_avg[sl] = torch.where(keep, m, self.exp_avg[sl].float()).to(torch.bfloat16)
            self.exp_avg_sq[sl] = torch.where(keep, v, self.exp_avg_sq[sl].float()).to(torch.bfloat16)

    @torch.no_grad()
    def _step_offloaded(self, g: torch.Tensor, st: torch.Tensor, lr: float) -> None:
        """Host-resident fp32 state streamed through the device: chunk i + 1 is copied in on a side
        stream while chunk i is updated by the fused kernel and chunk i - 1 is copied out."""
        c, n, ch = self.cfg, g.numel(), self._chunk
        main, side = torch.cuda.current_stream(), self._copy_stream
        host = (self.master, self.exp_avg, self.exp_avg_sq)
        ready = [torch.cuda.Event(), torch.cuda.Event()]
        drained = [None, None]

        def copy_in(i):
            b = i & 1
            a, e = i * ch, min(n, (i + 1) * ch)
            with torch.cuda.stream(side):
                if drained[b] is not None:
                    side.wait_event(drained[b])             # the buffer's previous contents are back on the host
                for buf, h in zip(self._bufs[b], host):
                    buf[:e - a].copy_(h[a:e], non_blocking=True)
                ready[b].record(side)

        n_chunks = (n + ch - 1) // ch
        copy_in(0)
        for i in range(n_chunks):
            b = i & 1
            a, e = i * ch, min(n, (i + 1) * ch)
            if i + 1 < n_chunks:
                copy_in(i + 1)
            main.wait_event(ready[b])
            p32, m, v = (buf[:e - a] for buf in self._bufs[b])
            OF.adamw_step_(p32, m, v, g[a:e], self.store.param_shard[a:e], st, lr, c.beta1, c.beta2, c.eps, c.weight_decay, self.step_count)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(side):
                side.wait_event(done)
                for buf, h in zip(self._bufs[b], host):
                    h[a:e].copy_(buf[:e - a], non_blocking=True)
                drained[b] = torch.cuda.Event()
                drained[b].record(side)
        main.wait_stream(side)

    # ------------------------------------------------------------------ (de)serialisation
    def state_dict(self) -> dict:
        return dict(master=self.master.cpu(), exp_avg=self.exp_avg.cpu(), exp_avg_sq=self.exp_avg_sq.cpu(),
                    step_count=self.step_count, sched_step=self.sched_step, shard_range=self.store.shard_range,
                    world_size=self.store.world_size)

    def load_state_dict(self, sd: dict) -> None:
        if tuple(sd["shard_range"]) != tuple(self.store.shard_range) or sd["world_size"] != self.store.world_size:
            raise ValueError("optimizer state was saved with a different sharding")
        self.master.copy_(sd["master"])
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.step_count, self.sched_step = int(sd["step_count"]), int(sd["sched_step"])

    def resync_master(self) -> None:
        """Re-reads the master copy from the compute weights (after loading a checkpoint)."""
        if self.bf16_state:
            self.master.zero_()                 # the compensation term restarts from the loaded weights
        else:
            self.master.copy_(self.store.param_shard.to(torch.float32))
