"""Delta weight transfer: after a small-learning-rate step most bf16 parameters keep their
bit pattern, so only the blocks that changed need to travel to the rollout replicas.

* :func:`changed_blocks` compares the new flat parameter buffer against the snapshot of what
  the receivers hold (exact detection);
* :func:`predict_changed_blocks` decides from the optimizer state alone, without a snapshot:
  a bf16 value can only change if the fp32 master moved by at least half a bf16 ulp, and the
  AdamW update is reconstructed from ``exp_avg / (sqrt(exp_avg_sq) + eps)`` (a conservative
  superset of the exact set);
* :class:`DeltaPusher` wraps a copy function and sends only changed blocks.

Reference: ``areal/v2/weight_update/awex/delta_detect.py`` (AdamW-inversion change detection),
``delta_config.py``, ``areal/utils/dte.py``."""
from __future__ import annotations

from typing import Callable, Optional

import torch


def changed_blocks(new_flat: torch.Tensor, old_flat: torch.Tensor, block: int = 4096) -> torch.Tensor:
    """bool [ceil(n / block)]: True where any element of the block differs bitwise."""
    n = new_flat.numel()
    assert old_flat.numel() == n and new_flat.dtype == old_flat.dtype
    full = n // block * block
    view = {2: torch.int16, 4: torch.int32, 1: torch.int8}[new_flat.element_size()]
    a, b = new_flat.view(view), old_flat.view(view)
    mask = (a[:full].view(-1, block) != b[:full].view(-1, block)).any(dim=1)
    if full < n:
        mask = torch.cat([mask, (a[full:] != b[full:]).any().reshape(1)])
    return mask


def predict_changed_blocks(master: torch.Tensor, exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, lr: float, beta1: float, beta2: float,
                           eps: float, weight_decay: float, step: int, block: int = 4096, safety: float = 1.0) -> torch.Tensor:
    """Blocks whose bf16 image MAY have changed in the step that produced ``master``. The step
    that was applied is ``lr * (m_hat / (sqrt(v_hat) + eps) + wd * p)``; an element is flagged
    when that step is at least ``0.5 * ulp_bf16(p) / safety`` or the master sits closer to a
    rounding boundary than the step."""
    bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
    upd = lr * ((exp_avg / bc1) / ((exp_avg_sq / bc2).sqrt() + eps) + weight_decay * master)
    # bf16 keeps 8 significant bits: ulp = 2^(floor(log2 |p|) - 7)
    mag = master.abs().clamp(min=1e-38)
    ulp = torch.exp2(torch.floor(torch.log2(mag)) - 7)
    bf = master.to(torch.bfloat16).float()
    dist_to_boundary = (0.5 * ulp - (master - bf).abs()).clamp(min=0)
    may = upd.abs() * safety >= dist_to_boundary
    n = master.numel()
    full = n // block * block
    mask = may[:full].view(-1, block).any(dim=1)
    if full < n:
        mask = torch.cat([mask, may[full:].any().reshape(1)])
    return mask


class DeltaPusher:
    """Sends only the blocks that changed since the last push.

    ``copy_fn(offset, length)`` moves ``flat[offset:offset+length]`` to the receivers. Adjacent
    changed blocks are merged into one copy. ``full_every``: force a full push periodically
    (guards receivers against drift if a push was lost)."""

    def __init__(self, flat: torch.Tensor, copy_fn: Callable[[int, int], None], block: int = 4096, full_every: int = 0):
        self.flat, self.copy_fn, self.block, self.full_every = flat, copy_fn, block, full_every
        self.snapshot: Optional[torch.Tensor] = None
        self.pushes = 0
        self.last_fraction = 1.0

    @torch.no_grad()
    def push(self) -> float:
        """Returns the fraction of bytes sent."""
        n = self.flat.numel()
        self.pushes += 1
        if self.snapshot is None or (self.full_every and self.pushes % self.full_every == 0):
            self.copy_fn(0, n)
            self.snapshot = self.flat.detach().clone()
            self.last_fraction = 1.0
            return 1.0
        mask = changed_blocks(self.flat, self.snapshot, self.block)
        idx = torch.nonzero(mask).flatten().tolist()
        sent = 0
        run_start = prev = None
        for b in idx + [None]:
            if run_start is None:
                run_start = prev = b
                continue
            if b is not None and b == prev + 1:
                prev = b
                continue
            off = run_start * self.block
            ln = min(n, (prev + 1) * self.block) - off
            self.copy_fn(off, ln)
            self.snapshot[off:off + ln].copy_(self.flat[off:off + ln])
            sent += ln
            run_start = prev = b
        self.last_fraction = sent / max(1, n)
        return self.last_fraction
