"""Batch containers and transformations: padded <-> packed layouts, micro-batch splitting by
token budget, page padding, DP redistribution helpers, reward/advantage normalisation and KL
estimators.

Behaviour follows the reference's ``areal/utils/data.py`` (pad_sequences_to_tensors :105,
concat_padded_tensors :241, pack_tensor_dict :496, MicroBatchList :590, split into
micro-batches :700, N_TOKENS_PER_PAGE :819, pad_packed_tensor_dict :822, Normalization
:1382-1637, KLEstimator :1640) with the layouts described there:

* padded batch: dict of ``[B, L]`` tensors with an ``attention_mask``; per-sequence scalars
  are ``[B]``;
* packed batch: dict of ``[T]`` tensors plus ``cu_seqlens [B+1] int32`` and ``max_seqlen``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Callable, Iterable, Optional, Sequence

import torch
import torch.distributed as dist

from . import seqpack

N_TOKENS_PER_PAGE = 256


# --------------------------------------------------------------------------- padded helpers
def pad_sequences_to_tensors(seqs: list[dict[str, Any]], pad_value: float = 0.0) -> dict[str, torch.Tensor]:
    """List of per-sample dicts -> padded ``[B, L]`` batch with ``attention_mask``.

    A value whose length equals the sample's ``input_ids`` length is a per-token field and is
    right-padded; anything else (rewards, ids, ...) is stacked as a per-sequence scalar."""
    if not seqs:
        return {}

    def n_tokens(s):
        v = s["input_ids"]
        return v.numel() if torch.is_tensor(v) else len(v)

    lens = [n_tokens(s) for s in seqs]
    L = max(lens)
    out: dict[str, Any] = {}
    for k in seqs[0].keys():
        vals = [s[k] for s in seqs]
        ts = []
        per_token = True
        for v, n in zip(vals, lens):
            if isinstance(v, (str, bytes, dict)) or v is None:
                per_token = None
                break
            t = v if torch.is_tensor(v) else torch.as_tensor(v)
            t = t.reshape(-1)
            if t.numel() != n or (t.numel() == 1 and k not in ("input_ids", "loss_mask", "logprobs", "versions")):
                per_token = False
            ts.append(t)
        if per_token is None:
            out[k] = vals
        elif per_token:
            out[k] = torch.stack([torch.nn.functional.pad(t, (0, L - t.numel()), value=pad_value) for t in ts])
        elif all(t.numel() == 1 for t in ts):
            out[k] = torch.stack([t.reshape(()) for t in ts])
        else:
            out[k] = vals
    am = torch.zeros(len(seqs), L, dtype=torch.bool)
    for i, n in enumerate(lens):
        am[i, :n] = True
    out["attention_mask"] = am
    return out


def concat_padded_tensors(dicts: list[dict[str, Any]], pad_value: float = 0.0) -> dict[str, Any]:
    """Concatenates padded batches along the batch dim, right-padding to the longest."""
    dicts = [d for d in dicts if d]
    if not dicts:
        return {}
    max_len = max(d["attention_mask"].shape[1] for d in dicts)
    out: dict[str, Any] = {}
    for k in dicts[0].keys():
        vs = []
        for d in dicts:
            v = d[k]
            if torch.is_tensor(v) and v.dim() >= 2 and v.shape[1] == d["attention_mask"].shape[1]:
                pad = max_len - v.shape[1]
                if pad > 0:
                    pv = False if v.dtype == torch.bool else (0 if k == "attention_mask" else pad_value)
                    shape = list(v.shape)
                    shape[1] = pad
                    v = torch.cat([v, torch.full(shape, pv, dtype=v.dtype, device=v.device)], dim=1)
            vs.append(v)
        if torch.is_tensor(vs[0]):
            out[k] = torch.cat(vs, dim=0)
        elif isinstance(vs[0], list):
            out[k] = [x for v in vs for x in v]
        else:
            out[k] = vs
    return out


def batch_size_of(data: dict[str, Any]) -> int:
    if "attention_mask" in data:
        return data["attention_mask"].shape[0]
    if "cu_seqlens" in data:
        return data["cu_seqlens"].numel() - 1
    for v in data.values():
        if torch.is_tensor(v) and v.dim() >= 1:
            return v.shape[0]
    return 0


def select_batch(data: dict[str, Any], idx: Sequence[int]) -> dict[str, Any]:
    """Rows ``idx`` of a padded batch, trimmed to the longest selected sequence."""
    idx_t = torch.as_tensor(list(idx), dtype=torch.long)
    B = batch_size_of(data)
    out = {}
    for k, v in data.items():
        if torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == B:
            out[k] = v[idx_t.to(v.device)]
        elif isinstance(v, list) and len(v) == B:
            out[k] = [v[i] for i in idx]
        else:
            out[k] = v
    if "attention_mask" in out and out["attention_mask"].numel() > 0:
        L = int(out["attention_mask"].sum(1).max().item()) if out["attention_mask"].shape[0] else 0
        full = data["attention_mask"].shape[1]
        for k, v in list(out.items()):
            if torch.is_tensor(v) and v.dim() >= 2 and v.shape[1] == full:
                out[k] = v[:, :L]
    return out


def split_batch(data: dict[str, Any], groups: list[list[int]]) -> list[dict[str, Any]]:
    return [select_batch(data, g) for g in groups]


def concat_batch(batches: list[dict[str, Any]]) -> dict[str, Any]:
    return concat_padded_tensors(batches)


# --------------------------------------------------------------------------- packing
def pack_tensor_dict(data: dict[str, Any]) -> dict[str, Any]:
    """Padded ``[B, L]`` batch -> packed 1-D batch with ``cu_seqlens`` / ``max_seqlen``."""
    am = data["attention_mask"].bool()
    B, L = am.shape
    lens = am.sum(1).to(torch.int32)
    cu = torch.zeros(B + 1, dtype=torch.int32, device=am.device)
    cu[1:] = torch.cumsum(lens, 0)
    out: dict[str, Any] = {}
    for k, v in data.items():
        if k == "attention_mask":
            continue
        if torch.is_tensor(v) and v.dim() >= 2 and v.shape[:2] == (B, L):
            out[k] = v[am]
        else:
            out[k] = v
    out["cu_seqlens"] = cu
    out["max_seqlen"] = int(lens.max().item()) if B else 0
    return out


def unpack_sequence(x: torch.Tensor, cu_seqlens: torch.Tensor) -> list[torch.Tensor]:
    cu = cu_seqlens.tolist()
    return [x[cu[i]:cu[i + 1]] for i in range(len(cu) - 1)]


def positions_from_cu_seqlens(cu_seqlens: torch.Tensor, total: Optional[int] = None) -> torch.Tensor:
    """position_ids of a packed batch (restart at 0 for every sequence); sync-free."""
    T = int(cu_seqlens[-1].item()) if total is None else total
    idx = torch.arange(T, device=cu_seqlens.device, dtype=torch.int64)
    seq = torch.searchsorted(cu_seqlens.to(torch.int64), idx, right=True) - 1
    seq = seq.clamp(min=0, max=cu_seqlens.numel() - 2)
    return (idx - cu_seqlens.to(torch.int64)[seq]).to(torch.int32)


def amend_position_ids(data: dict[str, Any]) -> dict[str, Any]:
    if "position_ids" in data:
        return data
    if "attention_mask" in data:
        am = data["attention_mask"].long()
        data["position_ids"] = (torch.cumsum(am, 1) - 1).clamp(min=0)
    elif "cu_seqlens" in data:
        data["position_ids"] = positions_from_cu_seqlens(data["cu_seqlens"])
    return data


@dataclass
class MicroBatchList:
    """Packed micro-batches of one batch plus the permutations that restore the order."""

    data: dict[str, Any]
    mbs: list[dict[str, Any]]
    groups: list[list[int]]                 # sample indices of each micro-batch
    forward_indices: list[int]              # concatenation order of the samples
    backward_indices: list[int]             # inverse permutation
    group_lens: list[int]                   # tokens per micro-batch (before padding)
    padded_mbs: Optional[list[dict[str, Any]]] = None
    padding_lengths: Optional[list[int]] = None
    old_cu_seqlens_list: Optional[list[torch.Tensor]] = None

    def __len__(self):
        return len(self.mbs)

    def to(self, device):
        def mv(d):
            return {k: (v.to(device, non_blocking=True) if torch.is_tensor(v) else v) for k, v in d.items()}

        self.mbs = [mv(m) for m in self.mbs]
        if self.padded_mbs is not None:
            self.padded_mbs = [mv(m) for m in self.padded_mbs]
        return self


def allocate_balanced_mbs(seqlens: Sequence[int], mb_spec, group: Optional[dist.ProcessGroup] = None) -> list[list[int]]:
    """Groups of sample indices per micro-batch under ``mb_spec``. With a process group the
    number of micro-batches is equalised across ranks (max over ranks)."""
    cap = mb_spec.max_tokens_per_mb or int(1e12)
    n_min = max(1, mb_spec.n_mbs or 1)
    div = max(1, mb_spec.n_mbs_divisor)
    alloc = seqpack.get_allocate_fn(mb_spec.packing_algorithm)

    def run(nmin):
        groups = alloc(list(seqlens), cap, nmin)
        while len(groups) % div != 0 and len(groups) < len(seqlens):
            groups = alloc(list(seqlens), cap, len(groups) + 1)
        return groups

    groups = run(n_min)
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        counts = [None] * dist.get_world_size(group)
        dist.all_gather_object(counts, len(groups), group=group)
        target = max(counts)
        if target > len(groups):
            groups = run(target)
            while len(groups) < target:  # not enough sequences: add empty micro-batches
                groups.append([])
    return groups


def split_padded_tensor_dict_into_mb_list(data: dict[str, Any], mb_spec, group: Optional[dist.ProcessGroup] = None
                                          ) -> MicroBatchList:
    """Splits a padded batch into packed micro-batches under the token budget of ``mb_spec``."""
    am = data["attention_mask"]
    lens = am.sum(1).tolist()
    groups = allocate_balanced_mbs(lens, mb_spec, group)
    fwd = [i for g in groups for i in g]
    bwd = [0] * len(fwd)
    for pos, i in enumerate(fwd):
        bwd[i] = pos
    mbs = []
    for g in groups:
        if g:
            mbs.append(pack_tensor_dict(select_batch(data, g)))
        else:
            mbs.append(_empty_packed_like(data))
    return MicroBatchList(data=data, mbs=mbs, groups=groups, forward_indices=fwd, backward_indices=bwd,
                          group_lens=[int(sum(lens[i] for i in g)) for g in groups])


def _empty_packed_like(data):
    out = {}
    B, L = data["attention_mask"].shape
    for k, v in data.items():
        if k == "attention_mask":
            continue
        if torch.is_tensor(v) and v.dim() >= 2 and v.shape[:2] == (B, L):
            out[k] = v.new_zeros((0,) + tuple(v.shape[2:]))
        elif torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == B:
            out[k] = v.new_zeros((0,) + tuple(v.shape[1:]))
        else:
            out[k] = v
    out["cu_seqlens"] = torch.zeros(1, dtype=torch.int32, device=data["attention_mask"].device)
    out["max_seqlen"] = 0
    return out


def pad_packed_tensor_dict(mb: dict[str, Any], pad_to: Optional[int] = None, align: int = N_TOKENS_PER_PAGE,
                           pad_value: float = 0.0) -> tuple[dict[str, Any], int, torch.Tensor]:
    """Appends one fake sequence so the token count becomes a multiple of ``align`` (or
    exactly ``pad_to``). Returns (padded mb, pad length, original cu_seqlens)."""
    cu = mb["cu_seqlens"]
    T = int(cu[-1].item())
    target = pad_to if pad_to is not None else max(align, -(-T // align) * align)
    pad = target - T
    if pad < 0:
        raise ValueError(f"cannot pad {T} tokens down to {target}")
    if pad == 0:
        return mb, 0, cu
    out = {}
    for k, v in mb.items():
        if k in ("cu_seqlens", "max_seqlen"):
            continue
        if torch.is_tensor(v) and v.dim() >= 1 and v.shape[0] == T:
            if k == "position_ids":
                filler = torch.arange(pad, dtype=v.dtype, device=v.device)
            else:
                filler = torch.full((pad,) + tuple(v.shape[1:]), 0 if v.dtype in (torch.bool,) else pad_value,
                                    dtype=v.dtype, device=v.device)
            out[k] = torch.cat([v, filler], dim=0)
        else:
            out[k] = v
    out["cu_seqlens"] = torch.cat([cu, torch.tensor([target], dtype=cu.dtype, device=cu.device)])
    out["max_seqlen"] = max(int(mb.get("max_seqlen", 0)), pad)
    return out, pad, cu


def pad_mb_list(mbl: MicroBatchList, pad_to_maximum: bool = False, max_tokens: Optional[int] = None,
                align: int = N_TOKENS_PER_PAGE) -> MicroBatchList:
    padded, pads, olds = [], [], []
    for mb in mbl.mbs:
        target = None
        if pad_to_maximum and max_tokens:
            target = -(-max_tokens // align) * align
        p, n, old = pad_packed_tensor_dict(mb, pad_to=target, align=align)
        padded.append(p)
        pads.append(n)
        olds.append(old)
    mbl.padded_mbs, mbl.padding_lengths, mbl.old_cu_seqlens_list = padded, pads, olds
    return mbl


def unpad_logits(x: torch.Tensor, pad_len: int) -> torch.Tensor:
    return x[: x.shape[0] - pad_len] if pad_len > 0 else x


def reorder_list(xs: list, indices: list[int]) -> list:
    return [xs[i] for i in indices]


def unpack_to_padded(flat: torch.Tensor, lens: Sequence[int], max_len: Optional[int] = None,
                     pad_value: float = 0.0) -> torch.Tensor:
    """Packed ``[T, ...]`` -> padded ``[B, L, ...]``."""
    B = len(lens)
    L = max_len or (max(lens) if lens else 0)
    out = flat.new_full((B, L) + tuple(flat.shape[1:]), pad_value)
    off = 0
    for i, n in enumerate(lens):
        out[i, :n] = flat[off:off + n]
        off += n
    return out


# --------------------------------------------------------------------------- distributed helpers
def broadcast_tensor_container(obj, src: int = 0, group=None, device=None):
    """Broadcasts a nested container of tensors / python objects from ``src``."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return obj
    box = [obj if dist.get_rank() == src else None]
    if dist.get_rank() == src:
        box = [_to_cpu(obj)]
    dist.broadcast_object_list(box, src=src, group=group)
    res = box[0]
    return _to_device(res, device) if device is not None else res


def all_gather_tensor_container(obj, group=None) -> list:
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return [obj]
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, _to_cpu(obj), group=group)
    return out


def _to_cpu(o):
    if torch.is_tensor(o):
        return o.detach().cpu()
    if isinstance(o, dict):
        return {k: _to_cpu(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return type(o)(_to_cpu(v) for v in o)
    return o


def _to_device(o, device):
    if torch.is_tensor(o):
        return o.to(device)
    if isinstance(o, dict):
        return {k: _to_device(v, device) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return type(o)(_to_device(v, device) for v in o)
    return o


def tensor_container_to(o, device):
    return _to_device(o, device)


def cycle_dataloader(dataloader: Iterable, num_cycles: Optional[int] = None):
    """Endless (or ``num_cycles``) iteration; calls ``sampler.set_epoch`` when present."""
    epoch = 0
    while num_cycles is None or epoch < num_cycles:
        sampler = getattr(dataloader, "sampler", None)
        if sampler is not None and hasattr(sampler, "set_epoch"):
            sampler.set_epoch(epoch)
        for item in dataloader:
            yield item
        epoch += 1


# --------------------------------------------------------------------------- normalisation
class Normalization:
    """``(x - mean) * mask / (std + eps)`` with mean/std taken over the whole (DP-global)
    batch, per prompt group, or not at all; leave-one-out mean (RLOO) optional. Sums are
    all-reduced in fp64 over ``reduce_group`` for the batch level."""

    def __init__(self, config):
        self.mean_level = config.mean_level if config.mean_level not in (None, "none") else None
        self.std_level = config.std_level if config.std_level not in (None, "none") else None
        self.mean_leave1out = config.mean_leave1out
        self.std_unbiased = config.std_unbiased
        self.eps = config.eps if self.std_level is not None else 0.0
        self.group_size = config.group_size

    def __call__(self, x: torch.Tensor, loss_mask: Optional[torch.Tensor] = None, group_sizes: Optional[list[int]] = None,
                 high_precision: bool = True, reduce_group=None) -> torch.Tensor:
        dtype = torch.float64 if high_precision else torch.float32
        xf = x.to(dtype)
        mask = torch.ones_like(xf) if loss_mask is None else loss_mask.to(dtype)
        B = x.shape[0]
        if group_sizes is None:
            gs = max(1, self.group_size)
            group_sizes = [gs] * (B // gs) + ([B % gs] if B % gs else [])
        # ---- mean
        if self.mean_level == "batch":
            mean = self._batch_mean(xf, mask, reduce_group).expand_as(xf)
        elif self.mean_level == "group":
            mean = torch.zeros_like(xf)
            off = 0
            for g in group_sizes:
                sl = slice(off, off + g)
                mean[sl] = self._local_mean(xf[sl], mask[sl], self.mean_leave1out)
                off += g
        else:
            mean = torch.zeros_like(xf)
        centered = xf - mean
        # ---- std
        if self.std_level == "batch":
            std = self._batch_std(xf, mask, mean, reduce_group).expand_as(xf)
        elif self.std_level == "group":
            std = torch.ones_like(xf)
            off = 0
            for g in group_sizes:
                sl = slice(off, off + g)
                std[sl] = self._local_std(xf[sl], mask[sl], mean[sl])
                off += g
        else:
            std = torch.ones_like(xf)
        out = centered * mask / (std + self.eps)
        return out.to(torch.float32)

    @staticmethod
    def _local_mean(x, mask, leave1out):
        n = mask.sum()
        s = (x * mask).sum()
        if leave1out:
            denom = (n - mask).clamp(min=1.0)
            return (s - x * mask) / denom
        return (s / n.clamp(min=1.0)).expand_as(x)

    def _local_std(self, x, mask, mean):
        n = mask.sum()
        var_sum = (((x - mean) ** 2) * mask).sum()
        denom = n - 1 if self.std_unbiased else n
        if float(n) <= 1 or float(denom) <= 0:
            return torch.ones_like(x)
        return torch.sqrt(var_sum / denom).expand_as(x)

    @staticmethod
    def _reduce(t, group):
        if dist.is_initialized() and (group is not None or dist.get_world_size() > 1):
            try:
                dist.all_reduce(t, group=group)
            except Exception:
                pass
        return t

    def _batch_mean(self, x, mask, group):
        stats = torch.stack([mask.sum(), (x * mask).sum()])
        stats = self._reduce(stats, group)
        if self.mean_leave1out:
            n, s = stats[0], stats[1]
            return (s - x * mask) / (n - mask).clamp(min=1.0)
        return (stats[1] / stats[0].clamp(min=1.0)).reshape(*([1] * x.dim()))

    def _batch_std(self, x, mask, mean, group):
        stats = torch.stack([mask.sum(), (((x - mean) ** 2) * mask).sum()])
        stats = self._reduce(stats, group)
        n = stats[0]
        denom = n - 1 if self.std_unbiased else n
        if float(n) <= 1 or float(denom) <= 0:
            return torch.ones([1] * x.dim(), dtype=x.dtype, device=x.device)
        return torch.sqrt(stats[1] / denom).reshape(*([1] * x.dim()))


class KLEstimator:
    """k1 / k2 / k3 estimators of KL(pi || pi_base) from per-token log-probs
    (d = logp - logp_base): k1 = d, k2 = d^2/2, k3 = exp(-d) - 1 + d; clamped to +-10."""

    def __init__(self, kind: str = "k1", apply_clamp: bool = True):
        if kind not in ("k1", "k2", "k3"):
            raise ValueError(f"unknown KL estimator {kind}")
        self.kind, self.apply_clamp = kind, apply_clamp

    def __call__(self, logp: torch.Tensor, logp_base: torch.Tensor) -> torch.Tensor:
        d = logp.float() - logp_base.float()
        if self.kind == "k1":
            kl = d
        elif self.kind == "k2":
            kl = 0.5 * d * d
        else:
            nd = -d
            kl = torch.exp(nd) - 1 - nd
        return kl.clamp(-10.0, 10.0) if self.apply_clamp else kl
