"""Context parallelism with the zig-zag layout: every packed sequence is cut into ``2 * cp``
equal chunks and rank ``r`` keeps chunks ``r`` and ``2 * cp - 1 - r``, so causal attention
costs every rank the same. Attention gathers the keys and values of the whole sequence (with
GQA they are a small fraction of the activations and NVSwitch moves them at full bandwidth to
every peer) and runs the local queries against them; the backward pass reduce-scatters dK / dV.

Reference: ``areal/engine/megatron_utils/packed_context_parallel.py`` provides this layout
(split :40-170, differentiable re-assembly of per-token outputs :174-211, output all-gather
:214-270) and leaves the attention itself to TransformerEngine's ring exchange. Here the
attention is part of the framework; on CUDA it currently runs as masked
``scaled_dot_product_attention`` per sequence (the flash kernels take equal query / key
lengths), so Ulysses (``parallel/ulysses.py``) stays the fast sequence-parallel path and this
one serves head counts that Ulysses cannot split.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def padded_lengths(cu_seqlens: torch.Tensor, cp: int) -> list[int]:
    """Per-sequence lengths rounded up to a multiple of ``2 * cp``."""
    cu = cu_seqlens.tolist()
    unit = 2 * cp
    return [-(-(b - a) // unit) * unit for a, b in zip(cu[:-1], cu[1:])]


def zigzag_indices(cu_seqlens: torch.Tensor, cp: int, rank: int) -> tuple[torch.Tensor, torch.Tensor, list[int]]:
    """For rank ``rank``: (``src`` indices into the packed batch, -1 for padding; positions inside
    the sequence of every local token; local lengths per sequence)."""
    cu = cu_seqlens.tolist()
    src, pos, local_lens = [], [], []
    for (a, b), Lp in zip(zip(cu[:-1], cu[1:]), padded_lengths(cu_seqlens, cp)):
        c = Lp // (2 * cp)
        for chunk in (rank, 2 * cp - 1 - rank):
            p = torch.arange(chunk * c, (chunk + 1) * c)
            idx = a + p
            idx[p >= (b - a)] = -1
            src.append(idx)
            pos.append(p)
        local_lens.append(2 * c)
    return torch.cat(src), torch.cat(pos), local_lens


def zigzag_split(x: torch.Tensor, cu_seqlens: torch.Tensor, cp: int, rank: int, pad_value=0) -> torch.Tensor:
    """Local slice ``[T_local, ...]`` of a packed tensor ``[T, ...]`` (padding rows hold ``pad_value``)."""
    src, _, _ = zigzag_indices(cu_seqlens, cp, rank)
    src = src.to(x.device)
    out = x[src.clamp(min=0)]
    if (src < 0).any():
        out = out.masked_fill((src < 0).view(-1, *([1] * (x.dim() - 1))), pad_value)
    return out


class _AllGatherCat(torch.autograd.Function):
    """all-gather along dim 0 (equal shapes); backward = reduce-scatter of the gradient."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = dist.get_world_size(group)
        out = x.new_empty((n * x.shape[0],) + tuple(x.shape[1:]))
        dist.all_gather_into_tensor(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        n = dist.get_world_size(ctx.group)
        g = g.contiguous()
        if dist.get_backend(ctx.group) == "gloo":
            dist.all_reduce(g, group=ctx.group)
            r = dist.get_rank(ctx.group)
            per = g.shape[0] // n
            return g[r * per:(r + 1) * per].clone(), None
        out = g.new_empty((g.shape[0] // n,) + tuple(g.shape[1:]))
        dist.reduce_scatter_tensor(out, g, group=ctx.group)
        return out, None


def gather_sequence(x_local: torch.Tensor, cu_seqlens: torch.Tensor, cp: int, group, keep_padding: bool = False) -> torch.Tensor:
    """Differentiable inverse of :func:`zigzag_split` over the whole group: ``[T_local, ...]`` on
    every rank -> the packed ``[T, ...]`` tensor in the original order on every rank."""
    full = _AllGatherCat.apply(x_local, group) if cp > 1 else x_local          # [cp * T_local, ...], rank-major
    T_local = x_local.shape[0]
    cu = cu_seqlens.tolist()
    T = cu[-1]
    order = torch.full((T,), -1, dtype=torch.long)
    for r in range(cp):
        src, _, _ = zigzag_indices(cu_seqlens, cp, r)
        ok = src >= 0
        order[src[ok]] = (r * T_local + torch.arange(T_local))[ok]
    return full[order.to(full.device)]


def cp_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor, cp: int, rank: int, group,
                 scale: Optional[float] = None) -> torch.Tensor:
    """Causal attention of the local (zig-zag) queries ``[T_local, Hq, D]`` against the whole
    sequences' keys / values, which are gathered from the group. Returns ``[T_local, Hq, D]``."""
    import math

    import torch.nn.functional as F

    Hq, D = q.shape[1], q.shape[2]
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    k_full = gather_sequence(k, cu_seqlens, cp, group)          # [T, Hkv, D] original order
    v_full = gather_sequence(v, cu_seqlens, cp, group)
    _, pos, local_lens = zigzag_indices(cu_seqlens, cp, rank)
    pos = pos.to(q.device)
    cu = cu_seqlens.tolist()
    outs, off = [], 0
    for (a, b), n in zip(zip(cu[:-1], cu[1:]), local_lens):
        qi = q[off:off + n].transpose(0, 1)                      # [Hq, n, D]
        ki = k_full[a:b].transpose(0, 1).repeat_interleave(Hq // Hkv, dim=0)
        vi = v_full[a:b].transpose(0, 1).repeat_interleave(Hq // Hkv, dim=0)
        mask = pos[off:off + n, None] >= torch.arange(b - a, device=q.device)[None, :]
        mask[:, 0] = True                                        # padding queries (beyond the sequence) still need one key
        o = F.scaled_dot_product_attention(qi[None], ki[None], vi[None], attn_mask=mask[None, None], scale=scale)[0]
        outs.append(o.transpose(0, 1))
        off += n
    return torch.cat(outs, 0)
