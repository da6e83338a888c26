"""Context parallelism with the zig-zag layout: every packed sequence is cut into ``2 * cp``
equal chunks and rank ``r`` keeps chunks ``r`` and ``2 * cp - 1 - r``, so causal attention
costs every rank the same. Attention gathers the keys and values of the whole sequence (with
GQA they are a small fraction of the activations and NVSwitch moves them at full bandwidth to
every peer) and runs the local queries against them; the backward pass reduce-scatters dK / dV.

Reference: ``areal/engine/megatron_utils/packed_context_parallel.py`` provides this layout
(split :40-170, differentiable re-assembly of per-token outputs :174-211, output all-gather
:214-270) and leaves the attention itself to TransformerEngine's ring exchange. Here the
attention is part of the framework and runs on the flash kernels chunk against chunk: with the
zig-zag layout every (query chunk, key chunk) pair is either fully visible, causal (the same
chunk) or invisible, and all chunks of a sequence have one length, so each visible pair is one
call of the varlen kernel (non-causal or causal) over the chunk-packed layout, and the partial
results are merged through their log-sum-exp. Every rank runs the local causal call plus two
full calls per peer, the same work everywhere. The backward pass replays the pairs with the
merged log-sum-exp (the standard blockwise flash backward) and reduce-scatters dK / dV.
A ring of point-to-point exchanges, as link-limited fabrics want it, buys nothing behind an
NVSwitch: one all-gather moves every rank's keys and values at full bandwidth, and with GQA
they are a small fraction of the activations.
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


def _chunk_indices(local_lens: list[int], device):
    """Index tensors that pick the first / second chunk of every sequence out of the local layout
    ``[seq0: lo, hi | seq1: lo, hi | ...]`` and the cu_seqlens of the chunk-packed layout."""
    lo, hi, cu, off = [], [], [0], 0
    for n in local_lens:
        c = n // 2
        lo.append(torch.arange(off, off + c))
        hi.append(torch.arange(off + c, off + n))
        cu.append(cu[-1] + c)
        off += n
    return (torch.cat(lo).to(device), torch.cat(hi).to(device), torch.tensor(cu, dtype=torch.int32, device=device))


def _block_fwd(q, k, v, cu, causal: bool, scale: float):
    """(o, lse [Hq, T]) of one (query chunk set, key chunk set) pair; the flash kernel on CUDA, the same
    math in the tensors' own precision elsewhere."""
    if q.is_cuda:
        from ..ops import functional as OF

        return OF.attention_fwd(q.contiguous(), k.contiguous(), v.contiguous(), cu, causal, scale)
    T, Hq, D = q.shape
    rep = Hq // k.shape[1]
    o = torch.zeros_like(q)
    lse = q.new_zeros(Hq, T)
    b = cu.tolist()
    for a, e in zip(b[:-1], b[1:]):
        if e <= a:
            continue
        s = torch.einsum("qhd,khd->hqk", q[a:e], k[a:e].repeat_interleave(rep, 1)) * scale
        if causal:
            s = s.masked_fill(~torch.ones(e - a, e - a, dtype=torch.bool, device=q.device).tril(), float("-inf"))
        lse[:, a:e] = torch.logsumexp(s, -1)
        o[a:e] = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v[a:e].repeat_interleave(rep, 1))
    return o, lse


def _block_bwd(q, k, v, o, lse, do, cu, causal: bool, scale: float):
    """(dq, dk, dv) of one pair given the MERGED output and log-sum-exp of the query rows."""
    if q.is_cuda:
        from ..ops import functional as OF

        return OF.attention_bwd(q.contiguous(), k.contiguous(), v.contiguous(), o.contiguous(), lse.contiguous(), do.contiguous(),
                                cu, causal, scale)
    Hq, Hkv, D = q.shape[1], k.shape[1], q.shape[2]
    rep = Hq // Hkv
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    b = cu.tolist()
    for a, e in zip(b[:-1], b[1:]):
        if e <= a:
            continue
        L = e - a
        kr, vr = k[a:e].repeat_interleave(rep, 1), v[a:e].repeat_interleave(rep, 1)
        s = torch.einsum("qhd,khd->hqk", q[a:e], kr) * scale
        if causal:
            s = s.masked_fill(~torch.ones(L, L, dtype=torch.bool, device=q.device).tril(), float("-inf"))
        p = torch.exp(s - lse[:, a:e].unsqueeze(-1))
        dp = torch.einsum("qhd,khd->hqk", do[a:e], vr)
        delta = (do[a:e] * o[a:e]).sum(-1).transpose(0, 1).unsqueeze(-1)
        ds = p * (dp - delta) * scale
        dq[a:e] = torch.einsum("hqk,khd->qhd", ds, kr)
        dk[a:e] = torch.einsum("hqk,qhd->khd", ds, q[a:e]).reshape(L, Hkv, rep, D).sum(2)
        dv[a:e] = torch.einsum("hqk,qhd->khd", p, do[a:e]).reshape(L, Hkv, rep, D).sum(2)
    return dq, dk, dv


def _merge(o, lse, o_b, lse_b):
    """Adds a partial attention result into the running one (fp32 / input precision accumulators)."""
    new = torch.logaddexp(lse, lse_b)
    w0 = torch.exp(lse - new).transpose(0, 1).unsqueeze(-1)
    w1 = torch.exp(lse_b - new).transpose(0, 1).unsqueeze(-1)
    return o * w0 + o_b.to(o.dtype) * w1, new


def _pairs(rank: int, peer: int):
    """Visible (query chunk, key chunk) pairs between this rank's queries and ``peer``'s keys as
    ((0 = lo | 1 = hi) query, key) tuples; a peer below sees its lo keys from both query chunks, a peer
    above shows both its chunks to the hi queries."""
    if peer < rank:
        return [(0, 0), (1, 0)]
    if peer > rank:
        return [(1, 0), (1, 1)]
    return []


def cp_block_forward(q, k_all, v_all, local_lens: list[int], rank: int, scale: float):
    """Attention of the local queries ``[T_local, Hq, D]`` against the keys / values of all ranks
    ``[cp, T_local, Hkv, D]`` (every rank in its own zig-zag layout). Returns (o, lse [Hq, T_local])."""
    cp = k_all.shape[0]
    acc_dtype = torch.float32 if q.dtype in (torch.bfloat16, torch.float16) else q.dtype
    lo, hi, cu_c = _chunk_indices(local_lens, q.device)
    cu_l = torch.tensor([0] + list(torch.tensor(local_lens).cumsum(0)), dtype=torch.int32, device=q.device)
    o, lse = _block_fwd(q, k_all[rank], v_all[rank], cu_l, True, scale)          # lo x lo causal, hi x lo full, hi x hi causal
    o, lse = o.to(acc_dtype), lse.to(acc_dtype)
    sel = (lo, hi)
    for peer in range(cp):
        for qc, kc in _pairs(rank, peer):
            qi, ki = sel[qc], sel[kc]
            ob, lb = _block_fwd(q.index_select(0, qi), k_all[peer].index_select(0, ki), v_all[peer].index_select(0, ki), cu_c, False, scale)
            om, lm = _merge(o.index_select(0, qi), lse.index_select(1, qi), ob, lb.to(acc_dtype))
            o = o.index_copy(0, qi, om)
            lse = lse.index_copy(1, qi, lm)
    return o.to(q.dtype), lse


def cp_block_backward(q, k_all, v_all, o, lse, do, local_lens: list[int], rank: int, scale: float):
    """Gradients of :func:`cp_block_forward`: dq ``[T_local, Hq, D]`` and the contributions of this rank's
    queries to every rank's keys / values ``[cp, T_local, Hkv, D]`` (to be summed over ranks)."""
    cp = k_all.shape[0]
    lo, hi, cu_c = _chunk_indices(local_lens, q.device)
    cu_l = torch.tensor([0] + list(torch.tensor(local_lens).cumsum(0)), dtype=torch.int32, device=q.device)
    acc_dtype = torch.float32 if q.dtype in (torch.bfloat16, torch.float16) else q.dtype
    lse_k = lse.float() if q.is_cuda else lse.to(q.dtype)
    dq, dk, dv = _block_bwd(q, k_all[rank], v_all[rank], o, lse_k, do, cu_l, True, scale)
    dq = dq.to(acc_dtype)
    dk_all = torch.zeros(k_all.shape, dtype=acc_dtype, device=q.device)
    dv_all = torch.zeros(v_all.shape, dtype=acc_dtype, device=q.device)
    dk_all[rank] += dk
    dv_all[rank] += dv
    sel = (lo, hi)
    for peer in range(cp):
        for qc, kc in _pairs(rank, peer):
            qi, ki = sel[qc], sel[kc]
            dqb, dkb, dvb = _block_bwd(q.index_select(0, qi), k_all[peer].index_select(0, ki), v_all[peer].index_select(0, ki),
                                       o.index_select(0, qi), lse_k.index_select(1, qi), do.index_select(0, qi), cu_c, False, scale)
            dq.index_add_(0, qi, dqb.to(acc_dtype))
            dk_all[peer].index_add_(0, ki, dkb.to(acc_dtype))
            dv_all[peer].index_add_(0, ki, dvb.to(acc_dtype))
    return dq.to(q.dtype), dk_all, dv_all


class _CPAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, local_lens, cp, rank, group, scale):
        if cp > 1:
            k_all = k.new_empty((cp,) + tuple(k.shape))
            v_all = v.new_empty((cp,) + tuple(v.shape))
            dist.all_gather_into_tensor(k_all.view((-1,) + tuple(k.shape[1:])), k.contiguous(), group=group)
            dist.all_gather_into_tensor(v_all.view((-1,) + tuple(v.shape[1:])), v.contiguous(), group=group)
        else:
            k_all, v_all = k.unsqueeze(0), v.unsqueeze(0)
        o, lse = cp_block_forward(q, k_all, v_all, local_lens, rank, scale)
        ctx.save_for_backward(q, k_all, v_all, o, lse)
        ctx.meta = (local_lens, cp, rank, group, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k_all, v_all, o, lse = ctx.saved_tensors
        local_lens, cp, rank, group, scale = ctx.meta
        dq, dk_all, dv_all = cp_block_backward(q, k_all, v_all, o, lse, do.contiguous(), local_lens, rank, scale)
        if cp > 1:
            if dist.get_backend(group) == "gloo":
                dist.all_reduce(dk_all, group=group)
                dist.all_reduce(dv_all, group=group)
                dk, dv = dk_all[rank], dv_all[rank]
            else:
                dk, dv = torch.empty_like(dk_all[0]), torch.empty_like(dv_all[0])
                dist.reduce_scatter_tensor(dk, dk_all.view((-1,) + tuple(dk.shape[1:])), group=group)
                dist.reduce_scatter_tensor(dv, dv_all.view((-1,) + tuple(dv.shape[1:])), group=group)
        else:
            dk, dv = dk_all[0], dv_all[0]
        return dq, dk.to(k_all.dtype), dv.to(v_all.dtype), None, None, None, None, None


def cp_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor, cp: int, rank: int, group,
                 scale: Optional[float] = None) -> torch.Tensor:
    """Causal attention of the local (zig-zag) queries ``[T_local, Hq, D]`` against the whole
    sequences' keys / values (gathered from the group), chunk pair by chunk pair on the flash kernels.
    Returns ``[T_local, Hq, D]``; differentiable in q, k and v."""
    import math

    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[2])
    _, _, local_lens = zigzag_indices(cu_seqlens, cp, rank)
    return _CPAttention.apply(q, k, v, local_lens, cp, rank, group, scale)
