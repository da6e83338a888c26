"""Ulysses sequence parallelism: activations are sharded along the sequence everywhere except
inside attention, where an all-to-all turns the layout into "all tokens, a slice of heads".

Per layer forward: q, k, v ``[T/n, h, D] -> [T, h/n, D]`` (3 all-to-all), attention over the
full packed batch, output ``[T, hq/n, D] -> [T/n, hq, D]`` (1 all-to-all); autograd runs the
inverse exchanges. KV heads are replicated when ``n_kv_heads < n``. Same data movement as the
reference's ``areal/models/fsdp/ulysses.py:153-190`` and
``areal/models/transformers/ulyssess_patch.py:39-78``; here the exchange is expressed on the
packed token dimension so no padding per sequence is needed (the engine pads the packed
length to a multiple of ``n``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _a2a(x: torch.Tensor, group) -> torch.Tensor:
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x.contiguous(), group=group)
    return out


class SeqToHead(torch.autograd.Function):
    """[t, h, D] (local tokens, all heads) -> [n*t, h/n, D] (all tokens, local heads)."""

    @staticmethod
    def forward(ctx, x, group, n):
        ctx.group, ctx.n = group, n
        t, h, D = x.shape
        xs = x.reshape(t, n, h // n, D).permute(1, 0, 2, 3).contiguous()   # [n(dst), t, h/n, D]
        out = _a2a(xs, group)                                               # [n(src), t, h/n, D]
        return out.reshape(n * t, h // n, D)

    @staticmethod
    def backward(ctx, g):
        n = ctx.n
        T, hl, D = g.shape
        t = T // n
        gs = _a2a(g.reshape(n, t, hl, D).contiguous(), ctx.group)           # [n(head group), t, hl, D]
        return gs.permute(1, 0, 2, 3).reshape(t, n * hl, D), None, None


class HeadToSeq(torch.autograd.Function):
    """[n*t, h/n, D] -> [t, h, D]: inverse of :class:`SeqToHead`."""

    @staticmethod
    def forward(ctx, x, group, n):
        ctx.group, ctx.n = group, n
        T, hl, D = x.shape
        t = T // n
        out = _a2a(x.reshape(n, t, hl, D).contiguous(), group)
        return out.permute(1, 0, 2, 3).reshape(t, n * hl, D)

    @staticmethod
    def backward(ctx, g):
        n = ctx.n
        t, h, D = g.shape
        gs = g.reshape(t, n, h // n, D).permute(1, 0, 2, 3).contiguous()
        return _a2a(gs, ctx.group).reshape(n * t, h // n, D), None, None


def install_ulysses(model, group, sp_size: int, sp_rank: int) -> None:
    """Marks every attention module of ``model`` as sequence-parallel."""
    nq, nkv = model.cfg.num_heads, model.cfg.num_kv_heads
    if nq % sp_size != 0:
        raise ValueError(f"sequence-parallel degree {sp_size} must divide the number of query heads {nq}")
    for layer in model.layers:
        a = layer.self_attn
        a.sp_group, a.sp_size, a.sp_rank = group, sp_size, sp_rank


def ulysses_attention(attn_module, q, k, v, full_cu_seqlens, causal, scale, tile_info, attention_fn):
    """q/k/v: local slices ``[T/n, heads, D]``; returns the local slice of the output."""
    n, group = attn_module.sp_size, attn_module.sp_group
    nkv = k.shape[1]
    if nkv < n:
        rep = n // nkv
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
    elif nkv % n:
        raise ValueError("number of KV heads must divide or be divisible by the sequence-parallel degree")
    qf = SeqToHead.apply(q, group, n)
    kf = SeqToHead.apply(k.contiguous(), group, n)
    vf = SeqToHead.apply(v.contiguous(), group, n)
    o = attention_fn(qf, kf, vf, full_cu_seqlens, causal, scale, tile_info)
    return HeadToSeq.apply(o, group, n)
